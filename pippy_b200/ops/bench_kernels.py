"""Micro-benchmarks of the package's kernels, timed with CUDA events (3 warm-ups, 10 timed launches).

    python -m pippy_b200.ops.bench_kernels gemm
    python -m pippy_b200.ops.bench_kernels attention
    python -m pippy_b200.ops.bench_kernels attention-once     # two forward+backward calls on a small case, for ncu
    python -m pippy_b200.ops.bench_kernels gemm-once          # three launches of one GEMM, for ncu
    python -m pippy_b200.ops.bench_kernels grouped            # grouped expert GEMMs vs a loop of plain GEMMs / cuBLAS
    python -m pippy_b200.ops.bench_kernels grouped-once       # three grouped launches on a small case, for ncu
    python -m pippy_b200.ops.bench_kernels route              # MoE router kernels vs the eager statement
    python -m pippy_b200.ops.bench_kernels elementwise        # RMSNorm, SwiGLU, attention delta on one 7B microbatch
    python -m pippy_b200.ops.bench_kernels elementwise-once   # one launch of each of them, for ncu
    python -m torch.distributed.run --nproc-per-node 2 -m pippy_b200.ops.bench_kernels tp | dp | moe | peer-copy

Library rates (cuBLAS via torch.matmul, SDPA) are printed beside ours for scale.
"""
from __future__ import annotations

import math
import sys

import torch


def _time(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def bench_gemm():
    from .gemm import gemm

    shapes = [  # (M, N, K, a_mn, b_mn, what)
        (8192, 8192, 8192, 0, 0, "square"),
        (8192, 12288, 4096, 0, 0, "llama7b qkv fwd"),
        (8192, 22016, 4096, 0, 0, "llama7b gate/up fwd"),
        (8192, 4096, 11008, 0, 1, "llama7b down dgrad"),
        (4096, 11008, 8192, 1, 1, "llama7b down wgrad"),
        (2048, 2304, 768, 0, 0, "gpt2 qkv fwd"),
    ]
    for M, N, K, a_mn, b_mn, what in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        for variant in (1, 2):
            ms = _time(lambda: gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=c, variant=variant))
            print(f"gemm {what:22s} M{M} N{N} K{K} variant {variant}: {ms:.3f} ms {2 * M * N * K / ms / 1e9:.0f} TFLOP/s")
        ms = _time(lambda: torch.matmul(A, B))
        print(f"     torch.matmul (cuBLAS) for scale:                 {ms:.3f} ms {2 * M * N * K / ms / 1e9:.0f} TFLOP/s")


def gemm_once():
    """Three launches of the CTA-pair GEMM on one Llama-7B forward shape (operands 64 + 96 MB, output 192 MB), for ncu."""
    from .gemm import gemm

    M, N, K = 8192, 12288, 4096
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        gemm(a, b, out=c, variant=2)
    torch.cuda.synchronize()
    print("done")


def _attn_inputs(B, S, Hq, Hkv, D):
    T = B * S
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    q, k, v = qkv[:, : Hq * D], qkv[:, Hq * D : (Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D :]
    do = torch.randn(T, Hq * D, device="cuda").bfloat16()
    return q, k, v, do


def bench_attention():
    from . import functional as pf

    for B, S, Hq, Hkv, D in [(2, 4096, 32, 32, 128), (2, 4096, 32, 8, 128), (2, 1024, 12, 12, 64)]:
        q, k, v, do = _attn_inputs(B, S, Hq, Hkv, D)
        scale = 1 / math.sqrt(D)
        o, lse = pf.flash_forward(q, k, v, B, S, Hq, Hkv, D, scale, True)
        fl = 4 * B * Hq * S * S * D / 2
        ms = _time(lambda: pf.flash_forward(q, k, v, B, S, Hq, Hkv, D, scale, True))
        print(f"attention fwd B{B} S{S} Hq{Hq} Hkv{Hkv} D{D}: {ms:.3f} ms {fl / ms / 1e9:.0f} TFLOP/s")
        ms = _time(lambda: pf.flash_backward(do, q, k, v, o, lse, B, S, Hq, Hkv, D, scale, True))
        print(f"attention bwd: {ms:.3f} ms {2.5 * fl / ms / 1e9:.0f} TFLOP/s (5-GEMM FLOPs)")
        qq = q.reshape(B, S, Hq, D).transpose(1, 2).contiguous().requires_grad_()
        kk = k.reshape(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1).contiguous().requires_grad_()
        vv = v.reshape(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1).contiguous().requires_grad_()
        ms = _time(lambda: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True))
        print(f"     SDPA fwd for scale: {ms:.3f} ms")
        oo = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True)
        gg = torch.randn_like(oo)
        ms = _time(lambda: oo.backward(gg, retain_graph=True))
        print(f"     SDPA bwd for scale: {ms:.3f} ms")


def attention_once():
    from . import functional as pf

    B, S, Hq, Hkv, D = 1, 4096, 16, 16, 128
    q, k, v, do = _attn_inputs(B, S, Hq, Hkv, D)
    for _ in range(2):
        o, lse = pf.flash_forward(q, k, v, B, S, Hq, Hkv, D, 1 / math.sqrt(D), True)
        pf.flash_backward(do, q, k, v, o, lse, B, S, Hq, Hkv, D, 1 / math.sqrt(D), True)
    torch.cuda.synchronize()
    print("done")


def bench_tp():
    """Fused all-gather->GEMM and GEMM->reduce-scatter against NCCL + cuBLAS, Llama-2-13B layer shapes.
    Launch with: python -m torch.distributed.run --nproc-per-node W -m pippy_b200.ops.bench_kernels tp"""
    import os

    import torch.distributed as dist

    from ..parallel.tp import TPContext
    from .gemm import set_sm_reserve

    rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    W = dist.get_world_size()
    T, d, ffn = 8192, 5120, 13824
    rows = T // W
    tp = TPContext(None, max_rows=rows, max_cols=max(d, 2 * ffn // W))

    def timed(fn):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(10):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / 10], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    for name, n_local in (("qkv", 3 * d // W), ("gate_up", 2 * ffn // W)):
        x = torch.randn(rows, d, device="cuda").bfloat16()
        w = (torch.randn(n_local, d, device="cuda") * 0.02).bfloat16()
        full = torch.empty(T, d, device="cuda", dtype=torch.bfloat16)

        def baseline():
            dist.all_gather_into_tensor(full, x)
            return full @ w.t()

        ms_f, ms_b = timed(lambda: tp.ag_gemm(x, w)), timed(baseline)
        flops = 2 * T * n_local * d
        wire = (W - 1) * rows * d * 2
        roof = max(flops / 1642e12, wire / 900e9) * 1e3  # measured cuBLAS burst vs NVLink nominal per direction
        if rank == 0:
            print(f"all-gather->GEMM {name:8s} [{rows}->{T},{d}]x[{n_local},{d}]: fused {ms_f:.3f} ms, NCCL+cuBLAS "
                  f"{ms_b:.3f} ms, roofline {roof:.3f} ms -> {roof / ms_f:.2f} of roofline")
    for name, k_local in (("o", d // W), ("down", ffn // W)):
        x = torch.randn(T, k_local, device="cuda").bfloat16()
        w = (torch.randn(d, k_local, device="cuda") * 0.02).bfloat16()
        out = torch.empty(rows, d, device="cuda", dtype=torch.bfloat16)

        def baseline():
            y = x @ w.t()
            dist.reduce_scatter_tensor(out, y)
            return out

        ms_f, ms_b = timed(lambda: tp.gemm_rs(x, w)), timed(baseline)
        flops = 2 * T * d * k_local
        wire = (W - 1) * rows * d * 2
        roof = max(flops / 1642e12, wire / 900e9) * 1e3  # measured cuBLAS burst vs NVLink nominal per direction
        if rank == 0:
            print(f"GEMM->reduce-scatter {name:5s} [{T},{k_local}]->[{rows},{d}]: fused {ms_f:.3f} ms, cuBLAS+NCCL "
                  f"{ms_b:.3f} ms, roofline {roof:.3f} ms -> {roof / ms_f:.2f} of roofline")
    dist.barrier()
    dist.destroy_process_group()


def _dist_setup():
    import os

    import torch.distributed as dist

    rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    return rank, dist.get_world_size()


def _dist_timed(fn, iters=10):
    import torch.distributed as dist

    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


NVLINK_NOMINAL = 900e9  # bytes/s per direction per GPU (NVLink 5); the rooflines below are quoted against this


def bench_peer_copy():
    """Measured peer-read bandwidth: every rank pulls the next rank's buffer with the package's peer all-gather kernel
    (plain 16-byte loads over NVLink, 4 in flight per thread).  With 2 ranks all of it crosses one direction of the link.
    Launch with: python -m torch.distributed.run --nproc-per-node 2 -m pippy_b200.ops.bench_kernels peer-copy"""
    import ctypes

    import torch.distributed as dist

    from ..comm.symm import SymmetricBuffer
    from . import _lib

    rank, W = _dist_setup()
    for nbytes in (64 << 20, 256 << 20, 1 << 30):
        src = SymmetricBuffer(nbytes, None, torch.device("cuda", torch.cuda.current_device()))
        flags = SymmetricBuffer(4096, None, torch.device("cuda", torch.cuda.current_device()))
        dst = torch.empty(W * nbytes, dtype=torch.uint8, device="cuda")
        counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        flg = (ctypes.POINTER(ctypes.c_int) * W)(
            *[ctypes.cast(ctypes.c_void_p(p_), ctypes.POINTER(ctypes.c_int)) for p_ in flags.ptrs])
        epoch = [0]
        for ctas in (32, 148, 296):
            def run():
                epoch[0] += 1
                _lib.check(_lib.lib().pb_peer_allgather(
                    _lib.ptr(dst), src.pointer_array(), flg, _lib.ptr(counter), _lib.ptr(_lib.err_word()),
                    _lib.c_ll(nbytes), _lib.c_int(rank), _lib.c_int(W), _lib.c_int(epoch[0]), _lib.c_int(ctas),
                    _lib.stream_ptr()), "pb_peer_allgather")

            ms = _dist_timed(run)
            if rank == 0:
                pulled = (W - 1) * nbytes
                print(f"peer all-gather {nbytes >> 20} MiB per rank, {W} ranks, {ctas} CTAs: {ms:.3f} ms, "
                      f"{pulled / ms / 1e6:.0f} GB/s pulled over NVLink per GPU ({pulled / ms / 1e6 / 900:.2f} of the "
                      f"900 GB/s nominal per direction)")
        del dst
    dist.barrier()
    dist.destroy_process_group()


def bench_dp():
    """Fused cast + scale + all-reduce of a stage's fp32 gradient buffer (bf16 on the wire) against NCCL.
    Launch with: python -m torch.distributed.run --nproc-per-node W -m pippy_b200.ops.bench_kernels dp"""
    import torch.distributed as dist

    from ..optim import FlatParams
    from ..parallel.dp import GradReducer

    rank, W = _dist_setup()
    for n in (21_000_000, 60_700_000, 256 * 1024 * 1024):  # GPT-2 stages (small / with embeddings), a 1 GiB buffer
        n = n // 64 * 64
        flat = FlatParams([torch.nn.Parameter(torch.zeros(n, device="cuda", dtype=torch.bfloat16))])
        flat.grad.normal_()
        red = GradReducer(flat, None)

        def fused():
            red.reduce_all()
            red.finish()

        wire16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)

        def nccl_bf16():
            torch.mul(flat.grad, 1.0 / W, out=flat.grad)
            wire16.copy_(flat.grad)
            dist.all_reduce(wire16)
            flat.grad.copy_(wire16)

        def nccl_fp32():
            flat.grad.mul_(1.0 / W)
            dist.all_reduce(flat.grad)

        ms_f, ms_16, ms_32 = _dist_timed(fused), _dist_timed(nccl_bf16), _dist_timed(nccl_fp32)
        # two-shot all-reduce: every rank sends and receives (W - 1) / W of the bf16 buffer twice
        wire = 2 * (W - 1) / W * n * 2
        # the slower of NVLink (per direction: (W - 1) / W of the bf16 bucket in each of the two shots) and HBM (the
        # fp32 bucket read and written once)
        roof = max(wire / 2 / NVLINK_NOMINAL, (n * 4 * 2) / 6549e9) * 1e3
        if rank == 0:
            print(f"DP all-reduce {n / 1e6:7.1f} M grads, {W} ranks: fused {ms_f:.3f} ms, NCCL bf16 wire (scale, cast, "
                  f"all-reduce, cast back) {ms_16:.3f} ms, NCCL fp32 {ms_32:.3f} ms, roofline {roof:.3f} ms (NVLink at "
                  f"900 GB/s per direction vs HBM at the measured 6549 GB/s) -> {roof / ms_f:.2f} of roofline")
        del red, flat
    dist.barrier()
    dist.destroy_process_group()


def bench_moe():
    """Fused permute + all-to-all dispatch and combine + weighted sum against all_to_all_single + index ops.
    Launch with: python -m torch.distributed.run --nproc-per-node W -m pippy_b200.ops.bench_kernels moe"""
    import torch.distributed as dist

    from ..parallel.ep import EPContext, _Plan, _RouteFn

    rank, W = _dist_setup()
    T, H, E, K = 8192, 4096, 8, 2
    ep = EPContext(None, max_tokens=T, hidden=H, top_k=K, n_experts=E)
    g = torch.Generator(device="cuda").manual_seed(rank)
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    logits = torch.randn(T, E, device="cuda", generator=g).bfloat16()
    plan = _Plan(ep, T)
    topw, _ = _RouteFn.apply(logits, plan, E, K)
    expert = plan.expert
    weight = topw.reshape(-1).contiguous()
    out = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    save = torch.empty(T * K, H, device="cuda", dtype=torch.bfloat16)
    epr = E // W

    def fused_dispatch():
        ep.dispatch(x, plan, None)

    def fused_combine():
        ep.combine(out, plan, weight, save)

    # the library way: sort assignments by destination expert, exchange counts-sized slabs, un-sort and weight
    order = torch.argsort(expert.long(), stable=True)
    tok = (order // K)
    counts = torch.bincount(expert.long(), minlength=E)
    send_splits = counts.view(W, epr).sum(1).tolist()
    allc = torch.empty(W, E, dtype=torch.int64, device="cuda")
    dist.all_gather_into_tensor(allc, counts)
    recv_splits = allc[:, rank * epr:(rank + 1) * epr].sum(1).tolist()
    recv_buf = torch.empty(sum(recv_splits), H, device="cuda", dtype=torch.bfloat16)
    back = torch.empty(T * K, H, device="cuda", dtype=torch.bfloat16)

    def lib_dispatch():
        dist.all_to_all_single(recv_buf, x[tok], recv_splits, send_splits)

    def lib_combine():
        dist.all_to_all_single(back, recv_buf, send_splits, recv_splits)
        contrib = back.float() * weight[order].unsqueeze(1)
        o = torch.zeros(T, H, device="cuda", dtype=torch.float32)
        o.index_add_(0, tok, contrib)
        return o.bfloat16()

    ms_fd, ms_ld = _dist_timed(fused_dispatch), _dist_timed(lib_dispatch)
    ms_fc, ms_lc = _dist_timed(fused_combine), _dist_timed(lib_combine)
    rows_remote = T * K * (W - 1) / W  # expected rows that leave this rank
    wire = rows_remote * H * 2
    roof = max(wire / NVLINK_NOMINAL, (T * K * H * 2 * 2) / 6549e9) * 1e3
    if rank == 0:
        print(f"MoE dispatch T{T} top-{K} H{H} E{E}, {W} ranks: fused {ms_fd:.3f} ms, all_to_all_single + gather "
              f"{ms_ld:.3f} ms, roofline {roof:.3f} ms -> {roof / ms_fd:.2f} of roofline")
        print(f"MoE combine  T{T} top-{K} H{H} E{E}, {W} ranks: fused {ms_fc:.3f} ms, all_to_all_single + index_add "
              f"{ms_lc:.3f} ms, roofline {roof:.3f} ms -> {roof / ms_fc:.2f} of roofline")
    dist.barrier()
    dist.destroy_process_group()


def _grouped_case(rows_per_group, dim, ffn2):
    """Expert-grouped activations with group starts on multiples of 256 rows, as the MoE dispatch lays them out."""
    from ..parallel.ep import EPContext, _Plan

    G = len(rows_per_group)
    starts, pos = [], 0
    for r in rows_per_group:
        starts.append(pos)
        pos += (r + 255) // 256 * 256
    ep = EPContext(None, max_tokens=max(pos // 2, 256), hidden=dim, top_k=2, n_experts=G, capacity_factor=1.0)
    plan = _Plan(ep, 1)
    plan.group_rows = torch.tensor(rows_per_group, dtype=torch.int32, device="cuda")
    plan.group_start = torch.tensor(starts, dtype=torch.int32, device="cuda")
    cap = pos
    x = torch.randn(cap, dim, device="cuda").bfloat16()
    w = (torch.randn(G, ffn2, dim, device="cuda") * 0.02).bfloat16()
    return plan, x, w, starts, cap


def bench_grouped():
    """One grouped launch over the local experts of a Mixtral layer (2 experts per rank at EP4, uneven groups) against
    the same work as a loop of this package's plain GEMM and as a loop of cuBLAS GEMMs."""
    from ..parallel.ep import grouped_gemm
    from .gemm import gemm

    dim, ffn2 = 4096, 28672
    for rows in ([4096, 4096], [5200, 3000], [1024, 1024, 1024, 1024, 1024, 1024, 1024, 1024]):
        plan, x, w, starts, cap = _grouped_case(rows, dim, ffn2)
        G = len(rows)
        y = torch.empty(cap, ffn2, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(cap, ffn2, device="cuda").bfloat16()
        dx = torch.empty(cap, dim, device="cuda", dtype=torch.bfloat16)
        dw = torch.zeros(G, ffn2, dim, device="cuda", dtype=torch.float32)
        flops = 2.0 * sum(rows) * dim * ffn2

        def loop_fwd():
            for g_, (s0, r) in enumerate(zip(starts, rows)):
                gemm(x[s0:s0 + r], w[g_], out=y[s0:s0 + r])

        def loop_cublas():
            for g_, (s0, r) in enumerate(zip(starts, rows)):
                torch.matmul(x[s0:s0 + r], w[g_].t(), out=y[s0:s0 + r])

        ms_f = _time(lambda: grouped_gemm(1, x, w, y, ffn2, dim, plan))
        ms_d = _time(lambda: grouped_gemm(1, dy, w, dx, dim, ffn2, plan, b_mn=True))
        ms_w = _time(lambda: grouped_gemm(2, dy, x, dw, dim, cap, plan, accumulate=True))
        ms_l, ms_c = _time(loop_fwd), _time(loop_cublas)
        print(f"grouped GEMM rows {rows} x [{dim} -> {ffn2}]: fwd {ms_f:.3f} ms {flops / ms_f / 1e9:.0f} TFLOP/s, dgrad "
              f"{ms_d:.3f} ms {flops / ms_d / 1e9:.0f}, wgrad (fp32 accumulate) {ms_w:.3f} ms {flops / ms_w / 1e9:.0f}; "
              f"fwd as a loop of plain GEMMs {ms_l:.3f} ms, as a loop of cuBLAS GEMMs {ms_c:.3f} ms")


def grouped_once():
    """Three grouped forward launches on a small case (operands 40 + 50 MB per launch, output 170 MB), for ncu."""
    from ..parallel.ep import grouped_gemm

    plan, x, w, starts, cap = _grouped_case([2300, 1500], 2048, 12288)
    y = torch.empty(cap, 12288, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        grouped_gemm(1, x, w, y, 12288, 2048, plan)
    torch.cuda.synchronize()
    print("grouped-once done", float(y[:2300].float().abs().mean()))


def bench_elementwise(once: bool = False):
    """Memory-bound kernels on one Llama-2-7B microbatch (T 8192, d 4096, ffn 11008), called through the C entry
    points so that no autograd bookkeeping sits between launches.  Each launch works on the next of three buffer sets
    (together larger than L2); the rate is algorithmic bytes over the CUDA-event time."""
    from . import _lib
    from .functional import _ensure_restypes, _norm_scratch, sm_count

    _ensure_restypes()
    L = _lib.lib()
    T, H, F = 8192, 4096, 11008
    dev = torch.device("cuda")
    sets = 1 if once else 3
    x = [torch.randn(T, H, device=dev).bfloat16() for _ in range(sets)]
    dy = [torch.randn(T, H, device=dev).bfloat16() for _ in range(sets)]
    y = [torch.empty(T, H, device=dev, dtype=torch.bfloat16) for _ in range(sets)]
    w = torch.randn(H, device=dev).bfloat16()
    rstd = torch.empty(T, device=dev, dtype=torch.float32)
    dw = torch.zeros(H, device=dev, dtype=torch.float32)
    scratch = _norm_scratch(H, dev)
    gu = [torch.randn(T, 2 * F, device=dev).bfloat16() for _ in range(sets)]
    h = [torch.empty(T, F, device=dev, dtype=torch.bfloat16) for _ in range(sets)]
    dgu = [torch.empty(T, 2 * F, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    k = [0]

    def nxt():
        k[0] = (k[0] + 1) % sets
        return k[0]

    def norm_fwd():
        i = nxt()
        _lib.check(L.pb_norm_fwd(_lib.ptr(x[i]), _lib.ptr(w), _lib.ptr(None), _lib.ptr(y[i]), _lib.ptr(None),
                                 _lib.ptr(rstd), _lib.c_int(T), _lib.c_int(H), _lib.c_float(1e-5), _lib.c_int(0),
                                 _lib.stream_ptr()), "pb_norm_fwd")

    def norm_bwd():
        i = nxt()
        _lib.check(L.pb_norm_bwd(_lib.ptr(dy[i]), _lib.ptr(x[i]), _lib.ptr(w), _lib.ptr(None), _lib.ptr(rstd),
                                 _lib.ptr(y[i]), _lib.ptr(dw), _lib.ptr(None), _lib.ptr(None), _lib.ptr(None),
                                 _lib.c_int(1), _lib.ptr(scratch), _lib.c_int(T), _lib.c_int(H), _lib.c_int(0),
                                 _lib.c_int(sm_count()), _lib.stream_ptr()), "pb_norm_bwd")

    def swiglu_fwd():
        i = nxt()
        _lib.check(L.pb_swiglu_fwd(_lib.ptr(gu[i]), _lib.ptr(h[i]), _lib.c_ll(T), _lib.c_int(F), _lib.ptr(None),
                                   _lib.stream_ptr()), "pb_swiglu_fwd")

    def swiglu_bwd():
        i = nxt()
        _lib.check(L.pb_swiglu_bwd(_lib.ptr(h[i]), _lib.ptr(gu[i]), _lib.ptr(dgu[i % 2]), _lib.c_ll(T), _lib.c_int(F),
                                   _lib.ptr(None), _lib.stream_ptr()), "pb_swiglu_bwd")

    cases = [
        ("norm_fwd (RMSNorm)", norm_fwd, 2 * T * H * 2),
        ("norm_bwd + partial fold", norm_bwd, 3 * T * H * 2),
        ("swiglu_fwd", swiglu_fwd, 3 * T * F * 2),
        ("swiglu_bwd", swiglu_bwd, 5 * T * F * 2),
    ]
    norm_fwd()  # rstd of a real input for the backward
    if once:
        for _, fn, _ in cases:
            fn()
        torch.cuda.synchronize()
        _lib.check_device_errors()
        return
    for name, fn, nbytes in cases:
        ms = _time(fn, iters=30)
        print(f"{name:26s} {ms * 1e3:7.1f} us  {nbytes / ms / 1e9:6.2f} TB/s")
    _lib.check_device_errors()


def bench_route():
    """Router kernels (softmax, top-2, weights, aux loss, positions: two launches) against the eager statement."""
    from ..parallel.ep import EPContext, _Plan, _RouteFn

    T, E, k = 8192, 8, 2
    ep = EPContext(None, max_tokens=T, hidden=64, top_k=k, n_experts=E)
    logits = torch.randn(T, E, device="cuda").bfloat16()
    plan = _Plan(ep, T)

    def eager():
        probs = logits.float().softmax(-1)
        w, i = probs.topk(k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        share = torch.zeros(E, device="cuda").scatter_add_(0, i.reshape(-1), torch.ones(T * k, device="cuda")) / (T * k)
        return w, i, E * (share * probs.mean(0)).sum()

    ms_k = _time(lambda: _RouteFn.apply(logits, plan, E, k))
    ms_e = _time(eager)
    print(f"MoE router T{T} E{E} top-{k}: kernels {ms_k * 1e3:.1f} us (incl. positions and counts), eager softmax/topk/"
          f"scatter_add {ms_e * 1e3:.1f} us (without positions)")


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    {"gemm": bench_gemm, "gemm-once": gemm_once, "attention": bench_attention, "attention-once": attention_once, "tp": bench_tp,
     "dp": bench_dp, "moe": bench_moe, "peer-copy": bench_peer_copy, "grouped": bench_grouped, "grouped-once": grouped_once,
     "route": bench_route, "elementwise": bench_elementwise,
     "elementwise-once": lambda: bench_elementwise(once=True)}[what]()
    from . import _lib

    _lib.check_device_errors()
