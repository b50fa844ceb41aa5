"""Micro-benchmarks of the package's kernels, timed with CUDA events (3 warm-ups, 10 timed launches).

    python -m pippy_b200.ops.bench_kernels gemm
    python -m pippy_b200.ops.bench_kernels attention
    python -m pippy_b200.ops.bench_kernels attention-once     # two forward+backward calls on a small case, for ncu

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
        roof = max(flops / 1642e12, wire / 770e9) * 1e3
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
        roof = max(flops / 1642e12, wire / 770e9) * 1e3
        if rank == 0:
            print(f"GEMM->reduce-scatter {name:5s} [{T},{k_local}]->[{rows},{d}]: fused {ms_f:.3f} ms, cuBLAS+NCCL "
                  f"{ms_b:.3f} ms, roofline {roof:.3f} ms -> {roof / ms_f:.2f} of roofline")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    {"gemm": bench_gemm, "attention": bench_attention, "attention-once": attention_once, "tp": bench_tp}[what]()
    from . import _lib

    _lib.check_device_errors()
