"""Numerics of every CUDA kernel against a plain PyTorch fp32 statement of the same op (needs a B200)."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _bf16(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6)).item()


@pytest.fixture(autouse=True)
def _seed_and_check():
    torch.manual_seed(0)
    yield
    from pippy_b200.ops import _lib

    _lib.check_device_errors()


@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1)])
def test_gemm_layouts(variant, a_mn, b_mn):
    from pippy_b200.ops.gemm import gemm

    M, N, K = 1000, 776, 520
    a = _bf16(K, M) if a_mn else _bf16(M, K)
    b = _bf16(K, N) if b_mn else _bf16(N, K)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    out = gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), variant=variant)
    assert _rel(out, ref) < 1e-2


@pytest.mark.parametrize("variant", [1, 2])
def test_gemm_epilogues(variant):
    from pippy_b200.ops.gemm import gemm

    M, N, K = 512, 768, 256
    a, b = _bf16(M, K), _bf16(N, K)
    bias, res = _bf16(N), _bf16(M, N)
    r0 = a.float() @ b.float().t()
    assert _rel(gemm(a, b, bias=bias, residual=res, variant=variant), r0 + bias.float() + res.float()) < 1e-2
    aux = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, bias=bias, act=1, aux=aux, variant=variant)
    assert _rel(out, F.gelu(r0 + bias.float(), approximate="tanh")) < 1e-2
    assert _rel(aux, r0 + bias.float()) < 1e-2
    acc = torch.ones(M, N, device="cuda")
    gemm(a, b, out=acc, accumulate=True, variant=variant)
    assert _rel(acc, r0 + 1) < 1e-4


@pytest.mark.parametrize("H", [768, 4096, 5120])
@pytest.mark.parametrize("layer", [False, True])
def test_norm(H, layer):
    from pippy_b200.ops import functional as pf

    T = 515
    x = _bf16(T, H).requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
    b = (0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_() if layer else None
    dy = _bf16(T, H)
    y = pf.layer_norm(x, w, b, 1e-5) if layer else pf.rms_norm(x, w, 1e-5)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    if layer:
        bf = b.detach().float().requires_grad_()
        yr = F.layer_norm(xf, (H,), wf, bf, 1e-5)
    else:
        yr = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    yr.backward(dy.float())
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xf.grad) < 1e-2
    assert _rel(w.grad, wf.grad) < 2e-2
    if layer:
        assert _rel(b.grad, bf.grad) < 2e-2


def test_norm_fork_adds_the_residual_gradient():
    """``rms_norm_fork`` hands back its input for the residual branch; the gradient that returns through it is added
    to the norm's input gradient by the backward kernel."""
    from pippy_b200.ops import functional as pf

    T, H = 515, 4096
    x = _bf16(T, H).requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
    dy, dr = _bf16(T, H), _bf16(T, H)
    y, xr = pf.rms_norm_fork(x, w, 1e-5)
    assert xr.data_ptr() == x.data_ptr()
    torch.autograd.backward([y, xr], [dy, dr])
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    torch.autograd.backward([yr, xf * 1.0], [dy.float(), dr.float()])
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xf.grad) < 1e-2
    assert _rel(w.grad, wf.grad) < 2e-2
    # only the residual branch used: the gradient passes through
    x2 = _bf16(T, H).requires_grad_()
    _, xr2 = pf.rms_norm_fork(x2, w, 1e-5)
    xr2.backward(dr)
    assert torch.equal(x2.grad, dr)


def test_llama_block_matches_fp32_reference():
    """One decoder layer on the kernels (bf16) against the same layer's plain PyTorch path in fp32 on the CPU:
    output, input gradient and the gradients of both norm weights and of the down projection."""
    from pippy_b200.models.llama import LlamaBlock, LlamaConfig

    cfg = LlamaConfig(vocab_size=256, dim=512, n_layers=1, n_heads=4, ffn_dim=1024)
    B, S = 2, 128
    torch.manual_seed(3)
    ref = LlamaBlock(cfg, dtype=torch.float32)
    with torch.no_grad():
        for name, prm in ref.named_parameters():
            if name.endswith("norm.weight"):
                prm.add_(0.1 * torch.randn_like(prm))
            prm.copy_(prm.bfloat16().float())  # both sides start from the same bf16-representable weights
    blk = LlamaBlock(cfg, device="cuda", dtype=torch.bfloat16)
    blk.load_state_dict({k: v.bfloat16() for k, v in ref.state_dict().items()})
    x = (0.5 * torch.randn(B * S, cfg.dim)).bfloat16()
    dy = (0.1 * torch.randn(B * S, cfg.dim)).bfloat16()
    xg = x.cuda().requires_grad_()
    out = blk(xg, B, S)
    out.backward(dy.cuda())
    xr = x.float().requires_grad_()
    out_ref = ref(xr, B, S)
    out_ref.backward(dy.float())
    assert _rel(out.cpu(), out_ref) < 2e-2
    assert _rel(xg.grad.cpu(), xr.grad) < 3e-2
    got = dict(blk.named_parameters())
    for name in ("attention_norm.weight", "ffn_norm.weight", "feed_forward.w_down.weight"):
        want = dict(ref.named_parameters())[name].grad
        g = got[name].grad if got[name].grad is not None else got[name].main_grad
        assert _rel(g.cpu(), want) < 5e-2, name


def test_swiglu_and_gelu_linear():
    from pippy_b200.ops import functional as pf

    T, Fd = 300, 1408
    gu = _bf16(T, 2 * Fd).requires_grad_()
    d = _bf16(T, Fd)
    out = pf.swiglu(gu)
    out.backward(d)
    gf = gu.detach().float().requires_grad_()
    g, u = gf.chunk(2, -1)
    ref = F.silu(g) * u
    ref.backward(d.float())
    assert _rel(out, ref) < 1e-2 and _rel(gu.grad, gf.grad) < 1e-2

    x = _bf16(T, 256).requires_grad_()
    w = _bf16(512, 256, scale=0.05).requires_grad_()
    bias = _bf16(512, scale=0.1).requires_grad_()
    res = _bf16(T, 512).requires_grad_()
    dy = _bf16(T, 512)
    y = pf.linear(x, w, bias, residual=res, activation="gelu_tanh")
    y.backward(dy)
    xf, wf, bf, rf = (t.detach().float().requires_grad_() for t in (x, w, bias, res))
    yr = F.gelu(F.linear(xf, wf, bf), approximate="tanh") + rf
    yr.backward(dy.float())
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xf.grad) < 2e-2
    assert _rel(w.grad, wf.grad) < 2e-2
    assert _rel(bias.grad, bf.grad) < 2e-2
    assert _rel(res.grad, rf.grad) < 1e-2


def test_linear_main_grad_accumulates_fp32():
    from pippy_b200.ops import functional as pf

    x = _bf16(256, 128).requires_grad_()
    w = _bf16(384, 128, scale=0.05).requires_grad_()
    w.main_grad = torch.zeros(384, 128, device="cuda")
    for _ in range(2):
        pf.linear(x, w).backward(torch.ones(256, 384, device="cuda", dtype=torch.bfloat16))
    ref = 2 * torch.ones(256, 384, device="cuda").t() @ x.detach().float()
    assert w.grad is None and _rel(w.main_grad, ref) < 1e-3


def test_cross_entropy():
    from pippy_b200.ops import functional as pf

    T, V, Vp = 257, 1000, 1024
    logits = _bf16(T, Vp, scale=2.0).requires_grad_()
    tgt = torch.randint(0, V, (T,), device="cuda")
    tgt[5] = -100
    loss = pf.cross_entropy(logits, tgt, vocab_size=V, reduction="mean")
    (loss * 3.0).backward()
    lf = logits.detach().float().requires_grad_()
    ref = F.cross_entropy(lf[:, :V], tgt, reduction="mean", ignore_index=-100)
    (ref * 3.0).backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item())
    assert (logits.grad.float() - lf.grad).abs().max().item() < 2e-4
    assert logits.grad[:, V:].abs().max().item() == 0


def test_embedding():
    from pippy_b200.ops import functional as pf

    V, H, B, S = 500, 256, 3, 64
    wte = _bf16(V, H).requires_grad_()
    wpe = _bf16(S, H).requires_grad_()
    ids = torch.randint(0, V, (B, S), device="cuda")
    out = pf.embedding(ids, wte, wpe, S)
    d = _bf16(B * S, H)
    out.backward(d)
    wf, pf_ = wte.detach().float().requires_grad_(), wpe.detach().float().requires_grad_()
    pos = torch.arange(B * S, device="cuda") % S
    ref = F.embedding(ids.reshape(-1), wf) + F.embedding(pos, pf_)
    ref.backward(d.float())
    assert _rel(out, ref) < 1e-2
    assert _rel(wte.grad, wf.grad) < 1e-2 and _rel(wpe.grad, pf_.grad) < 1e-2


def test_fused_adamw_matches_torch():
    import torch.nn as nn

    from pippy_b200.optim import FlatParams, FusedAdamW

    ps = [nn.Parameter(_bf16(300, 70)), nn.Parameter(_bf16(129))]
    ref = [nn.Parameter(p.detach().float().clone()) for p in ps]
    flat = FlatParams(ps)
    opt = FusedAdamW(flat, lr=1e-2, weight_decay=0.1, master_weights=True)
    ropt = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.1)
    for _ in range(3):
        for p, r in zip(ps, ref):
            g = torch.randn_like(r)
            p.main_grad.copy_(g)
            r.grad = g.clone()
        opt.step(zero_grad=True)
        ropt.step()
    for p, r in zip(ps, ref):
        assert _rel(p, r) < 1e-2
        assert p.main_grad.abs().max().item() == 0
    assert _rel(opt.master[0][: ps[0].numel()].view_as(ref[0]), ref[0]) < 1e-5


def _attn_ref(q, k, v, causal, scale):
    # q [B,S,Hq,D], k/v [B,S,Hkv,D] fp32
    rep = q.shape[2] // k.shape[2]
    k = k.repeat_interleave(rep, dim=2)
    v = v.repeat_interleave(rep, dim=2)
    att = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
    if causal:
        S = q.shape[1]
        att = att.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", att.softmax(-1), v)


@pytest.mark.parametrize("B,S,Hq,Hkv,D", [(2, 256, 4, 4, 128), (1, 384, 8, 2, 128), (2, 320, 4, 4, 64), (1, 1024, 2, 1, 64)])
def test_flash_attention_fwd_bwd(B, S, Hq, Hkv, D):
    from pippy_b200.ops import functional as pf

    T = B * S
    qkv = _bf16(T, (Hq + 2 * Hkv) * D).requires_grad_()
    do = _bf16(T, Hq * D)
    out = pf.rope_attention(qkv, None, None, B, S, Hq, Hkv, D)
    out.backward(do)
    qf = qkv.detach().float().requires_grad_()
    q = qf[:, : Hq * D].view(B, S, Hq, D)
    k = qf[:, Hq * D : (Hq + Hkv) * D].view(B, S, Hkv, D)
    v = qf[:, (Hq + Hkv) * D :].view(B, S, Hkv, D)
    ref = _attn_ref(q, k, v, True, 1 / math.sqrt(D)).reshape(T, Hq * D)
    ref.backward(do.float())
    assert _rel(out, ref) < 2e-2
    g, gr = qkv.grad.float(), qf.grad
    for name, sl in (("dq", slice(0, Hq * D)), ("dk", slice(Hq * D, (Hq + Hkv) * D)), ("dv", slice((Hq + Hkv) * D, None))):
        assert _rel(g[:, sl], gr[:, sl]) < 3e-2, name


def test_rope_attention_with_rotary():
    from pippy_b200.ops import functional as pf

    B, S, Hq, Hkv, D = 2, 256, 4, 2, 128
    T = B * S
    base = _bf16(T, (Hq + 2 * Hkv) * D)
    cos, sin = pf.rope_tables(S, D, 10000.0, "cuda")
    qkv = base.clone().requires_grad_()
    do = _bf16(T, Hq * D)
    qkv_in = qkv * 1  # the op rotates its input in place; give it a private buffer
    out = pf.rope_attention(qkv_in, cos, sin, B, S, Hq, Hkv, D)
    out.backward(do)
    qf = base.float().requires_grad_()
    q = pf._rope_ref(qf[:, : Hq * D].view(B, S, Hq, D), cos, sin)
    k = pf._rope_ref(qf[:, Hq * D : (Hq + Hkv) * D].view(B, S, Hkv, D), cos, sin)
    v = qf[:, (Hq + Hkv) * D :].view(B, S, Hkv, D)
    ref = _attn_ref(q.float(), k.float(), v, True, 1 / math.sqrt(D)).reshape(T, Hq * D)
    ref.backward(do.float())
    assert _rel(out, ref) < 2e-2
    assert _rel(qkv.grad, qf.grad) < 3e-2



@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1)])
def test_gemm_many_tiles_per_cta(variant, a_mn, b_mn):
    """4096 x 8192 has 512 tiles of 256 x 256 (2048 of 128 x 128): every persistent CTA works through several
    tiles, so the accumulator ping-pong in TMEM, the wrap of the shared-memory ring across tiles and the grouped
    rasterisation all run, as they do in a training step."""
    from pippy_b200.ops.gemm import gemm

    M, N, K = 4096, 8192, 1024
    a = _bf16(K, M) if a_mn else _bf16(M, K)
    b = _bf16(K, N) if b_mn else _bf16(N, K)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    out = gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), variant=variant)
    assert _rel(out, ref) < 1e-2
    # a dropped or doubled tile shows as an O(1) error somewhere; rounding alone stays far below this everywhere
    assert ((out.float() - ref).abs() / ref.abs().clamp(min=8.0)).max().item() < 5e-2


def test_gemm_many_tiles_with_reserved_sms():
    """The grid that leaves SMs free for communication kernels covers the same tiles."""
    from pippy_b200.ops.gemm import gemm, set_sm_reserve

    M, N, K = 4096, 4096, 512
    a, b = _bf16(M, K), _bf16(N, K)
    ref = a.float() @ b.float().t()
    try:
        set_sm_reserve(8)
        out = gemm(a, b)
    finally:
        set_sm_reserve(0)
    assert _rel(out, ref) < 1e-2


def test_flash_attention_long_sequence():
    """The training shape's sequence length: 32 key blocks per query block, head dim 128."""
    from pippy_b200.ops import functional as pf

    B, S, Hq, Hkv, D = 1, 4096, 2, 2, 128
    T = B * S
    qkv = _bf16(T, (Hq + 2 * Hkv) * D).requires_grad_()
    do = _bf16(T, Hq * D)
    out = pf.rope_attention(qkv * 1, None, None, B, S, Hq, Hkv, D)
    out.backward(do)
    qf = qkv.detach().float().requires_grad_()
    q = qf[:, : Hq * D].view(B, S, Hq, D)
    k = qf[:, Hq * D : (Hq + Hkv) * D].view(B, S, Hkv, D)
    v = qf[:, (Hq + Hkv) * D :].view(B, S, Hkv, D)
    ref = _attn_ref(q, k, v, True, 1 / math.sqrt(D)).reshape(T, Hq * D)
    ref.backward(do.float())
    assert _rel(out, ref) < 2e-2
    g, gr = qkv.grad.float(), qf.grad
    for name, sl in (("dq", slice(0, Hq * D)), ("dk", slice(Hq * D, (Hq + Hkv) * D)), ("dv", slice((Hq + Hkv) * D, None))):
        assert _rel(g[:, sl], gr[:, sl]) < 3e-2, name


def test_peer_wait_runs_out_and_reports():
    """Failure detection on the device: the all-reduce kernel is launched as rank 0 of 2 with a second flag block
    that nobody ever writes (both "ranks" are buffers of this one GPU) and a wait limit of a few milliseconds.
    The kernel must return by itself, the error word must say "peer wait ran out", and the next launch must work."""
    import ctypes

    from pippy_b200.ops import _lib

    lib = _lib.lib()
    lib.pb_set_peer_wait_ms.argtypes = [ctypes.c_double]
    n = 1 << 16
    grad = torch.randn(n, device="cuda")
    staging = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    flags = [torch.zeros(64, device="cuda", dtype=torch.int32) for _ in range(2)]
    counter = torch.zeros(2, device="cuda", dtype=torch.int32)
    stag = (ctypes.c_void_p * 2)(*[ctypes.c_void_p(t.data_ptr()) for t in staging])
    flg = (ctypes.POINTER(ctypes.c_int) * 2)(
        *[ctypes.cast(ctypes.c_void_p(t.data_ptr()), ctypes.POINTER(ctypes.c_int)) for t in flags])
    grid = ctypes.c_int(0)
    err = _lib.err_word(grad.device)
    try:
        lib.pb_set_peer_wait_ms(5.0)
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        rc = lib.pb_dp_allreduce(_lib.ptr(grad), stag, flg, _lib.ptr(counter), _lib.ptr(err), _lib.c_ll(n),
                                 _lib.c_float(0.5), _lib.c_int(0), _lib.c_int(2), _lib.c_int(1), _lib.c_int(8),
                                 ctypes.byref(grid), _lib.stream_ptr())
        assert rc == 0
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 1000.0  # gave up after milliseconds, not after the default 3 s
        with pytest.raises(_lib.KernelError, match="peer wait ran out"):
            _lib.check_device_errors()
    finally:
        lib.pb_set_peer_wait_ms(0.0)
    # the context is intact: the same kernel as a one-rank group completes and scales the gradients
    before = grad.clone()
    rc = lib.pb_dp_allreduce(_lib.ptr(grad), stag, flg, _lib.ptr(counter), _lib.ptr(err), _lib.c_ll(n),
                             _lib.c_float(0.5), _lib.c_int(0), _lib.c_int(1), _lib.c_int(2), _lib.c_int(8),
                             ctypes.byref(grid), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    _lib.check_device_errors()
    torch.testing.assert_close(grad, (before * 0.5).bfloat16().float())


@pytest.mark.parametrize("schedule", ["interleaved_1f1b", "zero_bubble"])
def test_llama_activation_checkpointing_same_gradients(schedule):
    """Recomputing each block's forward inside the backward gives the gradients of the plain run: the kernels are
    deterministic, so everything but the atomically accumulated sums (norm weights, embedding rows) is bit-equal."""
    from pippy_b200.models.llama import LlamaConfig
    from pippy_b200.train import build_llama_pipeline

    dev = torch.device("cuda", 0)
    cfg = LlamaConfig(vocab_size=1024, dim=512, n_layers=4, n_heads=4, ffn_dim=1024)
    ids = torch.randint(0, cfg.vocab_size, (4, 256), device=dev)
    grads, losses = {}, {}
    for ckpt in (False, True):
        pipe = build_llama_pipeline(cfg, 4, 256, 2, dev, schedule=schedule, virtual_stages=2, seed=11,
                                    with_optimizer=True, activation_checkpointing=ckpt)
        pipe.optimizer = None  # keep the accumulated gradients: compare them, not the updated weights
        losses[ckpt] = float(pipe.train_step(ids, ids))
        torch.cuda.synchronize()
        grads[ckpt] = {n: p.main_grad.clone() for st in pipe.stages for n, p in st.submod.named_parameters()}
    assert abs(losses[True] - losses[False]) < 1e-6
    for n, g in grads[False].items():
        assert g.abs().max().item() > 0, n
        assert _rel(grads[True][n], g) < 1e-3, n


def test_moe_router_kernels():
    """softmax / top-k / normalised weights / load-balance loss / positions, and the logit gradient, against the
    plain PyTorch statement."""
    from pippy_b200.parallel.ep import EPContext, _Plan, _RouteFn

    T, E, k, H = 1000, 8, 2, 64
    ep = EPContext(None, max_tokens=T, hidden=H, top_k=k, n_experts=E)
    logits = _bf16(T, E, scale=1.5).requires_grad_()
    plan = _Plan(ep, T)
    topw, aux = _RouteFn.apply(logits, plan, E, k)
    gw = torch.randn(T, k, device="cuda")
    ((topw * gw).sum() + 0.37 * aux).backward()

    lf = logits.detach().float().requires_grad_()
    probs = lf.softmax(-1)
    ri = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :k]  # ties: lower index first
    rw = probs.gather(-1, ri)
    rwn = rw / rw.sum(-1, keepdim=True)
    share = torch.bincount(ri.reshape(-1), minlength=E).float() / (T * k)
    raux = E * (share * probs.mean(0)).sum()
    ((rwn * gw).sum() + 0.37 * raux).backward()
    assert torch.equal(plan.expert.view(T, k).long(), ri)
    torch.testing.assert_close(topw, rwn, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(aux, raux, rtol=1e-5, atol=1e-6)
    assert torch.equal(plan.counts.long(), torch.bincount(ri.reshape(-1), minlength=E))
    # positions: assignment (t, j) is the n-th token (in token order) that chose its expert
    flat = ri.reshape(-1)
    want = torch.empty_like(flat)
    for e in range(E):
        idx = (flat == e).nonzero(as_tuple=True)[0]
        want[idx] = torch.arange(idx.numel(), device="cuda")
    assert torch.equal(plan.slot.long(), want)
    assert _rel(logits.grad, lf.grad) < 1e-2


@pytest.mark.parametrize("T", [384, 1500])
def test_moe_layer_one_rank_against_dense(T):
    """The whole expert-parallel layer (route, dispatch, grouped GEMMs, combine and their backward) with an
    expert-parallel group of one rank, against the dense PyTorch statement of the layer."""
    from pippy_b200.parallel.ep import EPContext, MoEFeedForward

    H, Fd, E, k = 256, 512, 4, 2
    ep = EPContext(None, max_tokens=T, hidden=H, top_k=k, n_experts=E, capacity_factor=1.0)
    torch.manual_seed(5)
    dense = MoEFeedForward(H, Fd, E, k, None, 1, 0, aux_coef=0.01, device="cuda", dtype=torch.bfloat16)
    fused = MoEFeedForward(H, Fd, E, k, ep, 1, 0, aux_coef=0.01, device="cuda", dtype=torch.bfloat16)
    fused.load_state_dict(dense.state_dict())
    for it in range(2):  # the second pass reuses buffers and flags
        x = _bf16(T, H)
        dy = _bf16(T, H)
        xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
        for m in (dense, fused):
            for p in m.parameters():
                p.grad = None
        out = fused(xa)
        out.backward(dy)
        ref = dense(xb)
        ref.backward(dy)
        torch.cuda.synchronize()
        assert _rel(out, ref) < 2e-2, ("out", it)
        assert _rel(xa.grad, xb.grad) < 2e-2, ("dx", it)
        assert _rel(fused.router.grad[:E], dense.router.grad[:E]) < 3e-2, ("drouter", it)
        assert _rel(fused.w_down.grad, dense.w_down.grad) < 2e-2, ("dWdown", it)
        assert _rel(fused.w_gate_up.grad, dense.w_gate_up.grad) < 2e-2, ("dWgu", it)
        assert abs(float(fused.last_aux_loss) - float(dense.last_aux_loss)) < 1e-3


def test_bounds_checking_library_reports_bad_indices():
    """The debug library (PIPPY_BOUNDS_CHECK=1) validates indices read from tensors: a token id and a class label
    outside their tables are reported through the device error word and the accesses are skipped, so the kernels
    finish, the context stays usable and the in-range rows are still right."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = """
import torch
from pippy_b200.ops import _lib, functional as pf
assert _lib.bounds_check_enabled()
_lib.err_word(torch.device("cuda", 0))
wte = torch.randn(100, 64, device="cuda").bfloat16()
ids = torch.tensor([[1, 5, 250, 7]], device="cuda")          # 250 is outside the 100-row table
out = pf.embedding(ids, wte)
torch.cuda.synchronize()
assert torch.equal(out[0], wte[1]) and torch.equal(out[3], wte[7])
try:
    _lib.check_device_errors()
    raise SystemExit("the bad token id was not reported")
except _lib.KernelError as e:
    assert "code 5" in str(e), e
logits = torch.randn(4, 104, device="cuda").bfloat16()
tgt = torch.tensor([3, 99, 1000, 5], device="cuda")           # 1000 is outside the 100 classes
loss = pf.cross_entropy(logits, tgt, vocab_size=100, reduction="sum")
torch.cuda.synchronize()
try:
    _lib.check_device_errors()
    raise SystemExit("the bad label was not reported")
except _lib.KernelError as e:
    assert "code 5" in str(e), e
ok = pf.cross_entropy(logits, torch.tensor([3, 99, 0, 5], device="cuda"), vocab_size=100, reduction="sum")
torch.cuda.synchronize()
_lib.check_device_errors()
print("bounds-check build ok", float(loss), float(ok))
"""
    env = dict(os.environ, PIPPY_BOUNDS_CHECK="1", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "bounds-check build ok" in res.stdout
