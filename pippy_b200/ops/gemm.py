"""Low-level wrapper of the tcgen05 GEMM kernel (``csrc/gemm.cu``)."""
from __future__ import annotations

import torch

from . import _lib

ACT_NONE = 0
ACT_GELU_TANH = 1


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    aux: torch.Tensor | None = None,
    act: int = ACT_NONE,
    out_fp32: bool = False,
    accumulate: bool = False,
    variant: int = 0,
) -> torch.Tensor:
    """``C[M, N] = sum_k A(m, k) * B(n, k)`` in bf16 with fp32 accumulation on the tensor cores.

    ``a`` is ``[M, K]`` (or ``[K, M]`` when ``a_mn``), ``b`` is ``[N, K]`` (or ``[K, N]`` when ``b_mn``);
    both must be 2-D bf16 CUDA tensors with unit inner stride. The epilogue optionally adds ``bias[N]``,
    applies GELU(tanh) (writing the pre-activation to ``aux``), adds ``residual[M, N]`` and either writes
    bf16, writes fp32, or accumulates into an fp32 ``out``.
    """
    assert a.is_cuda and b.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=torch.float32 if out_fp32 else torch.bfloat16)
    else:
        assert out.shape == (M, N) and out.stride(1) == 1
        out_fp32 = out.dtype == torch.float32
    if residual is not None:
        assert residual.shape == (M, N) and residual.stride(1) == 1 and residual.dtype == torch.bfloat16
    if aux is not None:
        assert aux.shape == (M, N) and aux.stride(0) == out.stride(0) and aux.dtype == torch.bfloat16
    rc = _lib.lib().pb_gemm_bf16(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out),
        _lib.c_int(M), _lib.c_int(N), _lib.c_int(K),
        _lib.c_ll(a.stride(0)), _lib.c_ll(b.stride(0)), _lib.c_ll(out.stride(0)),
        _lib.c_int(int(a_mn)), _lib.c_int(int(b_mn)),
        _lib.ptr(bias), _lib.ptr(residual), _lib.c_ll(residual.stride(0) if residual is not None else 0),
        _lib.ptr(aux), _lib.c_int(act), _lib.c_int(int(out_fp32)), _lib.c_int(int(accumulate)),
        _lib.c_int(variant), _lib.ptr(_lib.err_word(a.device)), _lib.stream_ptr(),
    )
    if rc != 0:
        raise _lib.KernelError(
            f"pb_gemm_bf16 failed with code {rc}: a {tuple(a.shape)} strides {a.stride()} ptr%16={a.data_ptr() % 16}, "
            f"b {tuple(b.shape)} strides {b.stride()} ptr%16={b.data_ptr() % 16}, out {tuple(out.shape)} "
            f"{out.dtype} strides {out.stride()}, a_mn={a_mn} b_mn={b_mn}, M={M} N={N} K={K}")
    return out


def set_sm_reserve(n: int) -> None:
    """Keeps ``n`` SMs out of the persistent GEMM grid so that communication kernels (NCCL point-to-point, the
    fused collectives of this package) always find a free SM while a GEMM is running."""
    _lib.lib().pb_set_sm_reserve(_lib.c_int(int(n)))


def set_tile_band(n: int) -> None:
    """Tile order of the plain and grouped GEMMs: output tiles are walked in bands of ``n`` row tiles, row-fastest
    inside a band (0 restores the default of 8 for CTA-pair tiles).  Which band is fastest depends on the shape by
    a few percent (measured under sustained load on the 7B shapes: 4 is 5 % ahead on the QKV forward, 8 is 2 % ahead
    on the gate/up dgrad, the rest within noise), so the default is left alone; the knob is for tuning a new shape."""
    _lib.lib().pb_set_gemm_group_m(_lib.c_int(int(n)))
