"""GEMM with a fused epilogue on the B200 kernels: the linear layers around attention.

Host side of `b200_gemm` (include/b200_attn.h), with the call contract of the reference's `DptFused.gemm`
(`src/fastforks/kernels/dpt_fused/__init__.py:179-220`): `epilogue(x @ w^T)` with
`epilogue(acc) = act((acc + bias) * scale + res)` (`src/fastforks/kernels/dpt_fused/dpt_fused.cu:7-18`). Nothing here
computes: without the CUDA library the call raises `KernelUnavailableError`.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib

ACT_NONE, ACT_RELU, ACT_GELU, ACT_GELU_TANH = 0, 1, 5, 6  # the reference's codes (dpt_fused/__init__.py)
_DTYPES = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def _rows(t: torch.Tensor, m: int, n: int, name: str) -> int:
    """Row stride of `t` seen as `[m, n]` rows (the reference's `_rows`): last dim contiguous, rows equally spaced."""
    if t.shape[-1] != n or t.numel() != m * n or t.stride(-1) != 1:
        msg = f"gemm: {name} must hold {m} rows of {n} contiguous values, got {tuple(t.shape)} strides {t.stride()}"
        raise ValueError(msg)
    if t.dim() == 1:
        return n
    flat = t.reshape(m, n) if t.is_contiguous() else None
    if flat is not None:
        return n
    if t.dim() == 2:  # noqa: PLR2004
        return t.stride(0)
    msg = f"gemm: {name} must be contiguous or a 2-D view with unit last stride"
    raise ValueError(msg)


def gemm(  # noqa: PLR0913 - the epilogue terms
    x: torch.Tensor,
    w: torch.Tensor,
    bias: torch.Tensor | None = None,
    *,
    act: int = ACT_NONE,
    scale: torch.Tensor | None = None,
    res: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """`act((x @ w^T + bias) * scale + res)` for x `[..., K]` and w `[N, K]` (contiguous), fp16 or bf16.

    Args:
        x: CUDA `[..., K]`, rows contiguous (a 2-D view with a row stride is fine).
        w: `[N, K]` contiguous, same dtype.
        bias: `[N]`, same dtype.
        act: `ACT_NONE`, `ACT_RELU`, `ACT_GELU` (erf) or `ACT_GELU_TANH`.
        scale: fp32 `[N]`, applied to `acc + bias` before the residual (LayerScale: `gamma`).
        res: `[..., N]` residual, same dtype.
        out: gets the result (may be `res` itself: in-place residual); else a new `[..., N]` tensor.

    Raises:
        ValueError: Operands outside the contract (checked before the launch).
        KernelUnavailableError: The CUDA library is not built or does not load.
    """
    if x.dtype not in _DTYPES or not x.is_cuda:
        msg = f"gemm: x must be a float16 / bfloat16 CUDA tensor, got {x.dtype} on {x.device}"
        raise ValueError(msg)
    if (x.requires_grad or w.requires_grad) and torch.is_grad_enabled():
        msg = "gemm: an operand requires grad; the kernels backend is inference-only (use torch.no_grad())"
        raise ValueError(msg)
    k = x.shape[-1]
    m = x.numel() // k
    n = w.shape[0]
    if w.dtype != x.dtype or w.device != x.device or w.dim() != 2 or w.shape[1] != k or not w.is_contiguous():  # noqa: PLR2004
        msg = f"gemm: weight must be contiguous {x.dtype} [N, {k}] on {x.device}, got {tuple(w.shape)} {w.dtype}"
        raise ValueError(msg)
    a = _lib.B200GemmArgs()
    a.struct_size = ctypes.sizeof(_lib.B200GemmArgs)
    a.dtype, a.m, a.n, a.k, a.act = _DTYPES[x.dtype], m, n, k, act
    a.x, a.lda, a.w = x.data_ptr(), _rows(x, m, k, "x"), w.data_ptr()
    y = out if out is not None else x.new_empty((*x.shape[:-1], n))
    if y.dtype != x.dtype or y.device != x.device:
        msg = f"gemm: out must be {x.dtype} on {x.device}"
        raise ValueError(msg)
    a.y, a.ldy = y.data_ptr(), _rows(y, m, n, "out")
    for name, t, dtype in (("bias", bias, x.dtype), ("scale", scale, torch.float32)):
        if t is not None and (t.shape != (n,) or t.dtype != dtype or t.device != x.device or not t.is_contiguous()):
            msg = f"gemm: {name} must be contiguous {dtype} [{n}] on {x.device}, got {tuple(t.shape)} {t.dtype}"
            raise ValueError(msg)
    a.bias = None if bias is None else bias.data_ptr()
    a.scale = None if scale is None else scale.data_ptr()
    if res is not None:
        if res.dtype != x.dtype or res.device != x.device:
            msg = f"gemm: res must be {x.dtype} on {x.device}"
            raise ValueError(msg)
        a.res, a.lres = res.data_ptr(), _rows(res, m, n, "res")
    with torch.cuda.device(x.device):
        code = _lib.library().b200_gemm(ctypes.byref(a), torch._C._cuda_getCurrentRawStream(x.device.index))  # noqa: SLF001
    _lib.raise_for_code(code, "gemm")
    return y
