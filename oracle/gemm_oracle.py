"""CPU oracle of the fused-epilogue GEMM: TEST INFRASTRUCTURE ONLY, never imported by the product.

A numpy restatement of the epilogue contract of the reference's `dpt_fused` GEMMs
(`src/fastforks/kernels/dpt_fused/dpt_fused.cu:7-18`, activation codes `:52-64`):

    y = act((x @ w^T + bias) * scale + res)          act: 0 none, 1 relu, 5 gelu (erf), 6 gelu (tanh form)

computed in fp32 (or the dtype given) on the operands as they are (the tests pass operands already rounded to
16 bits). Pinned by `tests/golden/gemm_epilogue.npz`, which `tests/golden/make_golden.py` writes with the torch calls
the reference's portable blocks make for these layers (`F.linear`, `F.gelu`, `F.relu`, LayerScale and residual as in
`NestedTensorBlock`), see `tests/test_oracle.py`.
"""

from __future__ import annotations

import math

import numpy as np

ACT_NONE, ACT_RELU, ACT_GELU, ACT_GELU_TANH = 0, 1, 5, 6


def _erf(x: np.ndarray) -> np.ndarray:
    try:
        from scipy.special import erf
    except ImportError:  # pragma: no cover - scipy is part of the image
        return np.vectorize(math.erf, otypes=[x.dtype])(x)
    return erf(x).astype(x.dtype)


def activation(v: np.ndarray, act: int) -> np.ndarray:
    if act == ACT_NONE:
        return v
    if act == ACT_RELU:
        return np.maximum(v, 0)
    if act == ACT_GELU:
        return (0.5 * v * (1.0 + _erf(v * v.dtype.type(0.70710678118654752)))).astype(v.dtype)
    if act == ACT_GELU_TANH:
        u = v.dtype.type(0.7978845608028654) * v * (1 + v.dtype.type(0.044715) * v * v)
        return (0.5 * v * (1.0 + np.tanh(u))).astype(v.dtype)
    msg = f"act {act} unknown"
    raise ValueError(msg)


def gemm_epilogue(x, w, bias=None, scale=None, res=None, act: int = ACT_NONE, dtype=np.float32):  # noqa: ANN001, ANN201, PLR0913
    """`act((x @ w^T + bias) * scale + res)` for x `[M, K]`, w `[N, K]`, bias / scale `[N]`, res `[M, N]`."""
    v = np.asarray(x, dtype=dtype) @ np.asarray(w, dtype=dtype).T
    if bias is not None:
        v = v + np.asarray(bias, dtype=dtype)
    if scale is not None:
        v = v * np.asarray(scale, dtype=dtype)
    if res is not None:
        v = v + np.asarray(res, dtype=dtype)
    return activation(v.astype(dtype), act)
