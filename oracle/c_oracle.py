"""ctypes binding of the C oracle (`attn_oracle.c`): TEST INFRASTRUCTURE ONLY, never imported by the product.

`build()` compiles `liboracle_attn.so` with gcc next to the source; `attention()` runs it over contiguous fp32
`[B, H, N, d]` arrays, splitting output rows over `threads` Python threads (ctypes releases the GIL).
"""

from __future__ import annotations

import ctypes
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SHARED_OBJECT = HERE / "liboracle_attn.so"


def build() -> Path:
    """Compile the C oracle if it is missing or older than its source."""
    src = HERE / "attn_oracle.c"
    if not SHARED_OBJECT.exists() or SHARED_OBJECT.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "liboracle_attn.so"], check=True, capture_output=True)
    return SHARED_OBJECT


def _lib() -> ctypes.CDLL:
    lib = ctypes.CDLL(str(build()))
    fp = ctypes.POINTER(ctypes.c_float)
    lib.attn_oracle_f32.argtypes = (
        fp, fp, fp, fp, fp, fp, ctypes.c_int, ctypes.c_int, fp,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
        ctypes.c_long, ctypes.c_long,
    )  # fmt: skip
    lib.attn_oracle_f32.restype = ctypes.c_int
    return lib


def attention(q, k, v, scale=None, bias=None, rel=None, threads: int = 1):  # noqa: ANN001, ANN201
    """`softmax(scale * q k^T + bias) v`; `bias` dense `[B, H, Nq, Nk]` or `rel=(rel_h, rel_w)` decomposed."""
    lib = _lib()
    fp = ctypes.POINTER(ctypes.c_float)

    def arr(x):  # noqa: ANN001, ANN202
        return None if x is None else np.ascontiguousarray(x, dtype=np.float32)

    def ptr(x):  # noqa: ANN001, ANN202
        return None if x is None else x.ctypes.data_as(fp)

    q, k, v = arr(q), arr(k), arr(v)
    b, h, nq, d = q.shape
    nk = k.shape[2]
    if bias is not None:
        bias = arr(np.broadcast_to(bias, (b, h, nq, nk)))
    rel_h, rel_w = (arr(rel[0]), arr(rel[1])) if rel is not None else (None, None)
    kh, kw = (rel_h.shape[-1], rel_w.shape[-1]) if rel is not None else (0, 0)
    out = np.empty_like(q)
    scale = d**-0.5 if scale is None else float(scale)
    rows = b * h * nq
    cuts = np.linspace(0, rows, max(1, threads) + 1).astype(np.int64)

    def run(i: int) -> int:
        return lib.attn_oracle_f32(ptr(q), ptr(k), ptr(v), ptr(bias), ptr(rel_h), ptr(rel_w), kh, kw, ptr(out),
                                   b, h, nq, nk, d, scale, int(cuts[i]), int(cuts[i + 1]))  # fmt: skip

    with ThreadPoolExecutor(max(1, threads)) as pool:
        codes = list(pool.map(run, range(len(cuts) - 1)))
    if any(codes):
        msg = f"attn_oracle_f32 failed with codes {codes}"
        raise RuntimeError(msg)
    return out
