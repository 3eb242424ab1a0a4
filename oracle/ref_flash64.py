"""ctypes binding of the reference's own `flash64_*` CUDA kernels: TEST INFRASTRUCTURE ONLY, never imported by the product.

`oracle/_ref/libref_flash64.so` is built by `make -C oracle _ref` from the reference checkout where it lies
(`src/fastforks/kernels/fastbb/fastbb_kernels.cu`, plain sm_100 target as in the reference's `build.toml`) behind
`ref_flash64_launcher.cu`; it is git-ignored and travels to a GPU machine as a built file. `run()` restates the
launch rule of `Flash64._run` (`src/fastforks/kernels/fastbb/__init__.py:124-136`).
"""

from __future__ import annotations

import ctypes
import functools
import math
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SHARED_OBJECT = HERE / "_ref" / "libref_flash64.so"
VARIANTS = {"hh": 0, "fh": 1, "ff": 2}


def build(reference: str | None = None) -> Path | None:
    """Compile the library from the reference checkout at `reference` (default: the environment variable
    `FASTFORKS_REFERENCE`); return its path, or None when there is no checkout and no earlier build exists."""
    import os

    reference = reference or os.environ.get("FASTFORKS_REFERENCE", "")
    src = Path(reference) / "src/fastforks/kernels/fastbb/fastbb_kernels.cu"
    if reference and src.exists():
        subprocess.run(["make", "-C", str(HERE), f"REFERENCE={reference}", "_ref"], check=True, capture_output=True)
    return SHARED_OBJECT if SHARED_OBJECT.exists() else None


def available() -> bool:
    return SHARED_OBJECT.exists()


@functools.cache
def _lib() -> ctypes.CDLL:
    lib = ctypes.CDLL(str(SHARED_OBJECT))
    lib.ref_flash64_launch.argtypes = (
        ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_longlong), ctypes.c_float, ctypes.c_void_p,
    )  # fmt: skip
    lib.ref_flash64_launch.restype = ctypes.c_int
    return lib


def run(variant, q, k, v, scale, out=None):  # noqa: ANN001, ANN201
    """The reference kernel on fp16 `[B, N, heads, 64]` CUDA views, on torch's current stream; returns `[B, N, heads, 64]`."""
    import torch

    b, n, h, d = q.shape
    if out is None:
        out = torch.empty((b, n, h, d), device=q.device, dtype=q.dtype)
    rm = 2 if n * b * h >= 36 * 2 * 128 * 4 else 1
    strides = (ctypes.c_longlong * 12)(*q.stride()[:3], *k.stride()[:3], *v.stride()[:3], *out.stride()[:3])
    stream = torch._C._cuda_getCurrentRawStream(q.device.index)  # noqa: SLF001
    code = _lib().ref_flash64_launch(
        VARIANTS[variant], rm, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), b, n, h, strides,
        float(scale * math.log2(math.e)), stream,
    )  # fmt: skip
    if code != 0:
        msg = f"reference flash64 launch failed with CUDA error {code}"
        raise RuntimeError(msg)
    return out
