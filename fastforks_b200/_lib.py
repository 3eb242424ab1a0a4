"""Loader and in-tree build of `libb200attn.so`, the C-ABI attention library declared in `include/b200_attn.h`.

The library is loaded with ctypes, the way the reference loads its `shared`-kind kernel libraries
(`src/fastforks/_core/kernels.py:481-494`): plain pointers and sizes go in, a status code comes back, and the
launch goes to torch's current raw stream (`src/fastforks/_core/kernels.py:426-428`).
"""

from __future__ import annotations

import ctypes
import functools
import hashlib
import os
import re
import shutil
import subprocess
import threading
from pathlib import Path

from .errors import KernelUnavailableError

LIBRARY = "b200attn"
PACKAGE_DIR = Path(__file__).resolve().parent
SOURCE = PACKAGE_DIR / "csrc" / "b200_attn.cu"
HEADERS = (
    PACKAGE_DIR / "csrc" / "sm100_ptx.cuh",
    PACKAGE_DIR / "csrc" / "attn_fwd_sm100.cuh",
    PACKAGE_DIR / "csrc" / "sam_rel_terms.cuh",
    PACKAGE_DIR / "csrc" / "rope_sm100.cuh",
    PACKAGE_DIR / "csrc" / "gemm_sm100.cuh",
    PACKAGE_DIR.parent / "include" / "b200_attn.h",
)
SHARED_OBJECT = PACKAGE_DIR / "libb200attn.so"

# sm_100a only: the kernels use tcgen05 / TMEM / TMA, which exist in no other target.
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-shared", "-Xcompiler", "-fPIC",
)  # fmt: skip

# Every symbol include/b200_attn.h declares.
EXPORTS = (
    "b200_attn_fwd", "b200_attn_fwd_static", "b200_gemm", "b200_sam_rel_terms", "b200_rope_qk", "b200_attn_query", "b200_attn_plan", "b200_attn_workspace_size", "b200_attn_status",
    "b200_attn_selftest_wait_limit", "b200_attn_last_error", "b200_attn_version",
)  # fmt: skip

OK, UNSUPPORTED, BAD_CONFIG, CUDA_ERROR_BASE = 0, 1, -1, 1000
F16, BF16, F32 = 0, 1, 2
SCHED_AUTO, SCHED_LONG, SCHED_SHORT = 0, 1, 2


class B200AttnArgs(ctypes.Structure):
    """Mirror of `struct B200AttnArgs` (include/b200_attn.h)."""

    _fields_ = (
        ("struct_size", ctypes.c_uint32),
        ("dtype", ctypes.c_uint32),
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p),
        ("q_stride", ctypes.c_int64 * 3),
        ("k_stride", ctypes.c_int64 * 3),
        ("v_stride", ctypes.c_int64 * 3),
        ("o_stride", ctypes.c_int64 * 3),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("q_tokens", ctypes.c_int32),
        ("kv_tokens", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("bias", ctypes.c_void_p),
        ("bias_dtype", ctypes.c_uint32),
        ("bias_stride", ctypes.c_int64 * 3),
        ("rel_h", ctypes.c_void_p),
        ("rel_w", ctypes.c_void_p),
        ("rel_dtype", ctypes.c_uint32),
        ("rel_kh", ctypes.c_int32),
        ("rel_kw", ctypes.c_int32),
        ("rel_h_stride", ctypes.c_int64 * 3),
        ("rel_w_stride", ctypes.c_int64 * 3),
        ("schedule", ctypes.c_int32),
        ("test_flags", ctypes.c_int32),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_int64),
    )


class B200GemmArgs(ctypes.Structure):
    """Mirror of `struct B200GemmArgs` (include/b200_attn.h)."""

    _fields_ = (
        ("struct_size", ctypes.c_uint32),
        ("dtype", ctypes.c_uint32),
        ("m", ctypes.c_int32),
        ("n", ctypes.c_int32),
        ("k", ctypes.c_int32),
        ("act", ctypes.c_int32),
        ("x", ctypes.c_void_p),
        ("lda", ctypes.c_int64),
        ("w", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("scale", ctypes.c_void_p),
        ("res", ctypes.c_void_p),
        ("lres", ctypes.c_int64),
        ("y", ctypes.c_void_p),
        ("ldy", ctypes.c_int64),
    )


class B200RelTermsArgs(ctypes.Structure):
    """Mirror of `struct B200RelTermsArgs` (include/b200_attn.h)."""

    _fields_ = (
        ("struct_size", ctypes.c_uint32),
        ("dtype", ctypes.c_uint32),
        ("q", ctypes.c_void_p),
        ("q_stride", ctypes.c_int64 * 3),
        ("rel_pos_h", ctypes.c_void_p),
        ("rel_pos_w", ctypes.c_void_p),
        ("rel_h", ctypes.c_void_p),
        ("rel_w", ctypes.c_void_p),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("side", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
    )


class B200RopeArgs(ctypes.Structure):
    """Mirror of `struct B200RopeArgs` (include/b200_attn.h)."""

    _fields_ = (
        ("struct_size", ctypes.c_uint32),
        ("dtype", ctypes.c_uint32),
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("q_stride", ctypes.c_int64 * 3),
        ("k_stride", ctypes.c_int64 * 3),
        ("cs", ctypes.c_void_p),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("tokens", ctypes.c_int32),
        ("prefix", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("q_scale", ctypes.c_float),
    )


def source_hash() -> str:
    """Digest of the sources the shared object is compiled from (16 hex digits). The build passes it to the compiler,
    which puts it into the library's version string, so a binary can be matched with the sources beside it."""
    digest = hashlib.sha256()
    for path in sorted((SOURCE, *HEADERS), key=lambda f: f.name):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()[:16]


_HASH_IN_BINARY = re.compile(rb"b200attn-src:([0-9a-f]{16})")


def built_hash() -> str | None:
    """The source digest compiled into the shared object on disk (read from the file, without loading it), or None."""
    if not SHARED_OBJECT.exists():
        return None
    found = _HASH_IN_BINARY.search(SHARED_OBJECT.read_bytes())
    return found.group(1).decode() if found else None


def needs_build() -> bool:
    """True when the shared object is missing or was compiled from other sources than the ones beside it."""
    return built_hash() != source_hash()


def build(*, force: bool = False, verbose: bool = False) -> Path:
    """Compile `csrc/b200_attn.cu` for sm_100a into `libb200attn.so` next to this file (needs nvcc, no GPU).

    Raises:
        KernelUnavailableError: nvcc is missing or the compilation failed.
    """
    if not force and not needs_build():
        return SHARED_OBJECT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise KernelUnavailableError(LIBRARY, "nvcc not found: cannot build libb200attn.so")
    tmp = SHARED_OBJECT.with_suffix(f".{os.getpid()}.tmp.so")
    cmd = [nvcc, *NVCC_FLAGS, f'-DB200_SOURCE_HASH="{source_hash()}"', *(("-Xptxas", "-v") if verbose else ()),
           "-o", str(tmp), str(SOURCE)]  # fmt: skip
    proc = subprocess.run(cmd, capture_output=True, text=True, check=False)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelUnavailableError(LIBRARY, f"nvcc failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    tmp.replace(SHARED_OBJECT)
    return SHARED_OBJECT


_LOCK = threading.Lock()


@functools.cache
def library() -> ctypes.CDLL:
    """The loaded `libb200attn.so` with argument types set.

    Raises:
        KernelUnavailableError: The shared object is not built or does not load (the message says which).
    """
    if needs_build():
        # A binary of other sources must never answer for these, and nothing is built behind the caller's back.
        state = "is not built" if not SHARED_OBJECT.exists() else "was built from other sources than the ones beside it"
        how = "run `python -c 'import fastforks_b200; fastforks_b200.build()'`"
        raise KernelUnavailableError(LIBRARY, f"{SHARED_OBJECT.name} {state}; {how}")
    try:
        lib = ctypes.CDLL(str(SHARED_OBJECT))
    except OSError as e:
        raise KernelUnavailableError(LIBRARY, f"cannot load {SHARED_OBJECT.name}: {e}") from e
    missing = [name for name in EXPORTS if not hasattr(lib, name)]
    if missing:
        raise KernelUnavailableError(LIBRARY, f"{SHARED_OBJECT.name} lacks the symbols {missing}")
    lib.b200_attn_fwd.argtypes = (ctypes.POINTER(B200AttnArgs), ctypes.c_void_p)
    lib.b200_attn_fwd.restype = ctypes.c_int
    lib.b200_attn_fwd_static.argtypes = (ctypes.POINTER(B200AttnArgs), ctypes.c_void_p)
    lib.b200_attn_fwd_static.restype = ctypes.c_int
    lib.b200_gemm.argtypes = (ctypes.POINTER(B200GemmArgs), ctypes.c_void_p)
    lib.b200_gemm.restype = ctypes.c_int
    lib.b200_sam_rel_terms.argtypes = (ctypes.POINTER(B200RelTermsArgs), ctypes.c_void_p)
    lib.b200_sam_rel_terms.restype = ctypes.c_int
    lib.b200_rope_qk.argtypes = (ctypes.POINTER(B200RopeArgs), ctypes.c_void_p)
    lib.b200_rope_qk.restype = ctypes.c_int
    lib.b200_attn_query.argtypes = (ctypes.POINTER(B200AttnArgs), ctypes.POINTER(ctypes.c_int32))
    lib.b200_attn_query.restype = ctypes.c_int
    i32p = ctypes.POINTER(ctypes.c_int32)
    lib.b200_attn_plan.argtypes = (ctypes.POINTER(B200AttnArgs), ctypes.c_int32, ctypes.c_int32, i32p, i32p, ctypes.c_int32, i32p, i32p)
    lib.b200_attn_plan.restype = ctypes.c_int
    lib.b200_attn_workspace_size.argtypes = (ctypes.POINTER(ctypes.c_int64),)
    lib.b200_attn_workspace_size.restype = ctypes.c_int
    lib.b200_attn_status.argtypes = (ctypes.POINTER(ctypes.c_uint32),)
    lib.b200_attn_status.restype = ctypes.c_int
    lib.b200_attn_selftest_wait_limit.argtypes = (ctypes.c_uint32, ctypes.c_void_p)
    lib.b200_attn_selftest_wait_limit.restype = ctypes.c_int
    lib.b200_attn_last_error.argtypes = ()
    lib.b200_attn_last_error.restype = ctypes.c_char_p
    lib.b200_attn_version.argtypes = ()
    lib.b200_attn_version.restype = ctypes.c_char_p
    return lib


def last_error() -> str:
    """Reason of the calling thread's last non-zero return code."""
    return library().b200_attn_last_error().decode()


def raise_for_code(code: int, what: str) -> None:
    """Map a non-zero return code to the exception the reference raises for it.

    `ValueError` for geometry / configuration the kernels cannot take, `RuntimeError` for CUDA errors
    (`src/fastforks/kernels/dpt_fused/__init__.py:101-106`).
    """
    if code == OK:
        return
    msg = f"{what}: {last_error()} (code {code})"
    if code in (UNSUPPORTED, BAD_CONFIG):
        raise ValueError(msg)
    raise RuntimeError(msg)
