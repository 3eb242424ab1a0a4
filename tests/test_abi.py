"""The C ABI without a GPU: the library loads, exports every symbol `include/b200_attn.h` declares, the ctypes
mirror of `B200AttnArgs` matches the C struct, and argument checks reject bad calls before any launch
(the reference checks the same way: signatures vs sources in tests/test_kernels.py:112-124, argument rejection
before launch in tests/test_kernels.py:346-392)."""

from __future__ import annotations

import ctypes
import re
import shutil
import subprocess
from pathlib import Path

import pytest

from fastforks_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200_attn.h"


@pytest.fixture(scope="module")
def lib() -> ctypes.CDLL:
    if _lib.needs_build():
        _lib.build()
    _lib.library.cache_clear()
    return _lib.library()


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return re.findall(r"^\s*(?:const\s+)?[\w\*]+\s+\*?\s*(b200_(?:attn|sam|gemm|rope)\w*)\s*\(", text, flags=re.M)


def test_header_declares_the_expected_entry_points() -> None:
    assert sorted(declared_functions()) == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol(lib: ctypes.CDLL) -> None:
    for name in declared_functions():
        assert hasattr(lib, name), name
    assert b"sm_100a" in lib.b200_attn_version()


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_ctypes_struct_matches_the_c_struct(tmp_path: Path) -> None:
    fields = [name for name, *_ in _lib.B200AttnArgs._fields_]  # noqa: SLF001
    src = tmp_path / "layout.c"
    lines = "\n".join(f'  printf("{f} %zu\\n", offsetof(B200AttnArgs, {f}));' for f in fields)
    src.write_text(
        f'#include <stdio.h>\n#include <stddef.h>\n#include "{HEADER}"\n'
        f'int main(void) {{\n  printf("sizeof %zu\\n", sizeof(B200AttnArgs));\n{lines}\n  return 0;\n}}\n'
    )
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-o", str(exe), str(src)], check=True)
    out = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    assert int(out.pop("sizeof")) == ctypes.sizeof(_lib.B200AttnArgs)
    for f in fields:
        assert int(out[f]) == getattr(_lib.B200AttnArgs, f).offset, f


def _args(**kw: object) -> _lib.B200AttnArgs:
    a = _lib.B200AttnArgs()
    a.struct_size = ctypes.sizeof(_lib.B200AttnArgs)
    a.dtype = _lib.F16
    a.q = a.k = a.v = a.o = 0x10000  # only inspected for alignment by b200_attn_query
    for s in (a.q_stride, a.k_stride, a.v_stride, a.o_stride):
        s[:] = (197 * 12 * 64, 12 * 64, 64)
    a.batch, a.heads, a.q_tokens, a.kv_tokens, a.head_dim = 1, 12, 197, 197, 64
    a.scale = 0.125
    for k, v in kw.items():
        if isinstance(v, tuple):
            getattr(a, k)[:] = v
        else:
            setattr(a, k, v)
    return a


def test_query_accepts_the_reference_shapes(lib: ctypes.CDLL) -> None:
    sched = ctypes.c_int32(-1)
    assert lib.b200_attn_query(ctypes.byref(_args()), ctypes.byref(sched)) == _lib.OK
    assert sched.value in (_lib.SCHED_LONG, _lib.SCHED_SHORT)
    packed = (197 * 3 * 12 * 64, 3 * 12 * 64, 64)  # views of packed qkv [B, N, 3, H, 64]
    assert lib.b200_attn_query(ctypes.byref(_args(q_stride=packed, k_stride=packed, v_stride=packed)), None) == _lib.OK
    assert lib.b200_attn_query(ctypes.byref(_args(dtype=_lib.BF16, q_tokens=4096, kv_tokens=4096)), None) == _lib.OK


@pytest.mark.parametrize(
    ("kw", "code", "word"),
    [
        ({"struct_size": 8}, _lib.BAD_CONFIG, "struct_size"),
        ({"dtype": 7}, _lib.BAD_CONFIG, "dtype"),
        ({"head_dim": 128}, _lib.UNSUPPORTED, "head dim"),
        ({"q_tokens": 0}, _lib.UNSUPPORTED, "empty"),
        ({"kv_tokens": 0}, _lib.UNSUPPORTED, "empty"),
        ({"scale": 0.0}, _lib.UNSUPPORTED, "scale"),
        ({"scale": float("nan")}, _lib.UNSUPPORTED, "scale"),
        ({"q": 0}, _lib.BAD_CONFIG, "NULL"),
        ({"k": 0x10008}, _lib.UNSUPPORTED, "aligned"),
        ({"v_stride": (197 * 12 * 64, 12 * 64 + 4, 64)}, _lib.UNSUPPORTED, "multiple of 8"),
        ({"bias": 0x10000, "rel_h": 0x10000, "rel_w": 0x10000}, _lib.BAD_CONFIG, "exclusive"),
        ({"rel_h": 0x10000}, _lib.BAD_CONFIG, "together"),
        ({"rel_h": 0x10000, "rel_w": 0x10000, "rel_kh": 14, "rel_kw": 13}, _lib.UNSUPPORTED, "kv_tokens"),
        ({"bias": 0x10000, "bias_dtype": 9}, _lib.BAD_CONFIG, "bias_dtype"),
        ({"schedule": 5}, _lib.BAD_CONFIG, "schedule"),
    ],
)
def test_query_rejects_before_launch(lib: ctypes.CDLL, kw: dict, code: int, word: str) -> None:
    assert lib.b200_attn_query(ctypes.byref(_args(**kw)), None) == code
    assert word in lib.b200_attn_last_error().decode()


def test_fwd_rejects_bad_arguments_without_a_gpu(lib: ctypes.CDLL) -> None:
    """`b200_attn_fwd` runs the same checks first, so a bad call returns before touching the CUDA runtime."""
    assert lib.b200_attn_fwd(ctypes.byref(_args(head_dim=32)), None) == _lib.UNSUPPORTED
    assert lib.b200_attn_fwd(None, None) == _lib.BAD_CONFIG


def test_return_codes_map_to_the_reference_exceptions(lib: ctypes.CDLL) -> None:
    lib.b200_attn_query(ctypes.byref(_args(head_dim=32)), None)
    with pytest.raises(ValueError, match="head dim"):
        _lib.raise_for_code(_lib.UNSUPPORTED, "attention")
    with pytest.raises(RuntimeError):
        _lib.raise_for_code(_lib.CUDA_ERROR_BASE + 2, "attention")
    _lib.raise_for_code(_lib.OK, "attention")
