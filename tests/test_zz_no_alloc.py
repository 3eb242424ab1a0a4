"""`b200_attn_fwd_static`: the attention call for hosts that cannot allocate device memory where they call it.

Some callers have no allocator at hand when they need attention: a server that gave all device memory to its own
pool at start-up, a pipeline that must not take the device-wide synchronisation of a `cudaMalloc` or `cudaFree`
in its steady state, a C or ctypes program that only holds the pointers of its inputs and outputs. For them the
library carries scratch memory of its own (one array per device, sized for 160 SMs) and this entry point uses it
instead of a caller's workspace. The test calls it through the C ABI exactly as such a host would - inputs and
outputs only - twice in a row (the array keeps the first call's contents: the second call must not trip over
them), on a shape that is split along the keys and so really uses the scratch, and holds the result to the
existing entry point's (same plan, same arithmetic: the bits agree; the bar asserted is the path's tolerance).

The file sorts last on purpose: a run that stops at the first failure has then run every other test already.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from conftest import assert_close
from fastforks_b200 import _lib

pytestmark = pytest.mark.gpu


def describe(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor) -> _lib.B200AttnArgs:
    """The C struct for `[B, N, heads, 64]` tensors: pointers, strides and sizes, nothing else."""
    a = _lib.B200AttnArgs()
    a.struct_size = ctypes.sizeof(_lib.B200AttnArgs)
    a.dtype = _lib.F16 if q.dtype == torch.float16 else _lib.BF16
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    for field, t in ((a.q_stride, q), (a.k_stride, k), (a.v_stride, v), (a.o_stride, out)):
        field[:] = (t.stride(0), t.stride(1), t.stride(2))
    a.batch, a.q_tokens, a.heads = q.shape[0], q.shape[1], q.shape[2]
    a.kv_tokens, a.head_dim, a.scale = k.shape[1], 64, 0.125
    return a


@pytest.mark.parametrize(("b", "h", "n", "dtype"), [(1, 12, 4096, torch.float16), (2, 16, 1370, torch.bfloat16), (2, 3, 197, torch.float16)])
def test_static_scratch_entry_point_matches_the_workspace_entry_point(b: int, h: int, n: int, dtype: torch.dtype) -> None:
    lib = _lib.library()
    stream = ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))  # noqa: SLF001
    gen = torch.Generator().manual_seed(n)
    qkv = torch.randn(b, n, 3, h, 64, generator=gen).to(dtype).cuda()
    q, k, v = qkv.unbind(2)

    # the existing entry point, with a workspace the caller allocated
    size = ctypes.c_int64(0)
    assert lib.b200_attn_workspace_size(ctypes.byref(size)) == 0
    workspace = torch.zeros(size.value, dtype=torch.uint8, device="cuda")
    want = torch.full((b, n, h, 64), float("nan"), dtype=dtype, device="cuda")
    a = describe(q, k, v, want)
    a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    assert lib.b200_attn_fwd(ctypes.byref(a), stream) == 0, _lib.last_error()

    # the new one: inputs and outputs only, twice in a row
    for call in range(2):
        got = torch.full((b, n, h, 64), float("nan"), dtype=dtype, device="cuda")
        assert lib.b200_attn_fwd_static(ctypes.byref(describe(q, k, v, got)), stream) == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert bool(torch.isfinite(got).all()), f"call {call}: rows left unwritten"
        assert_close(got.float().cpu().numpy(), want.float().cpu().numpy(), unit_scale=True, what=f"call {call}")
    word = ctypes.c_uint32(1)
    assert lib.b200_attn_status(ctypes.byref(word)) == 0 and word.value == 0
