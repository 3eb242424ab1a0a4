"""The attention operator of the kernels backend: `softmax(scale * q k^T + bias) v`, head dim 64, fp16 / bf16.

Host side of the path the reference runs through `Flash64._run` (`src/fastforks/kernels/fastbb/__init__.py:124-136`)
and through `F.scaled_dot_product_attention` in its kernels-mode block forwards
(`src/fastforks/_optimize/transformer.py:286-289`, `src/fastforks/promptable_segmentation/models/sam/fused.py:80-86`):
check the launch contract, allocate the output with torch, describe the (possibly strided) views to the C-ABI
library and launch on torch's current stream. Nothing here computes attention: without the CUDA library the call
raises `KernelUnavailableError`.
"""

from __future__ import annotations

import ctypes
import threading
from typing import TYPE_CHECKING

import torch

from . import _lib

if TYPE_CHECKING:
    from collections.abc import Sequence

HEAD_DIM = 64
_DTYPES = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
_BIAS_DTYPES = {**_DTYPES, torch.float32: _lib.F32}
_SCHEDULES = {"auto": _lib.SCHED_AUTO, "long": _lib.SCHED_LONG, "short": _lib.SCHED_SHORT}
LAYOUTS = ("bhnd", "bnhd")


def _strides(t: torch.Tensor, layout: str) -> tuple[int, int, int]:
    """(batch, token, head) element strides of a 4-D view in `layout`."""
    if layout == "bhnd":
        return t.stride(0), t.stride(2), t.stride(1)
    return t.stride(0), t.stride(1), t.stride(2)


def _sizes(t: torch.Tensor, layout: str) -> tuple[int, int, int]:
    """(batch, tokens, heads) of a 4-D view in `layout`."""
    if layout == "bhnd":
        return t.shape[0], t.shape[2], t.shape[1]
    return t.shape[0], t.shape[1], t.shape[2]


def check_operands(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout: str = "bhnd", out: torch.Tensor | None = None
) -> None:
    """Check the launch contract, before anything is launched (the reference's `check_flash64`,
    `src/fastforks/kernels/fastbb/__init__.py:51-67`, widened to bf16 and to both layouts).

    Raises:
        ValueError: A dtype, head dim, shape, device, stride or autograd state the kernels cannot take.
    """
    if layout not in LAYOUTS:
        msg = f"attention: layout {layout!r}: expected one of {LAYOUTS}"
        raise ValueError(msg)
    ts = (("q", q), ("k", k), ("v", v)) + ((("out", out),) if out is not None else ())
    for name, t in ts:
        if (
            t.dtype not in _DTYPES
            or not t.is_cuda
            or t.dim() != 4  # noqa: PLR2004
            or t.shape[-1] != HEAD_DIM
            or t.stride(-1) != 1
        ):
            msg = (
                f"attention: {name} must be a float16 / bfloat16 CUDA 4-D tensor with head dim {HEAD_DIM} and unit "
                f"last stride, got {tuple(t.shape)} {t.dtype} {t.device} strides {t.stride()}"
            )
            raise ValueError(msg)
        if t.dtype != q.dtype or t.device != q.device:
            msg = f"attention: {name} is {t.dtype} on {t.device}, q is {q.dtype} on {q.device}"
            raise ValueError(msg)
        if name != "out" and t.requires_grad and torch.is_grad_enabled():
            msg = f"attention: {name} requires grad; the kernels backend is inference-only (use torch.no_grad())"
            raise ValueError(msg)
    if k.shape != v.shape:
        msg = f"attention: k and v shapes differ: {tuple(k.shape)} vs {tuple(v.shape)}"
        raise ValueError(msg)
    bq, _, hq = _sizes(q, layout)
    bk, _, hk = _sizes(k, layout)
    if (bq, hq) != (bk, hk):
        msg = f"attention: q {tuple(q.shape)} and k / v {tuple(k.shape)} differ in batch or heads"
        raise ValueError(msg)
    if out is not None and out.shape != q.shape:
        msg = f"attention: out shape {tuple(out.shape)} differs from q {tuple(q.shape)}"
        raise ValueError(msg)
    if q.numel() == 0 or k.numel() == 0:
        msg = f"attention: empty operand: q {tuple(q.shape)}, k {tuple(k.shape)}"
        raise ValueError(msg)


def _tile_layout(t: torch.Tensor) -> bool:
    """Whether the kernel can fetch the 4-D bias `t` as tiles: 16-bit, 16-byte aligned base, rows and (where they are
    not broadcast) batch and head strides in multiples of 8 elements."""
    if t.dtype not in (torch.float16, torch.bfloat16) or t.data_ptr() % 16 or t.stride(3) != 1:
        return False
    sb, sh, sn, _ = (0 if extent == 1 else stride for extent, stride in zip(t.shape, t.stride(), strict=True))
    return sn % 8 == 0 and sb % 8 == 0 and sh % 8 == 0 and (sn > 0 or t.shape[2] == 1)


def tile_layout(bias: torch.Tensor) -> torch.Tensor:
    """A 16-bit additive bias `[B | 1, heads | 1, N, Nk]` (fewer leading dims allowed) as a view of the same values
    whose rows begin on 16-byte boundaries: a copy into rows padded to a multiple of 8 columns unless `bias` has that
    layout already.

    The kernel brings such a bias in through the tensor memory accelerator, tile by tile like K and V; any other
    layout is read row by row, several times slower. `attention` makes this copy itself on every call that needs
    it; a caller with a constant bias (a relative-position table per block, a window mask) converts it once.
    """
    t = bias
    while t.dim() < 4:  # noqa: PLR2004
        t = t.unsqueeze(0)
    if t.dtype not in (torch.float16, torch.bfloat16):
        msg = f"tile_layout: a float16 / bfloat16 bias is needed, got {t.dtype}"
        raise ValueError(msg)
    if _tile_layout(t):
        return t
    nk = t.shape[3]
    wide = torch.empty((*t.shape[:3], (nk + 7) // 8 * 8), dtype=t.dtype, device=t.device)
    out = wide[..., :nk]
    out.copy_(t)
    return out


def _bias_view(
    name: str, t: torch.Tensor, shape: Sequence[int], q: torch.Tensor, *, tiled: bool = False
) -> tuple[torch.Tensor, bool]:
    """`t` as a view broadcast to 4-D `shape` with unit last stride, and whether a copy had to be made for it
    (only if its last stride is not 1, its last two dims must be materialised, or, with `tiled`, a 16-bit bias
    does not have the layout of `tile_layout`)."""
    source = t
    if t.dtype not in _BIAS_DTYPES or t.device != q.device:
        msg = f"attention: {name} must be float16 / bfloat16 / float32 on {q.device}, got {t.dtype} on {t.device}"
        raise ValueError(msg)
    if t.dim() > 4:  # noqa: PLR2004
        msg = f"attention: {name} has {t.dim()} dims, at most 4 are allowed"
        raise ValueError(msg)
    while t.dim() < 4:  # noqa: PLR2004
        t = t.unsqueeze(0)
    if t.shape[-1] != shape[-1] or t.shape[-2] != shape[-2]:
        if t.shape[-1] not in (1, shape[-1]) or t.shape[-2] not in (1, shape[-2]):
            msg = f"attention: {name} of shape {tuple(t.shape)} does not broadcast to {tuple(shape)}"
            raise ValueError(msg)
        t = t.expand(t.shape[0], t.shape[1], shape[-2], shape[-1]).contiguous()
    if t.stride(-1) != 1:
        t = t.contiguous()
    if tiled and t.dtype != torch.float32 and not _tile_layout(t):
        t = tile_layout(t)
    copied = t.untyped_storage().data_ptr() != source.untyped_storage().data_ptr()
    try:
        return t.expand(*shape), copied
    except RuntimeError as e:
        msg = f"attention: {name} of shape {tuple(t.shape)} does not broadcast to {tuple(shape)}"
        raise ValueError(msg) from e


# Scratch memory for launches that split long sequences along the keys (include/b200_attn.h: `workspace`), one per
# (device, stream) like the reference's GEMM workspaces (`_PW_WS`, src/fastforks/_optimize/ops.py:248-296): launches
# on one stream run one after the other, launches on different streams never share one. Zeroed when allocated; the
# kernel leaves it ready for the next launch.
_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}
_WORKSPACES_LOCK = threading.Lock()


def reserve_workspace(device: torch.device | int | None = None) -> torch.Tensor:
    """The scratch tensor of the current stream of `device`, allocated and zeroed on first use.

    `attention()` calls this itself. Call it by hand, on the stream a CUDA graph will be captured on, BEFORE the
    capture: nothing is allocated while a stream is capturing, so a capture without a reserved workspace launches
    the unsplit form (same result within rounding, slower where the split pays).
    """
    index = device if isinstance(device, int) else None if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    stream = torch._C._cuda_getCurrentRawStream(index)  # noqa: SLF001
    ws = _WORKSPACES.get((index, stream))
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            return None  # type: ignore[return-value]
        size = ctypes.c_int64(0)
        with torch.cuda.device(index):
            _lib.raise_for_code(_lib.library().b200_attn_workspace_size(ctypes.byref(size)), "attention workspace")
        with _WORKSPACES_LOCK:
            ws = _WORKSPACES.get((index, stream))
            if ws is None:
                ws = _WORKSPACES[(index, stream)] = torch.zeros(size.value, dtype=torch.uint8, device=torch.device("cuda", index))
    return ws


_SPLIT_MIN_KEYS = 257  # the library only ever splits sequences of more than two 128-key tiles


def _attach_workspace(a: _lib.B200AttnArgs, index: int) -> None:
    """Point the launch description at the current stream's workspace (or at none: short sequences, which are
    never split and are the launch-bound ones, and captures without a reserved workspace)."""
    ws = reserve_workspace(index) if a.kv_tokens >= _SPLIT_MIN_KEYS else None
    if ws is None:
        a.workspace, a.workspace_bytes = None, 0
    else:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()


# Launch descriptions already checked once, per thread: geometry key -> (args struct, output shape). A ViT calls the
# operator with the same views in every block and every forward; for launch-bound shapes (one image of 197 tokens) the
# checks and the ctypes set-up of a call cost more than the kernel, so a repeated geometry only has its four
# pointers and the scale filled in again. The key holds everything `check_operands` looks at.
_PREPARED = threading.local()
_PREPARED_LIMIT = 256


def _geometry_key(q, k, v, layout, out, schedule, rel=None, bias=None):  # noqa: ANN001, ANN202, PLR0913
    return (
        q.dtype, k.dtype, v.dtype, q.device, k.device, v.device, layout, schedule, q.shape, k.shape, v.shape,
        q.stride(), k.stride(), v.stride(),
        None if out is None else (out.dtype, out.device, out.shape, out.stride()),
        None if rel is None else tuple((t.dtype, t.device, t.shape, t.stride()) for t in rel),
        None if bias is None else (bias.dtype, bias.device, bias.shape, bias.stride(), bias.data_ptr() % 16),
    )  # fmt: skip


def _launch_prepared(q, k, v, scale, layout, out, schedule, rel=None, bias=None):  # noqa: ANN001, ANN202, PLR0913
    """Launch from a remembered description of this geometry; None when there is none (the full path then runs)."""
    table = getattr(_PREPARED, "table", None)
    if table is None:
        return None
    try:
        entry = table.get(_geometry_key(q, k, v, layout, out, schedule, rel, bias))
    except (AttributeError, TypeError, ValueError):  # not tensors: let the full path raise its ValueError
        return None
    if entry is None:
        return None
    if (q.requires_grad or k.requires_grad or v.requires_grad) and torch.is_grad_enabled():
        return None
    a, o_shape, index = entry
    if index != torch.cuda.current_device():
        return None
    if out is None:
        o = torch.empty(o_shape, device=q.device, dtype=q.dtype)
        out = o.transpose(1, 2) if layout == "bhnd" else o
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    if rel is not None:  # remembered only where the tables went in as they are (broadcast views of the same memory)
        a.rel_h, a.rel_w = rel[0].data_ptr(), rel[1].data_ptr()
    if bias is not None:  # likewise
        a.bias = bias.data_ptr()
    a.scale = float(HEAD_DIM**-0.5 if scale is None else scale)
    _attach_workspace(a, index)
    code = _lib.library().b200_attn_fwd(ctypes.byref(a), torch._C._cuda_getCurrentRawStream(index))  # noqa: SLF001
    if code != _lib.OK:
        _lib.raise_for_code(code, "attention")
    return out


def _remember(a, q, k, v, out, layout, schedule, rel=None, bias=None) -> None:  # noqa: ANN001, PLR0913
    """Keep the checked description `a` of this geometry for the calling thread (`out` as the caller gave it)."""
    index = q.device.index
    if index is None or index != torch.cuda.current_device():
        return
    table = getattr(_PREPARED, "table", None)
    if table is None:
        table = _PREPARED.table = {}
    while len(table) >= _PREPARED_LIMIT:  # the oldest description goes (dicts keep insertion order)
        del table[next(iter(table))]
    copy = _lib.B200AttnArgs.from_buffer_copy(a)
    table[_geometry_key(q, k, v, layout, out, schedule, rel, bias)] = (copy, (a.batch, a.q_tokens, a.heads, HEAD_DIM), index)


def attention(  # noqa: PLR0913
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    scale: float | None = None,
    bias: torch.Tensor | None = None,
    rel: tuple[torch.Tensor, torch.Tensor] | None = None,
    layout: str = "bhnd",
    out: torch.Tensor | None = None,
    schedule: str = "auto",
    _general_merge: bool = False,
    _bias_as_given: bool = False,
) -> torch.Tensor:
    """`softmax(scale * q k^T + bias) v` on the B200 kernels; q, k, v are views, nothing is copied.

    Args:
        q: fp16 / bf16 CUDA `[B, heads, N, 64]` (`layout="bhnd"`, the SDPA layout) or `[B, N, heads, 64]`
            (`layout="bnhd"`, views of a packed qkv tensor); unit last stride, other strides multiples of 8.
        k: Same layout as q, `[.., Nk, ..]`.
        v: Same shape as k.
        scale: Softmax scale; default `64 ** -0.5` as in SDPA and the reference's modules.
        bias: Additive float bias broadcastable to `[B, heads, N, Nk]` (an SDPA float `attn_mask`). A 16-bit bias
            is fetched in tiles; if its rows do not begin on 16-byte boundaries it is first copied into rows that do
            (`tile_layout`: do that once for a constant bias). A float32 bias is read row by row, much slower.
        rel: SAM's decomposed relative-position term `(rel_h [B, heads, N, kh], rel_w [B, heads, N, kw])` with
            `kh * kw == Nk`: `bias[i, j] = rel_h[i, j // kw] + rel_w[i, j % kw]`
            (`src/fastforks/promptable_segmentation/models/sam/net/image_encoder.py:326-362`), never materialised.
        layout: `"bhnd"` or `"bnhd"`.
        out: Optional output view of q's shape and dtype.
        schedule: `"auto"`, `"long"` or `"short"` tile schedule; `"auto"` takes the short one for at most 256 keys whose last
            128-key tile holds at most 96 (e.g. 197 tokens). The result does not depend on it.

    Returns:
        A tensor of q's shape. Without `out` its memory is `[B, N, heads, 64]`-contiguous in both layouts, so the
        `transpose(1, 2).reshape(B, N, C)` that follows SDPA in the reference's block forwards is a free view.

    Raises:
        ValueError: Operands outside the launch contract (checked before the launch).
        KernelUnavailableError: The CUDA library is not built or does not load.
        RuntimeError: A CUDA error at launch.
    """
    if not _general_merge and not _bias_as_given:
        done = _launch_prepared(q, k, v, scale, layout, out, schedule, rel, bias)
        if done is not None:
            return done
    check_operands(q, k, v, layout, out)
    if schedule not in _SCHEDULES:
        msg = f"attention: schedule {schedule!r}: expected one of {tuple(_SCHEDULES)}"
        raise ValueError(msg)
    if bias is not None and rel is not None:
        msg = "attention: bias and rel are mutually exclusive"
        raise ValueError(msg)
    lib = _lib.library()
    b, n, h = _sizes(q, layout)
    _, nk, _ = _sizes(k, layout)
    given_out = out
    if out is None:
        o = torch.empty((b, n, h, HEAD_DIM), device=q.device, dtype=q.dtype)
        out = o.transpose(1, 2) if layout == "bhnd" else o

    a = _lib.B200AttnArgs()
    a.struct_size = ctypes.sizeof(_lib.B200AttnArgs)
    a.dtype = _DTYPES[q.dtype]
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.q_stride[:] = _strides(q, layout)
    a.k_stride[:] = _strides(k, layout)
    a.v_stride[:] = _strides(v, layout)
    a.o_stride[:] = _strides(out, layout)
    a.batch, a.heads, a.q_tokens, a.kv_tokens, a.head_dim = b, h, n, nk, HEAD_DIM
    a.scale = float(HEAD_DIM**-0.5 if scale is None else scale)
    a.schedule = _SCHEDULES[schedule]
    a.test_flags = 1 if _general_merge else 0  # tests only: every merge of a split launch takes its general route
    keep = []  # tensors made here, which the asynchronous launch still reads after this call returns
    if bias is not None:
        given_bias_dtype = bias.dtype
        if bias.dtype == torch.bool:  # SDPA: True = takes part in attention
            bias = torch.zeros_like(bias, dtype=q.dtype).masked_fill_(~bias, float("-inf"))
        made = bias.dtype != given_bias_dtype
        bv, copied = _bias_view("bias", bias, (b, h, n, nk), q, tiled=not _bias_as_given)
        if made or copied:
            keep.append(bv)
        a.bias, a.bias_dtype = bv.data_ptr(), _BIAS_DTYPES[bv.dtype]
        a.bias_stride[:] = bv.stride()[:3]
    if rel is not None:
        rel_h, rel_w = rel
        if rel_h.dim() != 4 or rel_w.dim() != 4 or rel_h.dtype != rel_w.dtype:  # noqa: PLR2004
            msg = "attention: rel_h and rel_w must be 4-D tensors of one dtype"
            raise ValueError(msg)
        kh, kw = rel_h.shape[-1], rel_w.shape[-1]
        if kh * kw != nk:
            msg = f"attention: rel_h / rel_w widths {kh} * {kw} must equal the number of keys {nk}"
            raise ValueError(msg)
        rh, copied_h = _bias_view("rel_h", rel_h, (b, h, n, kh), q)
        rw, copied_w = _bias_view("rel_w", rel_w, (b, h, n, kw), q)
        keep += [t for t, copied in ((rh, copied_h), (rw, copied_w)) if copied]
        a.rel_h, a.rel_w, a.rel_dtype, a.rel_kh, a.rel_kw = rh.data_ptr(), rw.data_ptr(), _BIAS_DTYPES[rh.dtype], kh, kw
        a.rel_h_stride[:] = rh.stride()[:3]
        a.rel_w_stride[:] = rw.stride()[:3]

    index = q.device.index if q.device.index is not None else torch.cuda.current_device()
    if index != torch.cuda.current_device():
        with torch.cuda.device(index):
            _attach_workspace(a, index)
            code = lib.b200_attn_fwd(ctypes.byref(a), torch._C._cuda_getCurrentRawStream(index))  # noqa: SLF001
    else:
        _attach_workspace(a, index)
        code = lib.b200_attn_fwd(ctypes.byref(a), torch._C._cuda_getCurrentRawStream(index))  # noqa: SLF001
    _lib.raise_for_code(code, "attention")
    if not keep and not _general_merge and not _bias_as_given:
        # accepted, and made of the caller's own tensors only: the same geometry can be launched from pointers alone
        _remember(a, q, k, v, given_out, layout, schedule, rel, bias)
    for t in keep:  # the launch is asynchronous: tie temporaries to the stream
        t.record_stream(torch.cuda.current_stream(q.device))
    return out


def device_status(device: torch.device | int | None = None) -> int:
    """Read and clear the device-side error word (synchronises the device). 0 = every kernel ran to the end.

    A non-zero value means a kernel gave up a bounded wait and returned early; its output is invalid.
    """
    word = ctypes.c_uint32(0)
    with torch.cuda.device(device):
        code = _lib.library().b200_attn_status(ctypes.byref(word))
        index = torch.cuda.current_device()
    _lib.raise_for_code(code, "attention status")
    if word.value != 0:  # a launch that gave up may have left flags raised in a workspace: start them from zero again
        for (dev, _), ws in list(_WORKSPACES.items()):
            if dev == index:
                ws.zero_()
    return int(word.value)
