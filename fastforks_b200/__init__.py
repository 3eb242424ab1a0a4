"""fastforks_b200: the attention of fastforks' kernels backend, written for B200 (sm_100a).

One operator - non-causal multi-head `softmax(scale * q k^T + bias) v`, head dim 64, fp16 / bf16 - behind the two
interfaces the reference calls it through: `Flash64(variant)(q, k, v, scale)` on `[B, N, heads, 64]` views and
`scaled_dot_product_attention(q, k, v, attn_mask, scale=...)` on `[B, heads, N, 64]` views. The arithmetic runs in
`libb200attn.so` (hand-written tcgen05 / TMA kernels, C ABI in `include/b200_attn.h`); this package holds the host
side only and raises when that library is missing.
"""

from __future__ import annotations

import logging

from . import _lib
from ._lib import build
from .attention import attention, check_operands, device_status, reserve_workspace, tile_layout
from .errors import BackendUnavailableError, KernelUnavailableError
from .graphs import GraphCache
from .gemm import ACT_GELU, ACT_GELU_TANH, ACT_NONE, ACT_RELU, gemm
from .flash64 import FLASH_VARIANTS, Flash64, check_flash64
from .host_io import HostAttention
from .rope import rope_qk_, rope_table
from .sam import sam_rel_terms
from .sdpa import scaled_dot_product_attention

__all__ = [
    "GraphCache",
    "ACT_GELU",
    "ACT_GELU_TANH",
    "ACT_NONE",
    "ACT_RELU",
    "FLASH_VARIANTS",
    "BackendUnavailableError",
    "Flash64",
    "HostAttention",
    "KernelUnavailableError",
    "attention",
    "build",
    "check_flash64",
    "check_operands",
    "device_status",
    "gemm",
    "kernels_unavailable_reason",
    "reserve_workspace",
    "resolve_mode",
    "rope_qk_",
    "rope_table",
    "sam_rel_terms",
    "tile_layout",
    "scaled_dot_product_attention",
    "version",
]

MODES = ("auto", "kernels", "portable")
_log = logging.getLogger(__name__)


def version() -> str:
    """Version string of the loaded kernel library."""
    return _lib.library().b200_attn_version().decode()


def kernels_unavailable_reason(device: object = None) -> str | None:
    """Why the kernels backend cannot run on `device` (default: the current CUDA device), or None if it can."""
    import torch  # noqa: PLC0415

    if not torch.cuda.is_available():
        return "no CUDA device"
    dev = torch.device("cuda" if device is None else device)
    if dev.type != "cuda":
        return f"device {dev} is not a CUDA device"
    cap = torch.cuda.get_device_capability(dev)
    if cap != (10, 0):
        return f"compute capability {cap[0]}.{cap[1]} is not sm_100 (B200)"
    try:
        _lib.library()
    except KernelUnavailableError as e:
        return e.reason
    return None


def resolve_mode(mode: str = "auto", device: object = None) -> str:
    """The backend a model should use: the reference's rule (`src/fastforks/_core/model.py:887-904`).

    `"kernels"` raises where the kernels cannot run, `"auto"` logs the reason and returns `"portable"`,
    `"portable"` is returned unchanged. There is no silent fallback.

    Raises:
        ValueError: Unknown mode.
        BackendUnavailableError: `mode="kernels"` and the kernels cannot run on `device`.
    """
    if mode not in MODES:
        msg = f"mode {mode!r}: expected one of {MODES}"
        raise ValueError(msg)
    if mode == "portable":
        return mode
    reason = kernels_unavailable_reason(device)
    if reason is None:
        return "kernels"
    if mode == "kernels":
        raise BackendUnavailableError(f"kernels backend unavailable: {reason}")
    _log.info("kernels unavailable (%s); using portable", reason)
    return "portable"
