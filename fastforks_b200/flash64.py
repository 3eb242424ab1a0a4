"""`Flash64`: the reference's attention launcher, backed by the B200 kernels.

Same contract as `fastforks.kernels.fastbb.Flash64` (`src/fastforks/kernels/fastbb/__init__.py:76-136`):
`Flash64(variant)(q, k, v, scale)` on same-shape `[B, N, heads, 64]` CUDA views with unit last stride returns a new
contiguous `[B, N, heads, 64]` tensor, `ValueError` before the launch on a contract violation, and the static
`_run(variant, q, k, v, scale)` is the single choke point every family launches through
(`tests/test_flash64_guard.py:164-172` in the reference).

Differences, all widening: bf16 is accepted next to fp16, and the variants `"hh"`, `"fh"`, `"ff"` (fp16 or fp32
accumulation of q k^T and p v in the reference) all run the same kernel, because the tcgen05 path always accumulates
both products in fp32 tensor memory. The reference's overflow probe (first 64 launches summed on the device, rerun with
a wider variant after a non-finite sum) therefore has nothing to fall back to and is not run; `probe` is accepted and
kept for signature compatibility.
"""

from __future__ import annotations

import torch

from .attention import HEAD_DIM, attention, check_operands

FLASH_VARIANTS = ("hh", "fh", "ff")
FLASH_PROBE = 64


def check_flash64(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor | None = None) -> None:
    """What `Flash64` accepts, checked before anything is launched: q, k, v (and o, if given) of one shape
    `[B, N, heads, 64]`, fp16 or bf16, on one CUDA device, last dimension contiguous.

    Raises:
        ValueError: An operand breaks one of these rules; the message names it.
    """
    check_operands(q, k, v, "bnhd", o)
    if k.shape != q.shape:
        msg = f"flash64: self-attention only, but q is {tuple(q.shape)} and k / v are {tuple(k.shape)}"
        raise ValueError(msg)


def _known_variant(variant: str) -> str:
    if variant not in FLASH_VARIANTS:
        msg = f"flash64: variant {variant!r} is not one of {', '.join(FLASH_VARIANTS)}"
        raise ValueError(msg)
    return variant


class Flash64:
    """A model's attention launcher with the reference's interface (see the module docstring). The attributes
    `variant`, `probe` and `window` exist because callers and tests of the reference read them; only `variant` is
    ever looked at here, and every variant runs the same kernel."""

    def __init__(self, variant: str = "hh", *, probe: int = FLASH_PROBE) -> None:
        self.variant = _known_variant(variant)
        self.probe = self.window = probe  # no overflow probe is needed with fp32 accumulation; kept for the interface

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        """Attention of strided `[B, N, heads, 64]` views; the result is a new contiguous tensor of that shape."""
        return self._run(self.variant, q, k, v, scale)

    @staticmethod
    def _run(variant: str, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        """The one place a launch happens (the reference's tests replace this method to observe launches)."""
        _known_variant(variant)
        check_flash64(q, k, v)
        b, n, h, _ = q.shape
        o = torch.empty((b, n, h, HEAD_DIM), device=q.device, dtype=q.dtype)
        return attention(q, k, v, scale=scale, layout="bnhd", out=o)
