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
    """Check the launch contract: same-shape fp16 / bf16 CUDA `[B, N, heads, 64]` views with unit last stride.

    Raises:
        ValueError: A dtype, head dim, shape, device or stride the kernel cannot read.
    """
    check_operands(q, k, v, "bnhd", o)
    if k.shape != q.shape:
        msg = f"flash64: q, k, v, o shapes differ: {[tuple(t.shape) for t in (q, k, v)]}"
        raise ValueError(msg)


class Flash64:
    """Attention of one model over `[B, N, heads, 64]` views (see the module docstring)."""

    def __init__(self, variant: str = "hh", *, probe: int = FLASH_PROBE) -> None:
        """`variant`: one of `FLASH_VARIANTS`; `probe`: kept for compatibility, nothing is probed."""
        if variant not in FLASH_VARIANTS:
            msg = f"flash64 variant {variant!r}: expected one of {FLASH_VARIANTS}"
            raise ValueError(msg)
        self.variant, self.probe, self.window = variant, probe, probe

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        """softmax(q k^T * scale) v of `[B, N, heads, 64]` views (unit last stride) -> new `[B, N, heads, 64]`."""
        return self._run(self.variant, q, k, v, scale)

    @staticmethod
    def _run(variant: str, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        if variant not in FLASH_VARIANTS:
            msg = f"flash64 variant {variant!r}: expected one of {FLASH_VARIANTS}"
            raise ValueError(msg)
        check_flash64(q, k, v)
        b, n, h, _ = q.shape
        o = torch.empty((b, n, h, HEAD_DIM), device=q.device, dtype=q.dtype)
        return attention(q, k, v, scale=scale, layout="bnhd", out=o)
