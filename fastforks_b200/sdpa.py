"""Drop-in for the `F.scaled_dot_product_attention` calls of the reference's kernels-mode block forwards.

Call sites it replaces: `_vit_kernels` (`src/fastforks/_optimize/transformer.py:286-289`), `_swin_block` with a dense
additive bias (`:476-479`), the DINOv2 `_sdpa_forward` (`src/fastforks/shared/depth_anything_v2/__init__.py:50-54`)
and SAM's `attention` (`src/fastforks/promptable_segmentation/models/sam/fast.py:128-135`), which here takes the
decomposed relative-position term directly instead of widening q and k.
"""

from __future__ import annotations

import torch

from .attention import attention


def scaled_dot_product_attention(  # noqa: PLR0913
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_mask: torch.Tensor | None = None,
    dropout_p: float = 0.0,
    is_causal: bool = False,  # noqa: FBT001, FBT002 - torch's signature
    scale: float | None = None,
    *,
    rel: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> torch.Tensor:
    """`softmax(scale * q k^T + attn_mask) v` on `[B, heads, N, 64]` views, torch's signature plus `rel`.

    `rel=(rel_h, rel_w)` is SAM's decomposed bias (see `attention`). The result has shape `[B, heads, N, 64]` and
    `[B, N, heads, 64]`-contiguous memory.

    Raises:
        ValueError: Operands outside the launch contract; dropout or a causal mask, which this inference path of the
            reference never uses (`dropout_p=0`, `is_causal=False` at every call site).
    """
    if dropout_p != 0.0:
        msg = "scaled_dot_product_attention: the kernels backend is inference-only, dropout_p must be 0"
        raise ValueError(msg)
    if is_causal:
        msg = "scaled_dot_product_attention: causal attention is not part of this path (ViT encoders are non-causal)"
        raise ValueError(msg)
    return attention(query, key, value, scale=scale, bias=attn_mask, rel=rel, layout="bhnd")
