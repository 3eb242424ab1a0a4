"""The reference's portable attention call, restated with torch on CPU: TEST INFRASTRUCTURE ONLY.

The reference's portable backend computes this path with `F.scaled_dot_product_attention` on fp32 tensors
(`src/fastforks/shared/timm_blocks/net/vit.py:44-48`, `src/fastforks/shared/depth_anything_v2/__init__.py:50-54`,
`src/fastforks/_optimize/transformer.py:257-260`), and SAM's portable path adds the decomposed bias to explicit
logits (`src/fastforks/promptable_segmentation/models/sam/net/image_encoder.py:225-241`). This file restates those
two calls so that `bench.py` can time the reference's CPU arithmetic on the host cores of the GPU machine
(`cpu_baseline`, `--impl reference`); the product never imports it.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F  # noqa: N812


def portable_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    """fp32 CPU `[B, H, N, d]` -> `[B, H, N, d]`, the portable block forwards' SDPA call."""
    return F.scaled_dot_product_attention(q, k, v, scale=scale)


def portable_attention_decomposed(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rel_h: torch.Tensor, rel_w: torch.Tensor, scale: float
) -> torch.Tensor:
    """SAM's portable attention: explicit logits plus `rel_h[..., None] + rel_w[..., None, :]`, softmax, `@ v`."""
    b, h, n, _ = q.shape
    kh, kw = rel_h.shape[-1], rel_w.shape[-1]
    attn = (q * scale) @ k.transpose(-2, -1)
    attn = (attn.view(b, h, n, kh, kw) + rel_h[..., :, None] + rel_w[..., None, :]).view(b, h, n, kh * kw)
    return attn.softmax(dim=-1) @ v
