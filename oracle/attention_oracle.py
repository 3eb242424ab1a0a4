"""CPU oracle of the attention path: TEST INFRASTRUCTURE ONLY.

A numpy restatement of the reference's portable (fp32) attention, used as the checker in `tests/`, in
`__graft_entry__.smoke()` and as the timed CPU baseline of `bench.py`. Nothing in the `fastforks_b200` package
imports it, and it is never a fallback for the CUDA path.

Pinned against golden vectors produced by the reference's own modules (`tests/golden/make_golden.py`,
`tests/test_oracle.py`).

What each function follows in the reference:

    attention          DINOv2 `Attention.forward`: q*scale, q k^T, softmax, attn v
                       (src/fastforks/shared/depth_anything_v2/net/dinov2_layers/attention.py:46-60), identical to
                       `F.scaled_dot_product_attention(q, k, v)` in the timm-style `Attention.forward`
                       (src/fastforks/shared/timm_blocks/net/vit.py:44-48) and to the check of the reference's kernel
                       fuzz test (tests/test_kernel_fuzz.py:284-296: fp32 SDPA on the fp16-rounded operands)
    get_rel_pos        src/fastforks/promptable_segmentation/models/sam/net/image_encoder.py:293-323
    decomposed_terms   the two einsums of `add_decomposed_rel_pos` (image_encoder.py:348-355)
    decomposed_bias    the broadcast sum of `add_decomposed_rel_pos` (image_encoder.py:357-360)
"""

from __future__ import annotations

import numpy as np


def attention(q, k, v, scale=None, bias=None, dtype=np.float32):  # noqa: ANN001, ANN201
    """`softmax(scale * q k^T + bias) v` over `[B, H, N, d]` arrays, computed in `dtype` (fp32 like the reference's
    portable backend; pass float64 for spot checks). `bias` broadcasts to `[B, H, Nq, Nk]`."""
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    logits = np.matmul(q * dtype(scale), np.swapaxes(k, -1, -2))
    if bias is not None:
        logits = logits + np.asarray(bias, dtype=dtype)
    logits = logits - logits.max(axis=-1, keepdims=True)
    p = np.exp(logits)
    p /= p.sum(axis=-1, keepdims=True)
    return np.matmul(p, v)


def get_rel_pos(q_size: int, k_size: int, rel_pos):  # noqa: ANN001, ANN201
    """Rows of the relative-position table for every (query, key) coordinate pair: `[q_size, k_size, C]`.

    Only the case the SAM encoder uses is restated: the table already has `2 * max(q_size, k_size) - 1` rows, so the
    reference's linear interpolation branch is not taken.
    """
    rel_pos = np.asarray(rel_pos)
    max_rel_dist = 2 * max(q_size, k_size) - 1
    if rel_pos.shape[0] != max_rel_dist:
        msg = f"table has {rel_pos.shape[0]} rows, {max_rel_dist} expected (interpolation is not restated)"
        raise ValueError(msg)
    q_coords = np.arange(q_size)[:, None] * max(k_size / q_size, 1.0)
    k_coords = np.arange(k_size)[None, :] * max(q_size / k_size, 1.0)
    relative = (q_coords - k_coords) + (k_size - 1) * max(q_size / k_size, 1.0)
    return rel_pos[relative.astype(np.int64)]


def decomposed_terms(q, rel_pos_h, rel_pos_w, hw):  # noqa: ANN001, ANN201
    """`rel_h [B, H, N, kh]`, `rel_w [B, H, N, kw]` from the UNSCALED q `[B, H, N, d]` (N = h * w)."""
    h, w = int(hw[0]), int(hw[1])
    q = np.asarray(q, dtype=np.float32)
    rh = get_rel_pos(h, h, rel_pos_h).astype(np.float32)
    rw = get_rel_pos(w, w, rel_pos_w).astype(np.float32)
    b, nh, n, d = q.shape
    r_q = q.reshape(b, nh, h, w, d)
    rel_h = np.einsum("bnhwc,hkc->bnhwk", r_q, rh).reshape(b, nh, n, h)
    rel_w = np.einsum("bnhwc,wkc->bnhwk", r_q, rw).reshape(b, nh, n, w)
    return rel_h, rel_w


def decomposed_bias(rel_h, rel_w):  # noqa: ANN001, ANN201
    """Dense `[B, H, N, kh * kw]` bias: `bias[.., i, a * kw + c] = rel_h[.., i, a] + rel_w[.., i, c]`."""
    rel_h = np.asarray(rel_h)
    rel_w = np.asarray(rel_w)
    out = rel_h[..., :, None] + rel_w[..., None, :]
    return out.reshape(*rel_h.shape[:-1], rel_h.shape[-1] * rel_w.shape[-1])
