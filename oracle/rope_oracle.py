"""CPU restatement of DINOv3's rotary position embedding as the reference applies it in front of attention.

TEST INFRASTRUCTURE: only `tests/` may import this file; the product never does.

* `rope_table` follows `rope_table` of the reference's portable network
  (`src/fastforks/features/models/dinov3/net.py:99-106`), cut to the half tables the kernels mode keeps
  (`src/fastforks/features/models/dinov3/model.py:185-188`).
* `rope_qk` follows the reference's kernel `rope_qk_h` (`src/fastforks/kernels/fastbb/fastbb_kernels.cu:793-818`):
  fp32 arithmetic on the 16-bit operands, `out[j] = (x[j] c - x[j+32] s) m`, `out[j+32] = (x[j+32] c + x[j] s) m`,
  prefix tokens unrotated (q scaled, k untouched); the caller rounds to the operands' dtype.
* `rope_portable` follows the portable block (`net.py:202-208` with the padded tables of `rope_padded`, `net.py:109-119`):
  `x cos + roll(x, 32) sin'`. Both forms are the same function; the golden vectors come from the second.
"""

from __future__ import annotations

import math

import numpy as np


def rope_table(h: int, w: int, theta: float = 100.0, head_dim: int = 64) -> np.ndarray:
    """fp32 `[h * w, 2, head_dim / 2]` = cos | sin."""
    ch = (np.arange(h, dtype=np.float32) + np.float32(0.5)) / np.float32(h)
    cw = (np.arange(w, dtype=np.float32) + np.float32(0.5)) / np.float32(w)
    yy, xx = np.meshgrid(ch, cw, indexing="ij")
    coords = np.float32(2.0) * np.stack([yy, xx], -1).reshape(-1, 2) - np.float32(1.0)
    inv = (np.float32(1.0) / np.float32(theta) ** np.arange(0, 1, 4 / head_dim, dtype=np.float32)).astype(np.float32)
    ang = (np.float32(2 * math.pi) * coords[:, :, None] * inv[None, None, :]).reshape(coords.shape[0], -1).astype(np.float32)
    return np.stack([np.cos(ang), np.sin(ang)], 1).astype(np.float32)


def rope_qk(q: np.ndarray, k: np.ndarray, cs: np.ndarray, q_scale: float = 1.0) -> tuple[np.ndarray, np.ndarray]:
    """q, k `[B, N, heads, d]` (any float dtype, taken as fp32) -> rotated fp32 copies; the first N - len(cs) tokens
    are the prefix."""
    q = q.astype(np.float32)
    k = k.astype(np.float32)
    n, half = q.shape[1], q.shape[-1] // 2
    prefix = n - cs.shape[0]
    c = cs[:, 0][None, :, None, :]
    s = cs[:, 1][None, :, None, :]

    def rotate(x: np.ndarray, m: np.float32, scale_prefix: bool) -> np.ndarray:
        out = x.copy()
        x1, x2 = x[:, prefix:, :, :half], x[:, prefix:, :, half:]
        out[:, prefix:, :, :half] = (x1 * c - x2 * s) * m
        out[:, prefix:, :, half:] = (x2 * c + x1 * s) * m
        if scale_prefix:
            out[:, :prefix] = x[:, :prefix] * m
        return out

    return rotate(q, np.float32(q_scale), True), rotate(k, np.float32(1.0), False)


def rope_portable(x: np.ndarray, cs: np.ndarray) -> np.ndarray:
    """`x cos + roll(x, d / 2) sin'` with the padded tables (prefix rows cos = 1, sin' = 0); x `[B, heads, N, d]`."""
    x = x.astype(np.float32)
    n, d = x.shape[2], x.shape[3]
    prefix = n - cs.shape[0]
    cos = np.concatenate([np.ones((prefix, d), np.float32), np.tile(cs[:, 0], (1, 2))])
    sin = np.concatenate([np.zeros((prefix, d), np.float32), np.concatenate([-cs[:, 1], cs[:, 1]], 1)])
    return x * cos[None, None] + np.roll(x, d // 2, -1) * sin[None, None]
