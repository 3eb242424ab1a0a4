"""DINOv3's rotary position embedding on the q and k views of a packed qkv tensor, the step in front of the attention
call in the reference's kernels-mode DINOv3 block (`src/fastforks/features/models/dinov3/model.py:199-201`).

`rope_table` builds the table the reference keeps per patch grid (`rope_table`, `dinov3/net.py:99-106`, in the layout of
`model.py:185-188`); `rope_qk_` rotates q and k in place on the B200 kernel (`b200_rope_qk`), which stands where the
reference launches `rope_qk_h` (`src/fastforks/kernels/fastbb/fastbb_kernels.cu:793-818`).
"""

from __future__ import annotations

import ctypes
import math

import torch

from . import _lib

HEAD_DIM = 64


def rope_table(h: int, w: int, theta: float = 100.0, device: torch.device | str | None = None) -> torch.Tensor:
    """fp32 `[h * w, 2, 32]` = cos | sin of an `h x w` patch grid (head dim 64; dims j and j + 32 share an angle).

    Patch centres in [-1, 1] per axis, sixteen frequencies `theta ** -(4 i / 64)` per axis, angle = 2 pi * coordinate *
    frequency, the y angles first, then the x angles.
    """
    ch = torch.arange(0.5, h, dtype=torch.float32, device=device) / h
    cw = torch.arange(0.5, w, dtype=torch.float32, device=device) / w
    coords = 2.0 * torch.stack(torch.meshgrid(ch, cw, indexing="ij"), -1).flatten(0, 1) - 1.0
    inv = 1 / theta ** torch.arange(0, 1, 4 / HEAD_DIM, dtype=torch.float32, device=device)
    ang = (2 * math.pi * coords[:, :, None] * inv[None, None, :]).flatten(1, 2)  # [h * w, 32]
    return torch.stack((ang.cos(), ang.sin()), 1).contiguous()


def rope_qk_(qkv: torch.Tensor, cs: torch.Tensor, *, q_scale: float = 1.0) -> torch.Tensor:
    """Rotate q and k of the packed `qkv` `[B, N, 3, heads, 64]` in place and return `qkv`.

    Args:
        qkv: fp16 / bf16 CUDA tensor, unit last stride, other strides multiples of 8 (a contiguous qkv GEMM output).
        cs: `rope_table` of the patch grid, fp32 `[P, 2, 32]` on the same device; the first `N - P` tokens (class token
            and registers) are not rotated.
        q_scale: Factor applied to every q (the reference passes `64 ** -0.5` and calls attention with scale 1).

    Raises:
        ValueError: Operands outside the contract (checked before the launch).
    """
    if qkv.dim() != 5 or qkv.shape[2] != 3 or qkv.shape[-1] != HEAD_DIM or not qkv.is_cuda or qkv.dtype not in (torch.float16, torch.bfloat16):  # noqa: PLR2004
        msg = f"rope_qk_: qkv must be a float16 / bfloat16 CUDA [B, N, 3, heads, 64] tensor, got {tuple(qkv.shape)} {qkv.dtype} {qkv.device}"
        raise ValueError(msg)
    if qkv.stride(-1) != 1:
        msg = "rope_qk_: qkv must have unit last stride"
        raise ValueError(msg)
    b, n, _, heads, _ = qkv.shape
    if cs.dim() != 3 or cs.shape[1:] != (2, HEAD_DIM // 2) or cs.dtype != torch.float32 or cs.device != qkv.device or cs.shape[0] > n:  # noqa: PLR2004
        msg = f"rope_qk_: cs must be float32 [P <= {n}, 2, 32] on {qkv.device}, got {tuple(cs.shape)} {cs.dtype} {cs.device}"
        raise ValueError(msg)
    if qkv.requires_grad and torch.is_grad_enabled():
        msg = "rope_qk_: the kernels have no backward; qkv requires grad"
        raise ValueError(msg)
    cs = cs.contiguous()
    q, k = qkv[:, :, 0], qkv[:, :, 1]
    a = _lib.B200RopeArgs()
    a.struct_size = ctypes.sizeof(_lib.B200RopeArgs)
    a.dtype = _lib.F16 if qkv.dtype == torch.float16 else _lib.BF16
    a.q, a.k, a.cs = q.data_ptr(), k.data_ptr(), cs.data_ptr()
    a.q_stride[:] = (q.stride(0), q.stride(1), q.stride(2))
    a.k_stride[:] = (k.stride(0), k.stride(1), k.stride(2))
    a.batch, a.heads, a.tokens, a.prefix, a.head_dim = b, heads, n, n - cs.shape[0], HEAD_DIM
    a.q_scale = float(q_scale)
    with torch.cuda.device(qkv.device):
        code = _lib.library().b200_rope_qk(ctypes.byref(a), torch._C._cuda_getCurrentRawStream(qkv.device.index))  # noqa: SLF001
    _lib.raise_for_code(code, "rope_qk_")
    return qkv
