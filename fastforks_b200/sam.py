"""Kernels-mode SAM image encoder (ViT-B: 1024 x 1024 image, 64 x 64 patch grid, 12 blocks) around the attention operator.

The caller side of the hot path for SAM: blocks with 14 x 14 windowed attention (zero-padded windows, 25 of them at
1024 px) and global attention in blocks 2, 5, 8, 11, both with the decomposed relative-position term added to the
logits. Written from the math of the upstream module the reference vendors
(`src/fastforks/promptable_segmentation/models/sam/net/image_encoder.py:17-241, 293-362`): the attention of every
block is this library's kernel with `rel=(rel_h, rel_w)` - q, k, v stay 64 wide views of the packed qkv tensor -
where the reference's kernels mode widens q and k instead (`sam/fast.py:92-113`). Everything else is a plain torch
call. It exists for model-level parity (cosine >= 0.999 against the reference's portable encoder,
`tests/golden/make_golden.py`) and for timing SAM's two attention shapes in place.

Parameter names are the upstream ones, so a state dict of `ImageEncoderViT` loads unchanged.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F  # noqa: N812

from .attention import attention


@dataclass(frozen=True)
class SamConfig:
    img: int = 1024
    patch: int = 16
    dim: int = 768
    depth: int = 12
    heads: int = 12
    out_chans: int = 256
    window: int = 14
    global_blocks: tuple[int, ...] = (2, 5, 8, 11)
    eps: float = 1e-6  # LayerNorm2d of the neck; the blocks' LayerNorm uses torch's default 1e-5

    @property
    def grid(self) -> int:
        return self.img // self.patch


SAM_VIT_B = SamConfig()


def sam_state_shapes(cfg: SamConfig) -> dict[str, tuple[int, ...]]:
    """Parameter names and shapes in the order of upstream `ImageEncoderViT.state_dict()`."""
    d = cfg.dim // cfg.heads
    shapes: dict[str, tuple[int, ...]] = {
        "pos_embed": (1, cfg.grid, cfg.grid, cfg.dim),
        "patch_embed.proj.weight": (cfg.dim, 3, cfg.patch, cfg.patch),
        "patch_embed.proj.bias": (cfg.dim,),
    }
    for i in range(cfg.depth):
        p = f"blocks.{i}."
        side = cfg.grid if i in cfg.global_blocks else cfg.window
        shapes |= {
            p + "norm1.weight": (cfg.dim,), p + "norm1.bias": (cfg.dim,),
            p + "attn.rel_pos_h": (2 * side - 1, d), p + "attn.rel_pos_w": (2 * side - 1, d),
            p + "attn.qkv.weight": (3 * cfg.dim, cfg.dim), p + "attn.qkv.bias": (3 * cfg.dim,),
            p + "attn.proj.weight": (cfg.dim, cfg.dim), p + "attn.proj.bias": (cfg.dim,),
            p + "norm2.weight": (cfg.dim,), p + "norm2.bias": (cfg.dim,),
            p + "mlp.lin1.weight": (4 * cfg.dim, cfg.dim), p + "mlp.lin1.bias": (4 * cfg.dim,),
            p + "mlp.lin2.weight": (cfg.dim, 4 * cfg.dim), p + "mlp.lin2.bias": (cfg.dim,),
        }  # fmt: skip
    shapes |= {
        "neck.0.weight": (cfg.out_chans, cfg.dim, 1, 1),
        "neck.1.weight": (cfg.out_chans,), "neck.1.bias": (cfg.out_chans,),
        "neck.2.weight": (cfg.out_chans, cfg.out_chans, 3, 3),
        "neck.3.weight": (cfg.out_chans,), "neck.3.bias": (cfg.out_chans,),
    }  # fmt: skip
    return shapes


def sam_seeded_state(cfg: SamConfig, seed: int = 0, *, std: float = 0.02, rel_std: float = 0.1) -> dict[str, torch.Tensor]:
    """Random-init weights on the CPU, identical everywhere: matrices ~ N(0, std), biases 0, norm weights 1, and the
    relative-position tables ~ N(0, rel_std) (upstream initialises them to zero, which would leave the bias path
    untested)."""
    gen = torch.Generator().manual_seed(seed)
    state = {}
    for name, shape in sam_state_shapes(cfg).items():
        if "rel_pos" in name:
            t = torch.randn(shape, generator=gen) * rel_std
        elif name.endswith(".bias"):
            t = torch.zeros(shape)
        elif "norm" in name or name in ("neck.1.weight", "neck.3.weight"):
            t = torch.ones(shape)
        else:
            t = torch.randn(shape, generator=gen) * std
        state[name] = t
    return state


def rel_table(size: int, rel_pos: torch.Tensor) -> torch.Tensor:
    """`[size, size, d]`: row (i, j) is `rel_pos[i - j + size - 1]` (upstream `get_rel_pos` with equal query and key
    sizes and a table of `2 * size - 1` rows, the only case the encoder has)."""
    idx = torch.arange(size, device=rel_pos.device)
    return rel_pos[(idx[:, None] - idx[None, :]) + (size - 1)]


def sam_rel_terms(q: torch.Tensor, rel_pos_h: torch.Tensor, rel_pos_w: torch.Tensor, side: int) -> tuple[torch.Tensor, torch.Tensor]:
    """`rel_h`, `rel_w` `[B, heads, N, side]` for `attention(..., rel=)`, on the B200 kernel (`b200_sam_rel_terms`).

    Args:
        q: UNSCALED queries, fp16 / bf16 CUDA `[B, N, heads, 64]` with N = side * side (row-major grid), a strided view
            of the packed qkv tensor is fine (unit last stride, other strides multiples of 8).
        rel_pos_h: The attention module's parameter `[2 * side - 1, 64]`, same dtype and device (made contiguous if not).
        rel_pos_w: Likewise.
        side: Even, at most 64 (14 for SAM's windows, 64 for its global blocks).

    Replaces `get_rel_pos` and the two einsums of the reference's `augmented`
    (`src/fastforks/promptable_segmentation/models/sam/fast.py:104-106`): q is read once, nothing else is materialised.

    Raises:
        ValueError: Operands outside the contract (checked before the launch).
    """
    import ctypes

    from . import _lib

    if q.dim() != 4 or q.shape[-1] != 64 or q.stride(-1) != 1 or not q.is_cuda or q.dtype not in (torch.float16, torch.bfloat16):  # noqa: PLR2004
        msg = f"sam_rel_terms: q must be a float16 / bfloat16 CUDA [B, N, heads, 64] view with unit last stride, got {tuple(q.shape)} {q.dtype} {q.device}"
        raise ValueError(msg)
    b, n, heads, _ = q.shape
    if side % 2 != 0 or not 2 <= side <= 64:  # noqa: PLR2004
        msg = f"sam_rel_terms: side {side} must be even, 2 .. 64"
        raise ValueError(msg)
    if n != side * side:
        msg = f"sam_rel_terms: {n} tokens is not a {side} x {side} grid"
        raise ValueError(msg)
    for name, t in (("rel_pos_h", rel_pos_h), ("rel_pos_w", rel_pos_w)):
        if t.shape != (2 * side - 1, 64) or t.dtype != q.dtype or t.device != q.device:
            msg = f"sam_rel_terms: {name} must be [{2 * side - 1}, 64] {q.dtype} on {q.device}, got {tuple(t.shape)} {t.dtype} {t.device}"
            raise ValueError(msg)
    rel_pos_h, rel_pos_w = rel_pos_h.contiguous(), rel_pos_w.contiguous()
    rel_h = torch.empty(b, heads, n, side, device=q.device, dtype=q.dtype)
    rel_w = torch.empty_like(rel_h)
    a = _lib.B200RelTermsArgs()
    a.struct_size = ctypes.sizeof(_lib.B200RelTermsArgs)
    a.dtype = _lib.F16 if q.dtype == torch.float16 else _lib.BF16
    a.q = q.data_ptr()
    a.q_stride[:] = (q.stride(0), q.stride(1), q.stride(2))
    a.rel_pos_h, a.rel_pos_w, a.rel_h, a.rel_w = rel_pos_h.data_ptr(), rel_pos_w.data_ptr(), rel_h.data_ptr(), rel_w.data_ptr()
    a.batch, a.heads, a.side, a.head_dim = b, heads, side, 64
    with torch.cuda.device(q.device):
        code = _lib.library().b200_sam_rel_terms(ctypes.byref(a), torch._C._cuda_getCurrentRawStream(q.device.index))  # noqa: SLF001
    _lib.raise_for_code(code, "sam_rel_terms")
    return rel_h, rel_w


def rel_terms(q: torch.Tensor, table_h: torch.Tensor, table_w: torch.Tensor, side: int) -> tuple[torch.Tensor, torch.Tensor]:
    """`rel_h`, `rel_w` `[B, heads, N, side]` from the UNSCALED q `[B, N, heads, d]` (N = side * side, row-major) and
    the tables of `rel_table`: `rel_h[b, n, (y, x), k] = q[b, (y, x), n] . table_h[y, k]`, `rel_w` with `table_w[x, k]`
    (the two einsums of upstream `add_decomposed_rel_pos`, image_encoder.py:348-355)."""
    b, n, heads, d = q.shape
    r_q = q.reshape(b, side, side, heads, d)
    rel_h = torch.einsum("byxnc,ykc->bnyxk", r_q, table_h).reshape(b, heads, n, side)
    rel_w = torch.einsum("byxnc,xkc->bnyxk", r_q, table_w).reshape(b, heads, n, side)
    return rel_h, rel_w


class SamEncoder:
    """`images [B, 3, 1024, 1024]` -> `[B, 256, 64, 64]`, every block's attention on the B200 kernels."""

    def __init__(self, cfg: SamConfig, state: dict[str, torch.Tensor], device: torch.device | str = "cuda",
                 dtype: torch.dtype = torch.float16) -> None:  # fmt: skip
        missing = set(sam_state_shapes(cfg)) - set(state)
        if missing:
            msg = f"state dict lacks {sorted(missing)[:4]}..."
            raise ValueError(msg)
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(self.device, dtype) for k, v in state.items()}
        self.tables = {}
        for i in range(cfg.depth):
            side = cfg.grid if i in cfg.global_blocks else cfg.window
            p = f"blocks.{i}.attn."
            self.tables[i] = (rel_table(side, self.w[p + "rel_pos_h"]), rel_table(side, self.w[p + "rel_pos_w"]), side)

    def attend(self, i: int, x: torch.Tensor) -> torch.Tensor:
        """`[B', s, s, C]` (windows or whole grids) -> the same shape: qkv, attention with the bias, projection."""
        w, p = self.w, f"blocks.{i}.attn."
        table_h, table_w, side = self.tables[i]
        b, _, _, c = x.shape
        heads = self.cfg.heads
        qkv = F.linear(x.reshape(b, side * side, c), w[p + "qkv.weight"], w[p + "qkv.bias"]).view(b, side * side, 3, heads, c // heads)
        q, k, v = qkv.unbind(2)  # strided views of the packed tensor
        if q.is_cuda and side % 2 == 0 and side <= 64:  # noqa: PLR2004 - the producer kernel reads q and the parameters in place
            rel = sam_rel_terms(q, w[p + "rel_pos_h"], w[p + "rel_pos_w"], side)
        else:
            rel = rel_terms(q, table_h, table_w, side)
        o = attention(q, k, v, scale=(c // heads) ** -0.5, rel=rel, layout="bnhd")
        return F.linear(o.view(b, side, side, c), w[p + "proj.weight"], w[p + "proj.bias"])

    def block(self, i: int, x: torch.Tensor) -> torch.Tensor:
        w, cfg, p = self.w, self.cfg, f"blocks.{i}."
        b, gh, gw, c = x.shape
        y = F.layer_norm(x, (c,), w[p + "norm1.weight"], w[p + "norm1.bias"])
        if i in cfg.global_blocks:
            y = self.attend(i, y)
        else:
            ws = cfg.window
            ph, pw = (ws - gh % ws) % ws, (ws - gw % ws) % ws
            y = F.pad(y, (0, 0, 0, pw, 0, ph))  # zero tokens, which take part in their window's attention as upstream
            hp, wp = gh + ph, gw + pw
            y = y.view(b, hp // ws, ws, wp // ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(-1, ws, ws, c)
            y = self.attend(i, y)
            y = y.view(b, hp // ws, wp // ws, ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(b, hp, wp, c)[:, :gh, :gw]
        x = x + y
        y = F.layer_norm(x, (c,), w[p + "norm2.weight"], w[p + "norm2.bias"])
        y = F.linear(F.gelu(F.linear(y, w[p + "mlp.lin1.weight"], w[p + "mlp.lin1.bias"])), w[p + "mlp.lin2.weight"], w[p + "mlp.lin2.bias"])
        return x + y

    def norm2d(self, x: torch.Tensor, name: str) -> torch.Tensor:
        """Normalisation over the channels of `[B, C, H, W]` (upstream `LayerNorm2d`)."""
        u = x.mean(1, keepdim=True)
        s = (x - u).pow(2).mean(1, keepdim=True)
        x = (x - u) / torch.sqrt(s + self.cfg.eps)
        return self.w[name + ".weight"][:, None, None] * x + self.w[name + ".bias"][:, None, None]

    @torch.no_grad()
    def __call__(self, images: torch.Tensor) -> torch.Tensor:
        w, cfg = self.w, self.cfg
        x = F.conv2d(images.to(self.device, self.dtype), w["patch_embed.proj.weight"], w["patch_embed.proj.bias"], stride=cfg.patch)
        x = x.permute(0, 2, 3, 1) + w["pos_embed"]
        for i in range(cfg.depth):
            x = self.block(i, x)
        x = F.conv2d(x.permute(0, 3, 1, 2), w["neck.0.weight"])
        x = self.norm2d(x, "neck.1")
        x = F.conv2d(x, w["neck.2.weight"], padding=1)
        return self.norm2d(x, "neck.3")
