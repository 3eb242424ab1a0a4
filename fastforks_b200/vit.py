"""Kernels-mode ViT encoder around the attention operator: the caller side of the hot path.

A restatement of the reference's kernels-mode DINOv2 forward (`FastViT.tokens` / `FastViT.block`,
`src/fastforks/shared/depth_anything_v2/fast_vit.py:131-180`) as a thin harness: packed qkv GEMM, attention on
strided `[B, N, heads, 64]` views of it through `Flash64`, projection with LayerScale and residual, MLP or fused
SwiGLU. Every non-attention op is a plain torch call (cuBLAS GEMMs, LayerNorm, GELU); the attention is the B200
kernel. It exists to measure whole-model throughput and to check model-level parity (cosine >= 0.999 against the
reference's portable network, `tests/golden/make_golden.py`), not to replace the reference's model zoo.

Parameter names follow the reference's vendored DINOv2 (`net/dinov2.py`), so a state dict of that network loads here
unchanged; `seeded_state` builds the random-init weights the benchmark configurations ask for.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F  # noqa: N812

from .flash64 import Flash64


@dataclass(frozen=True)
class ViTConfig:
    """Geometry of one encoder (names as in the reference's `DinoVisionTransformer`)."""

    dim: int
    depth: int
    heads: int
    patch: int
    img: int  # side of the image the position table was made for
    ffn: str = "mlp"  # "mlp" (fc1, GELU, fc2) or "swiglu" (fused w12, w3), as `vit_giant2`
    layerscale: bool = True
    interpolate_offset: float = 0.1
    eps: float = 1e-6

    @property
    def hidden(self) -> int:
        if self.ffn == "swiglu":  # `SwiGLUFFNFused`: 2/3 of 4x, rounded up to a multiple of 8
            return (int(self.dim * 4 * 2 / 3) + 7) // 8 * 8
        return self.dim * 4

    def tokens(self, height: int, width: int) -> int:
        return 1 + (height // self.patch) * (width // self.patch)


CONFIGS = {
    # DINOv2 / Depth-Anything-V2 encoders (`DINOv2(model_name)`, net/dinov2.py:425-442): patch 14, table for 518 px
    "dinov2-vits14": ViTConfig(384, 12, 6, 14, 518),
    "dinov2-vitb14": ViTConfig(768, 12, 12, 14, 518),
    "dinov2-vitl14": ViTConfig(1024, 24, 16, 14, 518),
    "dinov2-vitg14": ViTConfig(1536, 40, 24, 14, 518, ffn="swiglu"),
    # timm ViT-B/16 (`_VIT`, src/fastforks/shared/timm_blocks/net/vit.py:69-85): no LayerScale
    "vit-b16": ViTConfig(768, 12, 12, 16, 224, layerscale=False, interpolate_offset=0.0),
}


def state_shapes(cfg: ViTConfig) -> dict[str, tuple[int, ...]]:
    """Parameter names and shapes, in the order of the reference network's `state_dict()`."""
    grid = cfg.img // cfg.patch
    shapes: dict[str, tuple[int, ...]] = {
        "cls_token": (1, 1, cfg.dim),
        "pos_embed": (1, 1 + grid * grid, cfg.dim),
        "mask_token": (1, cfg.dim),
        "patch_embed.proj.weight": (cfg.dim, 3, cfg.patch, cfg.patch),
        "patch_embed.proj.bias": (cfg.dim,),
    }
    for i in range(cfg.depth):
        p = f"blocks.{i}."
        shapes |= {
            p + "norm1.weight": (cfg.dim,), p + "norm1.bias": (cfg.dim,),
            p + "attn.qkv.weight": (3 * cfg.dim, cfg.dim), p + "attn.qkv.bias": (3 * cfg.dim,),
            p + "attn.proj.weight": (cfg.dim, cfg.dim), p + "attn.proj.bias": (cfg.dim,),
        }  # fmt: skip
        if cfg.layerscale:
            shapes[p + "ls1.gamma"] = (cfg.dim,)
        shapes |= {p + "norm2.weight": (cfg.dim,), p + "norm2.bias": (cfg.dim,)}
        if cfg.ffn == "swiglu":
            shapes |= {
                p + "mlp.w12.weight": (2 * cfg.hidden, cfg.dim), p + "mlp.w12.bias": (2 * cfg.hidden,),
                p + "mlp.w3.weight": (cfg.dim, cfg.hidden), p + "mlp.w3.bias": (cfg.dim,),
            }  # fmt: skip
        else:
            shapes |= {
                p + "mlp.fc1.weight": (cfg.hidden, cfg.dim), p + "mlp.fc1.bias": (cfg.hidden,),
                p + "mlp.fc2.weight": (cfg.dim, cfg.hidden), p + "mlp.fc2.bias": (cfg.dim,),
            }  # fmt: skip
        if cfg.layerscale:
            shapes[p + "ls2.gamma"] = (cfg.dim,)
    shapes |= {"norm.weight": (cfg.dim,), "norm.bias": (cfg.dim,)}
    return shapes


def seeded_state(cfg: ViTConfig, seed: int = 0, *, std: float = 0.02, qk_gain: float = 1.0) -> dict[str, torch.Tensor]:
    """Random-init weights on the CPU, identical on every machine and rank: matrices and tokens ~ N(0, std),
    biases 0, LayerNorm weight 1, LayerScale gamma 1. `qk_gain` scales the q and k rows of every qkv matrix
    (sharper attention than the near-uniform one that std 0.02 gives)."""
    gen = torch.Generator().manual_seed(seed)
    state = {}
    for name, shape in state_shapes(cfg).items():
        if name.endswith((".bias",)):
            t = torch.zeros(shape)
        elif "norm" in name or name.endswith(".gamma"):
            t = torch.ones(shape)
        else:
            t = torch.randn(shape, generator=gen) * std
            if name.endswith("attn.qkv.weight"):
                t[: 2 * cfg.dim] *= qk_gain
        state[name] = t
    return state


class ViTEncoder:
    """`images [B, 3, H, W]` -> normalised tokens `[B, N, dim]`, every block's attention on the B200 kernels."""

    def __init__(self, cfg: ViTConfig, state: dict[str, torch.Tensor], device: torch.device | str = "cuda",
                 dtype: torch.dtype = torch.float16, variant: str = "hh") -> None:  # fmt: skip
        missing = set(state_shapes(cfg)) - set(state)
        if missing:
            msg = f"state dict lacks {sorted(missing)[:4]}..."
            raise ValueError(msg)
        if cfg.dim // cfg.heads != 64:  # noqa: PLR2004
            msg = f"head dim {cfg.dim // cfg.heads}: the kernels backend is built for head dim 64"
            raise ValueError(msg)
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(self.device, dtype) for k, v in state.items()}
        self.pos_table = state["pos_embed"].to(self.device, torch.float32)  # interpolated in fp32, as upstream
        self.attn = Flash64(variant)
        self._pos: dict[tuple[int, int], torch.Tensor] = {}

    def pos_embed(self, gh: int, gw: int) -> torch.Tensor:
        """Position table for a `gh x gw` patch grid (upstream `interpolate_pos_encoding`, net/dinov2.py:198-237)."""
        key = (gh, gw)
        if key not in self._pos:
            table = self.pos_table
            n = table.shape[1] - 1
            side = int(math.sqrt(n))
            if gh * gw == n and gh == gw:
                pos = table
            else:
                off = self.cfg.interpolate_offset
                grid = table[:, 1:].reshape(1, side, side, -1).permute(0, 3, 1, 2)
                grid = F.interpolate(grid, scale_factor=((gh + off) / side, (gw + off) / side), mode="bicubic")
                if grid.shape[-2:] != (gh, gw):
                    msg = f"position grid {tuple(grid.shape[-2:])} != {(gh, gw)}"
                    raise RuntimeError(msg)
                pos = torch.cat([table[:, :1], grid.permute(0, 2, 3, 1).reshape(1, gh * gw, -1)], 1)
            self._pos[key] = pos.to(self.dtype)
        return self._pos[key]

    def tokens(self, images: torch.Tensor) -> torch.Tensor:
        """Patch embedding, class token and position embedding (`prepare_tokens_with_masks`, net/dinov2.py:239-258)."""
        w, ps = self.w, self.cfg.patch
        x = F.conv2d(images.to(self.dtype), w["patch_embed.proj.weight"], w["patch_embed.proj.bias"], stride=ps)
        b, c, gh, gw = x.shape
        x = x.flatten(2).transpose(1, 2)
        x = torch.cat([w["cls_token"].expand(b, -1, -1), x], 1)
        return x + self.pos_embed(gh, gw)

    def block(self, i: int, x: torch.Tensor) -> torch.Tensor:
        """One pre-norm block, the unfused branch of `FastViT.block` (fast_vit.py:163-180)."""
        w, cfg, p = self.w, self.cfg, f"blocks.{i}."
        b, n, c = x.shape
        h = cfg.heads
        y = F.layer_norm(x, (c,), w[p + "norm1.weight"], w[p + "norm1.bias"], cfg.eps)
        qkv = F.linear(y, w[p + "attn.qkv.weight"], w[p + "attn.qkv.bias"]).view(b, n, 3, h, c // h)
        q, k, v = qkv.unbind(2)  # strided views of the packed tensor: nothing is copied
        o = self.attn(q, k, v, (c // h) ** -0.5).view(b, n, c)
        o = F.linear(o, w[p + "attn.proj.weight"], w[p + "attn.proj.bias"])
        x = torch.addcmul(x, o, w[p + "ls1.gamma"]) if cfg.layerscale else x + o
        y = F.layer_norm(x, (c,), w[p + "norm2.weight"], w[p + "norm2.bias"], cfg.eps)
        if cfg.ffn == "swiglu":
            x1, x2 = F.linear(y, w[p + "mlp.w12.weight"], w[p + "mlp.w12.bias"]).chunk(2, dim=-1)
            o = F.linear(F.silu(x1) * x2, w[p + "mlp.w3.weight"], w[p + "mlp.w3.bias"])
        else:
            o = F.linear(F.gelu(F.linear(y, w[p + "mlp.fc1.weight"], w[p + "mlp.fc1.bias"])),
                         w[p + "mlp.fc2.weight"], w[p + "mlp.fc2.bias"])  # fmt: skip
        return x.addcmul_(o, w[p + "ls2.gamma"]) if cfg.layerscale else x.add_(o)

    @torch.no_grad()
    def __call__(self, images: torch.Tensor) -> torch.Tensor:
        x = self.tokens(images.to(self.device))
        for i in range(self.cfg.depth):
            x = self.block(i, x)
        c = x.shape[-1]
        return F.layer_norm(x, (c,), self.w["norm.weight"], self.w["norm.bias"], self.cfg.eps)

    @torch.no_grad()
    def intermediate(self, images: torch.Tensor, layers: tuple[int, ...]) -> list[torch.Tensor]:
        """Normalised tokens after the blocks in `layers`: what the depth models hand to their DPT head
        (upstream `get_intermediate_layers(..., norm=True)`, net/dinov2.py:300-336; Depth-Anything-V2-L takes blocks
        4, 11, 17, 23)."""
        x = self.tokens(images.to(self.device))
        c = x.shape[-1]
        outs = []
        for i in range(max(layers) + 1):
            x = self.block(i, x)
            if i in layers:
                outs.append(F.layer_norm(x, (c,), self.w["norm.weight"], self.w["norm.bias"], self.cfg.eps))
        return outs

    def attention_flops(self, batch: int, height: int, width: int) -> float:
        """FLOPs of the attention calls of one forward: depth * 4 * B * heads * N^2 * 64."""
        n = self.cfg.tokens(height, width)
        return self.cfg.depth * 4.0 * batch * self.cfg.heads * n * n * 64
