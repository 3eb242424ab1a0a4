"""Kernels-mode ViT encoder around the attention operator: the caller side of the hot path.

A harness of the DINOv2 / timm ViT block family: layer norms, packed qkv, attention on strided `[B, N, heads, 64]`
views of it through `Flash64`, projection with LayerScale and residual, MLP or fused SwiGLU. On a CUDA device every
linear layer is one launch of this library's GEMM with the fused epilogue (bias, GELU, LayerScale, in-place residual:
what the reference's kernels mode does with its `dpt_fused` library, `src/fastforks/shared/depth_anything_v2/
fast_vit.py:192-208`) and the attention is the B200 kernel; LayerNorm, the patch embedding and SiLU stay torch calls.
It exists to measure whole-model throughput and to check model-level parity (cosine >= 0.999 against the reference's
portable network, `tests/golden/make_golden.py`), not to replace the reference's model zoo.

Parameter names follow the reference's vendored DINOv2 (`net/dinov2.py`), so a state dict of that network loads here
unchanged; `seeded_state` builds the random-init weights the benchmark configurations ask for.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F  # noqa: N812

from .flash64 import Flash64
from .gemm import ACT_GELU_TANH, ACT_NONE, gemm


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
                 dtype: torch.dtype = torch.float16, variant: str = "hh", fused: bool | None = None,
                 fuse_plain: bool = False) -> None:  # fmt: skip
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
        # On a CUDA device the linear layers run on this library's GEMM with the fused epilogue, which takes the
        # LayerScale factors as fp32 vectors; elsewhere (CPU harness tests) they are torch calls.
        self.fused = self.device.type == "cuda" if fused is None else fused
        # Layers with nothing but a bias behind the product (qkv, SwiGLU's w12) go to torch's library GEMM unless
        # `fuse_plain`: without an epilogue to fuse there is no traffic to save, and without cluster multicast (which
        # this library never uses) a GEMM of its own is bound by the L2 at about 0.8 of the library's rate.
        self.fuse_plain = fuse_plain
        self.scales = {k: v.to(self.device, torch.float32) for k, v in state.items() if k.endswith(".gamma")}

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

    def linear(self, x: torch.Tensor, name: str, *, act: int = ACT_NONE, gamma: str | None = None,
               residual: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
        """`act(x @ W^T + b)`, or with `gamma` and `residual`: `residual + gamma * (x @ W^T + b)`, written into
        `residual`. On a CUDA device this is ONE launch of this library's GEMM with the fused epilogue
        (`gemm`: bias, activation, LayerScale and in-place residual leave the accumulator together); elsewhere the
        same formula in torch ops (the CPU harness tests)."""
        w, b = self.w[name + ".weight"], self.w[name + ".bias"]
        if self.fused and act == ACT_NONE and residual is None and not self.fuse_plain:
            return F.linear(x, w, b)  # nothing to fuse: a plain library GEMM with bias (see `fuse_plain`)
        if self.fused:
            scale = self.scales[gamma] if gamma is not None else None
            return gemm(x, w, b, act=act, scale=scale, res=residual, out=residual)
        y = F.linear(x, w, b)
        if act == ACT_GELU_TANH:
            y = F.gelu(y)  # the tanh form is the fused epilogue's stand-in for this exact GELU
        if residual is None:
            return y
        return residual.addcmul_(y, self.w[gamma]) if gamma is not None else residual.add_(y)

    def block(self, i: int, x: torch.Tensor) -> torch.Tensor:
        """One pre-norm block of the DINOv2 / timm ViT family on `[B, N, C]` tokens, in place:
        `x += ls1 * proj(attention(qkv(norm1(x))))`, `x += ls2 * ffn(norm2(x))`
        (upstream `NestedTensorBlock.forward`, net/dinov2_layers/block.py; timm `Block.forward`,
        src/fastforks/shared/timm_blocks/net/vit.py:60-62). q, k, v are strided views of the packed qkv tensor."""
        w, cfg, p = self.w, self.cfg, f"blocks.{i}."
        b, n, c = x.shape
        heads = cfg.heads
        ls1, ls2 = (p + "ls1.gamma", p + "ls2.gamma") if cfg.layerscale else (None, None)
        qkv = self.linear(F.layer_norm(x, (c,), w[p + "norm1.weight"], w[p + "norm1.bias"], cfg.eps), p + "attn.qkv")
        q, k, v = qkv.view(b, n, 3, heads, c // heads).unbind(2)
        attended = self.attn(q, k, v, (c // heads) ** -0.5).view(b, n, c)
        x = self.linear(attended, p + "attn.proj", gamma=ls1, residual=x)
        y = F.layer_norm(x, (c,), w[p + "norm2.weight"], w[p + "norm2.bias"], cfg.eps)
        if cfg.ffn == "swiglu":
            gate, up = self.linear(y, p + "mlp.w12").chunk(2, dim=-1)
            return self.linear(F.silu(gate).mul_(up), p + "mlp.w3", gamma=ls2, residual=x)
        hidden = self.linear(y, p + "mlp.fc1", act=ACT_GELU_TANH)
        return self.linear(hidden, p + "mlp.fc2", gamma=ls2, residual=x)

    @torch.no_grad()
    def __call__(self, images: torch.Tensor) -> torch.Tensor:
        x = self.tokens(images.to(self.device))
        for i in range(self.cfg.depth):
            x = self.block(i, x)
        c = x.shape[-1]
        return F.layer_norm(x, (c,), self.w["norm.weight"], self.w["norm.bias"], self.cfg.eps)

    def checked(self, images: torch.Tensor) -> torch.Tensor:
        """`self(images)`, then one read of the device's error word (one synchronisation per model call, like the
        reference's `kernels.checked`): every wait inside the kernels is bounded, and a kernel that gave one up
        returns normally with an invalid output, which only this word shows.

        Raises:
            RuntimeError: A kernel of this call gave up a wait; the output must not be used.
        """
        from .attention import device_status

        out = self(images)
        status = device_status(self.device)
        if status != 0:
            msg = f"a kernel gave up a bounded wait during this call (status word {status}); the output is invalid"
            raise RuntimeError(msg)
        return out

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
