"""Writes the golden vectors of `tests/golden/*.npz` by running the reference's own portable modules on CPU.

Run where the reference checkout is available (it is not on the GPU machines, so the outputs are committed):

    python tests/golden/make_golden.py /path/to/fastforks [case ...]

For each case a reference attention module (seeded random weights, fp32, CPU) is run on a seeded input; hooks on
its `qkv` and `proj` layers capture the hot path's inputs (q, k, v after the projection) and its output (the tensor
fed to `proj`). For SAM the dense bias that `add_decomposed_rel_pos` adds to the logits is captured by calling that
function on zero logits. Modules used (paths inside the reference):

    dinov2   src/fastforks/shared/depth_anything_v2/net/dinov2_layers/attention.py:46-60   (Attention.forward)
    timm     src/fastforks/shared/timm_blocks/net/vit.py:32-48                             (Attention.forward, SDPA)
    sam      src/fastforks/promptable_segmentation/models/sam/net/image_encoder.py:225-241, 293-362
"""

from __future__ import annotations

import importlib.metadata
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _import_reference(root: Path) -> None:
    sys.path.insert(0, str(root / "src"))
    real = importlib.metadata.version

    def version(name: str) -> str:  # the checkout is not an installed distribution
        return "0.0.0" if name == "fastforks-core" else real(name)

    importlib.metadata.version = version


def _capture(module: torch.nn.Module, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Run `module(x)`; returns (output of module.qkv, input of module.proj)."""
    got: dict[str, torch.Tensor] = {}
    h1 = module.qkv.register_forward_hook(lambda _m, _i, o: got.__setitem__("qkv", o.detach().clone()))
    h2 = module.proj.register_forward_pre_hook(lambda _m, i: got.__setitem__("out", i[0].detach().clone()))
    with torch.no_grad():
        module(x)
    h1.remove()
    h2.remove()
    return got["qkv"], got["out"]


def _init(module: torch.nn.Module, gen: torch.Generator, std: float) -> None:
    with torch.no_grad():
        for p in module.parameters():
            p.copy_(torch.randn(p.shape, generator=gen) * std)


def dinov2_case(seed: int, b: int, n: int, dim: int, heads: int, std: float) -> dict[str, np.ndarray]:
    from fastforks.shared.depth_anything_v2.net.dinov2_layers.attention import Attention

    gen = torch.Generator().manual_seed(seed)
    m = Attention(dim, num_heads=heads, qkv_bias=True).eval()
    _init(m, gen, std)
    x = torch.randn(b, n, dim, generator=gen)
    qkv, out = _capture(m, x)
    q, k, v = qkv.reshape(b, n, 3, heads, dim // heads).permute(2, 0, 3, 1, 4)  # [B, heads, N, d]
    o = out.reshape(b, n, heads, dim // heads).permute(0, 2, 1, 3)
    return {"q": q, "k": k, "v": v, "out": o, "scale": np.float32(m.scale)}


def timm_case(seed: int, b: int, n: int, dim: int, heads: int, std: float) -> dict[str, np.ndarray]:
    from fastforks.shared.timm_blocks.net.vit import Attention

    gen = torch.Generator().manual_seed(seed)
    m = Attention(dim, heads).eval()
    _init(m, gen, std)
    x = torch.randn(b, n, dim, generator=gen)
    qkv, out = _capture(m, x)
    q, k, v = qkv.reshape(b, n, 3, heads, dim // heads).permute(2, 0, 3, 1, 4)
    o = out.reshape(b, n, heads, dim // heads).permute(0, 2, 1, 3)
    return {"q": q, "k": k, "v": v, "out": o, "scale": np.float32((dim // heads) ** -0.5)}


def sam_case(seed: int, b: int, hw: tuple[int, int], dim: int, heads: int, std: float) -> dict[str, np.ndarray]:
    from fastforks.promptable_segmentation.models.sam.net.image_encoder import Attention, add_decomposed_rel_pos

    gen = torch.Generator().manual_seed(seed)
    m = Attention(dim, num_heads=heads, qkv_bias=True, use_rel_pos=True, input_size=hw).eval()
    _init(m, gen, std)  # also fills rel_pos_h / rel_pos_w, which upstream initialises to zero
    h, w = hw
    x = torch.randn(b, h, w, dim, generator=gen)
    qkv, out = _capture(m, x)
    d = dim // heads
    q, k, v = qkv.reshape(b, h * w, 3, heads, d).permute(2, 0, 3, 1, 4)  # [B, heads, N, d]
    with torch.no_grad():
        zeros = torch.zeros(b * heads, h * w, h * w)
        bias = add_decomposed_rel_pos(zeros, q.reshape(b * heads, h * w, d), m.rel_pos_h, m.rel_pos_w, hw, hw)
    o = out.reshape(b, h * w, heads, d).permute(0, 2, 1, 3)
    return {
        "q": q, "k": k, "v": v, "out": o, "scale": np.float32(m.scale),
        "bias": bias.reshape(b, heads, h * w, h * w),
        "rel_pos_h": m.rel_pos_h.detach(), "rel_pos_w": m.rel_pos_w.detach(), "hw": np.array(hw, dtype=np.int32),
    }  # fmt: skip


def dinov2_model_case(seed: int, name: str, hw: tuple[int, int], qk_gain: float) -> dict[str, np.ndarray]:
    """The reference's vendored DINOv2 network (portable fp32, CPU) on the seeded weights of
    `fastforks_b200.vit.seeded_state`, loaded strictly: the harness and the reference share one parameterisation.
    Only the input seed and the output are stored; the weights are regenerated from the seed."""
    sys.path.insert(0, str(HERE.parent.parent))
    from fastforks.shared.depth_anything_v2 import DINOv2

    from fastforks_b200.vit import CONFIGS, seeded_state

    cfg = CONFIGS[name]
    net = DINOv2({"dinov2-vits14": "vits", "dinov2-vitb14": "vitb"}[name]).eval()
    state = seeded_state(cfg, seed, qk_gain=qk_gain)
    assert list(net.state_dict()) == list(state), "parameter names / order differ from the reference network"
    net.load_state_dict(state, strict=True)
    images = torch.rand(1, 3, *hw, generator=torch.Generator().manual_seed(seed + 1))
    with torch.no_grad():
        feats = net.forward_features(images)
    tokens = torch.cat([feats["x_norm_clstoken"][:, None], feats["x_norm_patchtokens"]], 1)
    return {"out": tokens, "seed": np.int64(seed), "image_seed": np.int64(seed + 1), "hw": np.array(hw, dtype=np.int32),
            "qk_gain": np.float32(qk_gain)}  # fmt: skip


def _sample_tokens(tokens: torch.Tensor, every: int) -> torch.Tensor:
    """Class token and every `every`-th patch token: enough for a cosine check, small enough to commit."""
    return torch.cat([tokens[:, :1], tokens[:, 1::every]], 1)


def dinov2_block_case(seed: int, name: str, depth: int, hw: tuple[int, int], qk_gain: float) -> dict[str, np.ndarray]:
    """The first `depth` blocks of a vendored DINOv2 network (for ViT-g/14: the fused SwiGLU feed-forward) on seeded
    weights: the reference constructor is called with that depth, everything else as `DINOv2(name)` does."""
    import dataclasses

    sys.path.insert(0, str(HERE.parent.parent))
    from fastforks.shared.depth_anything_v2.net import dinov2 as ref

    from fastforks_b200.vit import CONFIGS, seeded_state

    cfg = dataclasses.replace(CONFIGS[name], depth=depth)
    from functools import partial

    # `vit_giant2` / `vit_large` (net/dinov2.py:385-420) fix the depth: the same constructor call with `depth` blocks
    net = ref.DinoVisionTransformer(
        patch_size=14, embed_dim=cfg.dim, depth=depth, num_heads=cfg.heads, mlp_ratio=4,
        block_fn=partial(ref.Block, attn_class=ref.MemEffAttention), num_register_tokens=0, img_size=518, init_values=1.0,
        ffn_layer="swiglufused" if cfg.ffn == "swiglu" else "mlp", block_chunks=0, interpolate_antialias=False,
        interpolate_offset=0.1,
    ).eval()  # fmt: skip
    state = seeded_state(cfg, seed, qk_gain=qk_gain)
    assert list(net.state_dict()) == list(state), "parameter names / order differ from the reference network"
    net.load_state_dict(state, strict=True)
    images = torch.rand(1, 3, *hw, generator=torch.Generator().manual_seed(seed + 1))
    with torch.no_grad():
        feats = net.forward_features(images)
    tokens = torch.cat([feats["x_norm_clstoken"][:, None], feats["x_norm_patchtokens"]], 1)
    return {"out": tokens.half(), "seed": np.int64(seed), "image_seed": np.int64(seed + 1), "hw": np.array(hw, dtype=np.int32),
            "qk_gain": np.float32(qk_gain), "depth": np.int64(depth)}  # fmt: skip


def dinov2_518_case(seed: int, name: str, qk_gain: float, every: int) -> dict[str, np.ndarray]:
    """ViT-S/14 at 518 x 518: N = 1370 tokens, the long-sequence kernel inside a whole model."""
    case = dinov2_model_case(seed, name, (518, 518), qk_gain)
    case["out"] = _sample_tokens(case["out"], every).half()
    case["every"] = np.int64(every)
    return case


def dav2_encoder_case(seed: int, qk_gain: float, every: int) -> dict[str, np.ndarray]:
    """Depth-Anything-V2-L's encoder as its depth model calls it: `get_intermediate_layers` of ViT-L/14 at 518 px for
    blocks 4, 11, 17, 23 with class tokens (src/fastforks/shared/depth_anything_v2/net/dpt.py:176-191). The DPT head
    behind it is convolutions only and is not part of the fixture."""
    sys.path.insert(0, str(HERE.parent.parent))
    from fastforks.shared.depth_anything_v2 import DINOv2

    from fastforks_b200.vit import CONFIGS, seeded_state

    cfg = CONFIGS["dinov2-vitl14"]
    net = DINOv2("vitl").eval()
    state = seeded_state(cfg, seed, qk_gain=qk_gain)
    net.load_state_dict(state, strict=True)
    images = torch.rand(1, 3, 518, 518, generator=torch.Generator().manual_seed(seed + 1))
    layers = [4, 11, 17, 23]
    with torch.no_grad():
        feats = net.get_intermediate_layers(images, layers, return_class_token=True)
    out = torch.stack([torch.cat([cls[:, None], patches[:, ::every]], 1) for patches, cls in feats])  # [4, 1, 1 + n, C]
    return {"out": out.half(), "seed": np.int64(seed), "image_seed": np.int64(seed + 1), "qk_gain": np.float32(qk_gain),
            "layers": np.array(layers, dtype=np.int32), "every": np.int64(every)}  # fmt: skip


def timm_blocks_case(seed: int, qk_gain: float) -> dict[str, np.ndarray]:
    """The twelve blocks of `vit_base_patch16_224` (src/fastforks/shared/timm_blocks/net/vit.py:51-85) on seeded tokens
    `[1, 197, 768]`: the reference builds only the blocks (patch embedding and head come from the caller's model)."""
    sys.path.insert(0, str(HERE.parent.parent))
    from fastforks.shared.timm_blocks.net.vit import create_vit_blocks

    from fastforks_b200.vit import CONFIGS, seeded_state

    cfg = CONFIGS["vit-b16"]
    net = create_vit_blocks("vit_base_patch16_224").eval()
    state = seeded_state(cfg, seed, qk_gain=qk_gain)
    blocks = {k: v for k, v in state.items() if k.startswith("blocks.")}
    assert list(net.state_dict()) == list(blocks), "parameter names / order differ from the reference blocks"
    net.load_state_dict(blocks, strict=True)
    tokens = torch.randn(1, 197, cfg.dim, generator=torch.Generator().manual_seed(seed + 1))
    with torch.no_grad():
        out = net.blocks(tokens)
    return {"out": out.half(), "seed": np.int64(seed), "token_seed": np.int64(seed + 1), "qk_gain": np.float32(qk_gain)}


def sam_encoder_case(seed: int, every: int) -> dict[str, np.ndarray]:
    """SAM ViT-B's image encoder at 1024 x 1024 (8 windowed and 4 global blocks, relative-position tables filled:
    upstream initialises them to zero) on seeded weights; stored: every `every`-th position of the 64 x 64 output."""
    sys.path.insert(0, str(HERE.parent.parent))
    from fastforks.promptable_segmentation.models.sam.net.image_encoder import ImageEncoderViT

    from fastforks_b200.sam import SAM_VIT_B, sam_seeded_state

    cfg = SAM_VIT_B
    net = ImageEncoderViT(img_size=cfg.img, patch_size=cfg.patch, embed_dim=cfg.dim, depth=cfg.depth, num_heads=cfg.heads,
                          out_chans=cfg.out_chans, use_rel_pos=True, window_size=cfg.window,
                          global_attn_indexes=cfg.global_blocks, norm_layer=torch.nn.LayerNorm).eval()  # fmt: skip
    state = sam_seeded_state(cfg, seed)
    assert list(net.state_dict()) == list(state), "parameter names / order differ from the reference encoder"
    net.load_state_dict(state, strict=True)
    images = torch.rand(1, 3, cfg.img, cfg.img, generator=torch.Generator().manual_seed(seed + 1))
    with torch.no_grad():
        out = net(images)
    return {"out": out[:, :, ::every, ::every].half(), "seed": np.int64(seed), "image_seed": np.int64(seed + 1), "every": np.int64(every)}


def gemm_epilogue_case(seed: int) -> dict[str, np.ndarray]:
    """The layers around attention as the reference's portable blocks compute them, in torch fp32 on the CPU:
    `F.linear` alone (qkv), with `F.gelu` (fc1: erf form, `nn.GELU()`; and the tanh form its fused path uses on
    full-rate cards), with `F.relu`, and `residual + gamma * F.linear(...)` (LayerScale and residual of
    `NestedTensorBlock`, net/dinov2_layers/block.py) - the cases of the fused epilogue's formula."""
    import torch.nn.functional as F  # noqa: N812

    gen = torch.Generator().manual_seed(seed)
    m, n, k = 70, 40, 72
    x, w = torch.randn(m, k, generator=gen), torch.randn(n, k, generator=gen) * k**-0.5
    bias, gamma, res = torch.randn(n, generator=gen), torch.rand(n, generator=gen) + 0.5, torch.randn(m, n, generator=gen)
    lin = F.linear(x, w, bias)
    return {"x": x, "w": w, "bias": bias, "scale": gamma, "res": res, "linear": lin, "gelu": F.gelu(lin),
            "gelu_tanh": F.gelu(lin, approximate="tanh"), "relu": F.relu(lin), "layerscale_residual": res + gamma * lin,
            "no_bias_residual": res + F.linear(x, w)}  # fmt: skip


def dinov3_attention_case(seed: int, hw: tuple[int, int], dim: int, heads: int, std: float) -> dict[str, np.ndarray]:
    """The reference's portable DINOv3 attention (`DINOv3ViT.attention`, features/models/dinov3/net.py:191-210) on one
    seeded layer: q, k, v before RoPE, the rotated q and k it hands to SDPA, the input of the output projection, and
    the half tables of `rope_table` in the layout of the kernels mode (model.py:185-188). 1 + 4 prefix tokens."""
    import torch.nn.functional as F  # noqa: N812

    from fastforks.features.models.dinov3 import net as dv3

    gen = torch.Generator().manual_seed(seed)
    cfg = dv3.Config(dim, heads, 1, 2 * dim, gated=False)
    model = dv3.DINOv3ViT(cfg)
    _init(model, gen, std)
    blk = model.layer[0]
    n = 1 + dv3.REGISTERS + hw[0] * hw[1]
    y = torch.randn(2, n, dim, generator=gen)
    rope = model.rope(hw[0], hw[1], torch.float32, y.device)
    a = blk.attention
    got: dict[str, torch.Tensor] = {}
    qkv = torch.stack([p(y).view(2, n, heads, dim // heads).transpose(1, 2) for p in (a.q_proj, a.k_proj, a.v_proj)])
    real_sdpa = F.scaled_dot_product_attention

    def spy(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, **kw: object) -> torch.Tensor:
        got.update(q_rot=q.detach().clone(), k_rot=k.detach().clone())
        return real_sdpa(q, k, v, **kw)

    h = a.o_proj.register_forward_pre_hook(lambda _m, i: got.__setitem__("out", i[0].detach().clone()))
    dv3.F.scaled_dot_product_attention = spy
    try:
        with torch.no_grad():
            model.attention(blk, y, rope)
    finally:
        dv3.F.scaled_dot_product_attention = real_sdpa
        h.remove()
    cos, sin = dv3.rope_table(hw[0], hw[1], dim // heads, cfg.rope_theta, y.device)
    half = dim // heads // 2
    return {"q": qkv[0].detach(), "k": qkv[1].detach(), "v": qkv[2].detach(), "q_rot": got["q_rot"], "k_rot": got["k_rot"],
            "out": got["out"].view(2, n, heads, dim // heads).transpose(1, 2),
            "cs": torch.stack((cos[:, :half], sin[:, :half]), 1), "hw": np.array(hw), "theta": np.float32(cfg.rope_theta),
            "scale": np.float32((dim // heads) ** -0.5)}  # fmt: skip


CASES = {
    # name: (builder, kwargs). Token counts follow the reference: 97 = its feature-golden input (112x168, patch 14),
    # 197 = ViT-B/16 at 224, 196 = one 14x14 SAM window; 8x16 exercises kh != kw.
    "dinov2_n97": (dinov2_case, {"seed": 0, "b": 2, "n": 97, "dim": 128, "heads": 2, "std": 0.08}),
    "dinov2_n257_peaky": (dinov2_case, {"seed": 1, "b": 1, "n": 257, "dim": 128, "heads": 2, "std": 0.25}),
    "timm_n197": (timm_case, {"seed": 2, "b": 1, "n": 197, "dim": 128, "heads": 2, "std": 0.08}),
    "sam_window_14x14": (sam_case, {"seed": 3, "b": 1, "hw": (14, 14), "dim": 128, "heads": 2, "std": 0.08}),
    "sam_grid_8x16": (sam_case, {"seed": 4, "b": 2, "hw": (8, 16), "dim": 64, "heads": 1, "std": 0.1}),
    # whole encoder, N = 1 + 16 * 12 = 193 tokens (a non-square grid exercises the position interpolation)
    "model_dinov2_vits14": (dinov2_model_case, {"seed": 7, "name": "dinov2-vits14", "hw": (224, 168), "qk_gain": 1.0}),
    "model_dinov2_vits14_sharp": (dinov2_model_case, {"seed": 8, "name": "dinov2-vits14", "hw": (224, 224), "qk_gain": 8.0}),
    # N = 1370 inside a whole model; one SwiGLU block of ViT-g/14; the encoder call of Depth-Anything-V2-L; the blocks of
    # timm's ViT-B/16; SAM ViT-B's encoder. Outputs are stored as fp16 samples: the checks are cosine checks.
    "model_dinov2_vits14_518": (dinov2_518_case, {"seed": 9, "name": "dinov2-vits14", "qk_gain": 4.0, "every": 4}),
    "model_dinov2_vitg14_block": (dinov2_block_case, {"seed": 10, "name": "dinov2-vitg14", "depth": 1, "hw": (224, 168), "qk_gain": 4.0}),
    "model_dav2l_encoder_518": (dav2_encoder_case, {"seed": 11, "qk_gain": 4.0, "every": 8}),
    "model_timm_vitb16_blocks": (timm_blocks_case, {"seed": 12, "qk_gain": 4.0}),
    "model_sam_vitb_1024": (sam_encoder_case, {"seed": 13, "every": 2}),
    "gemm_epilogue": (gemm_epilogue_case, {"seed": 14}),
    # DINOv3: rotary embedding on q and k in front of SDPA; 5 prefix tokens + a 6 x 5 patch grid
    "dinov3_attention_6x5": (dinov3_attention_case, {"seed": 15, "hw": (6, 5), "dim": 128, "heads": 2, "std": 0.08}),
}


def main() -> None:
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/fastforks [case ...]")
    _import_reference(Path(sys.argv[1]))
    wanted = sys.argv[2:] or list(CASES)
    for name in wanted:
        fn, kwargs = CASES[name]
        torch.set_num_threads(1 if not name.startswith("model_") else 8)  # op-level cases: one thread, bit-stable sums
        case = fn(**kwargs)
        arrays = {k: (v.contiguous().numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in case.items()}
        (np.savez_compressed if name.startswith("model_") and name not in ("model_dinov2_vits14", "model_dinov2_vits14_sharp")
         else np.savez)(HERE / f"{name}.npz", **arrays)  # fmt: skip
        print(name, {k: a.shape for k, a in arrays.items()})


if __name__ == "__main__":
    main()
