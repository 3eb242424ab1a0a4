"""Writes the golden vectors of `tests/golden/*.npz` by running the reference's own portable modules on CPU.

Run where the reference checkout is available (it is not on the GPU machines, so the outputs are committed):

    python tests/golden/make_golden.py /path/to/fastforks

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
}


def main() -> None:
    root = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    _import_reference(root)
    torch.set_num_threads(1)  # one thread: bit-stable sums
    for name, (fn, kwargs) in CASES.items():
        case = fn(**kwargs)
        arrays = {k: (v.contiguous().numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in case.items()}
        np.savez(HERE / f"{name}.npz", **arrays)
        print(name, {k: a.shape for k, a in arrays.items()})


if __name__ == "__main__":
    main()
