"""Model-level parity of the kernels-mode ViT harness with the reference's portable DINOv2 network.

The golden outputs (`tests/golden/model_*.npz`) come from the reference's own vendored network, run in fp32 on CPU
on the weights of `seeded_state` (loaded strictly, so names and shapes are the reference's). Bar: cosine similarity
>= 0.999 between final outputs (the path's model-level tolerance).

On CPU the harness runs with `Flash64._run` replaced by the oracle, the way the reference's guard tests replace it by
a fake kernel (tests/test_flash64_guard.py:29-172): that checks the harness, not the kernel. On a GPU the real kernel runs.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import load_golden
from fastforks_b200.flash64 import Flash64
from fastforks_b200.vit import CONFIGS, ViTEncoder, seeded_state, state_shapes

MODEL_CASES = ("model_dinov2_vits14", "model_dinov2_vits14_sharp")  # whole fp32 outputs; the other goldens are fp16 samples


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def golden_inputs(name: str) -> tuple[dict, dict, torch.Tensor]:
    g = load_golden(name)
    state = seeded_state(CONFIGS["dinov2-vits14"], int(g["seed"]), qk_gain=float(g["qk_gain"]))
    h, w = (int(x) for x in g["hw"])
    images = torch.rand(1, 3, h, w, generator=torch.Generator().manual_seed(int(g["image_seed"])))
    return g, state, images


def test_seeded_state_is_deterministic_and_complete() -> None:
    cfg = CONFIGS["dinov2-vitg14"]
    shapes = state_shapes(cfg)
    assert shapes["blocks.0.mlp.w12.weight"] == (2 * 4096, 1536)  # SwiGLU hidden of ViT-g/14
    assert shapes["pos_embed"] == (1, 1 + 37 * 37, 1536)
    small = CONFIGS["dinov2-vits14"]
    a, b = seeded_state(small, 3), seeded_state(small, 3)
    assert list(a) == list(state_shapes(small))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["cls_token"], seeded_state(small, 4)["cls_token"])
    assert float(a["blocks.0.ls1.gamma"].min()) == 1.0
    assert float(a["blocks.3.attn.qkv.bias"].abs().max()) == 0.0
    assert CONFIGS["dinov2-vits14"].tokens(518, 518) == 1370


@pytest.mark.parametrize("name", MODEL_CASES)
def test_harness_matches_reference_network_on_cpu(name: str, monkeypatch: pytest.MonkeyPatch) -> None:
    from oracle import attention_oracle as ao

    def oracle_run(variant: str, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        out = ao.attention(*(t.permute(0, 2, 1, 3).numpy() for t in (q, k, v)), scale)
        return torch.from_numpy(out).permute(0, 2, 1, 3).contiguous()

    monkeypatch.setattr(Flash64, "_run", staticmethod(oracle_run))
    g, state, images = golden_inputs(name)
    enc = ViTEncoder(CONFIGS["dinov2-vits14"], state, device="cpu", dtype=torch.float32)
    out = enc(images).numpy()
    assert out.shape == g["out"].shape
    np.testing.assert_allclose(out, g["out"], rtol=0, atol=2e-4)
    assert cosine(out, g["out"]) > 0.999999


@pytest.mark.gpu
@pytest.mark.parametrize("name", MODEL_CASES)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_kernels_encoder_matches_reference_network(name: str, dtype: torch.dtype) -> None:
    import fastforks_b200 as ff

    g, state, images = golden_inputs(name)
    enc = ViTEncoder(CONFIGS["dinov2-vits14"], state, device="cuda", dtype=dtype)
    out = enc(images).float().cpu().numpy()
    assert ff.device_status() == 0
    assert np.isfinite(out).all()
    assert cosine(out, g["out"]) >= 0.999, cosine(out, g["out"])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_kernels_encoder_with_every_linear_layer_on_the_own_gemm(dtype: torch.dtype) -> None:
    """By default the layers with nothing to fuse behind the product (qkv) go to torch's library GEMM; with
    `fuse_plain` all four linear layers of every block run on this library's GEMM."""
    import fastforks_b200 as ff

    g, state, images = golden_inputs("model_dinov2_vits14_sharp")
    enc = ViTEncoder(CONFIGS["dinov2-vits14"], state, device="cuda", dtype=dtype, fuse_plain=True)
    out = enc(images).float().cpu().numpy()
    assert ff.device_status() == 0 and np.isfinite(out).all()
    assert cosine(out, g["out"]) >= 0.999, cosine(out, g["out"])


@pytest.mark.gpu
def test_kernels_encoder_batches_are_independent() -> None:
    """Image-wise sharding relies on it: an image's output does not depend on what else is in the batch."""
    cfg = CONFIGS["dinov2-vits14"]
    enc = ViTEncoder(cfg, seeded_state(cfg, 1, qk_gain=4.0), device="cuda", dtype=torch.float16)
    images = torch.rand(3, 3, 224, 224, generator=torch.Generator().manual_seed(5))
    full = enc(images)
    for i in range(3):
        single = enc(images[i : i + 1])
        assert cosine(single.float().cpu().numpy(), full[i : i + 1].float().cpu().numpy()) > 0.9999


# ---- the other model families and the long-sequence case ------------------------------------------------------------
# Goldens: `tests/golden/make_golden.py` (the reference's portable fp32 networks on the seeded weights of this
# package's `seeded_state` / `sam_seeded_state`, loaded strictly), stored as fp16 samples of the outputs.


def _oracle_flash(monkeypatch: pytest.MonkeyPatch) -> None:
    from oracle import attention_oracle as ao

    def oracle_run(variant: str, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        out = ao.attention(*(t.permute(0, 2, 1, 3).numpy() for t in (q, k, v)), scale)
        return torch.from_numpy(out).permute(0, 2, 1, 3).contiguous()

    monkeypatch.setattr(Flash64, "_run", staticmethod(oracle_run))


def _giant_block(device: str, dtype: torch.dtype) -> tuple[np.ndarray, np.ndarray]:
    import dataclasses

    g = load_golden("model_dinov2_vitg14_block")
    cfg = dataclasses.replace(CONFIGS["dinov2-vitg14"], depth=int(g["depth"]))
    state = seeded_state(cfg, int(g["seed"]), qk_gain=float(g["qk_gain"]))
    h, w = (int(x) for x in g["hw"])
    images = torch.rand(1, 3, h, w, generator=torch.Generator().manual_seed(int(g["image_seed"])))
    out = ViTEncoder(cfg, state, device=device, dtype=dtype)(images).float().cpu().numpy()
    return out, g["out"].astype(np.float32)


def _timm_blocks(device: str, dtype: torch.dtype) -> tuple[np.ndarray, np.ndarray]:
    g = load_golden("model_timm_vitb16_blocks")
    cfg = CONFIGS["vit-b16"]
    enc = ViTEncoder(cfg, seeded_state(cfg, int(g["seed"]), qk_gain=float(g["qk_gain"])), device=device, dtype=dtype)
    x = torch.randn(1, 197, cfg.dim, generator=torch.Generator().manual_seed(int(g["token_seed"]))).to(device, dtype)
    with torch.no_grad():
        for i in range(cfg.depth):
            x = enc.block(i, x)
    return x.float().cpu().numpy(), g["out"].astype(np.float32)


@pytest.mark.parametrize("case", [_giant_block, _timm_blocks])
def test_swiglu_block_and_timm_blocks_harness_on_cpu(case, monkeypatch: pytest.MonkeyPatch) -> None:  # noqa: ANN001
    """The harness' SwiGLU branch (one ViT-g/14 block) and its no-LayerScale branch (timm ViT-B/16 blocks) against the
    reference modules, with the oracle standing in for the kernel: checks the harness, not the kernel."""
    _oracle_flash(monkeypatch)
    out, ref = case("cpu", torch.float32)
    assert out.shape == ref.shape
    assert cosine(out, ref) > 0.99999


@pytest.mark.gpu
@pytest.mark.parametrize("case", [_giant_block, _timm_blocks])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_swiglu_block_and_timm_blocks_on_the_kernels(case, dtype: torch.dtype) -> None:  # noqa: ANN001
    import fastforks_b200 as ff

    out, ref = case("cuda", dtype)
    assert ff.device_status() == 0 and np.isfinite(out).all()
    assert cosine(out, ref) >= 0.999, cosine(out, ref)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_vits14_at_518px_matches_reference_network(dtype: torch.dtype) -> None:
    """N = 1370: the long-sequence kernel (and, at this size, the key-split plan) inside a whole model."""
    import fastforks_b200 as ff

    g, state, images = golden_inputs("model_dinov2_vits14_518")
    out = ViTEncoder(CONFIGS["dinov2-vits14"], state, device="cuda", dtype=dtype)(images).float().cpu()
    every = int(g["every"])
    got = torch.cat([out[:, :1], out[:, 1::every]], 1).numpy()
    assert ff.device_status() == 0 and np.isfinite(got).all()
    assert got.shape == g["out"].shape
    assert cosine(got, g["out"].astype(np.float32)) >= 0.999, cosine(got, g["out"].astype(np.float32))


@pytest.mark.gpu
def test_depth_anything_v2_l_encoder_call_matches_reference_network() -> None:
    """ViT-L/14 at 518 px, bf16, the four intermediate outputs Depth-Anything-V2-L feeds to its DPT head (class token
    and a sample of the patch tokens of blocks 4, 11, 17, 23): each at cosine >= 0.999."""
    import fastforks_b200 as ff

    g = load_golden("model_dav2l_encoder_518")
    cfg = CONFIGS["dinov2-vitl14"]
    state = seeded_state(cfg, int(g["seed"]), qk_gain=float(g["qk_gain"]))
    images = torch.rand(1, 3, 518, 518, generator=torch.Generator().manual_seed(int(g["image_seed"])))
    enc = ViTEncoder(cfg, state, device="cuda", dtype=torch.bfloat16)
    outs = enc.intermediate(images, tuple(int(x) for x in g["layers"]))
    every = int(g["every"])
    assert ff.device_status() == 0
    for got, ref in zip(outs, g["out"]):
        got = torch.cat([got[:, :1], got[:, 1:][:, ::every]], 1).float().cpu().numpy()
        assert got.shape == ref.shape
        assert cosine(got, ref.astype(np.float32)) >= 0.999, cosine(got, ref.astype(np.float32))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_sam_vit_b_encoder_matches_reference_encoder(dtype: torch.dtype) -> None:
    """SAM ViT-B at 1024 x 1024: eight blocks of 25 zero-padded 14 x 14 windows and four global blocks of 4096 tokens,
    all with the decomposed relative-position term (tables filled), against upstream's `ImageEncoderViT` in fp32."""
    import fastforks_b200 as ff
    from fastforks_b200.sam import SAM_VIT_B, SamEncoder, sam_seeded_state

    g = load_golden("model_sam_vitb_1024")
    images = torch.rand(1, 3, 1024, 1024, generator=torch.Generator().manual_seed(int(g["image_seed"])))
    out = SamEncoder(SAM_VIT_B, sam_seeded_state(SAM_VIT_B, int(g["seed"])), device="cuda", dtype=dtype)(images)
    every = int(g["every"])
    got = out[:, :, ::every, ::every].float().cpu().numpy()
    assert ff.device_status() == 0 and np.isfinite(got).all()
    assert got.shape == g["out"].shape
    assert cosine(got, g["out"].astype(np.float32)) >= 0.999, cosine(got, g["out"].astype(np.float32))


def test_sam_seeded_state_follows_the_upstream_parameter_list() -> None:
    from fastforks_b200.sam import SAM_VIT_B, rel_table, sam_seeded_state, sam_state_shapes

    shapes = sam_state_shapes(SAM_VIT_B)
    assert shapes["blocks.0.attn.rel_pos_h"] == (27, 64)  # windowed block: 2 * 14 - 1
    assert shapes["blocks.2.attn.rel_pos_w"] == (127, 64)  # global block: 2 * 64 - 1
    assert shapes["neck.2.weight"] == (256, 256, 3, 3)
    state = sam_seeded_state(SAM_VIT_B, 3)
    assert list(state) == list(shapes)
    assert float(state["blocks.5.attn.rel_pos_h"].abs().max()) > 0  # the bias path is exercised
    table = rel_table(3, torch.arange(5.0)[:, None])  # rows 0..4 stand for relative positions -2..2
    assert table[:, :, 0].tolist() == [[2.0, 1.0, 0.0], [3.0, 2.0, 1.0], [4.0, 3.0, 2.0]]
