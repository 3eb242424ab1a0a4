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

MODEL_CASES = ("model_dinov2_vits14", "model_dinov2_vits14_sharp")


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
def test_kernels_encoder_batches_are_independent() -> None:
    """Image-wise sharding relies on it: an image's output does not depend on what else is in the batch."""
    cfg = CONFIGS["dinov2-vits14"]
    enc = ViTEncoder(cfg, seeded_state(cfg, 1, qk_gain=4.0), device="cuda", dtype=torch.float16)
    images = torch.rand(3, 3, 224, 224, generator=torch.Generator().manual_seed(5))
    full = enc(images)
    for i in range(3):
        single = enc(images[i : i + 1])
        assert cosine(single.float().cpu().numpy(), full[i : i + 1].float().cpu().numpy()) > 0.9999
