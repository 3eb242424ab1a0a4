"""Pins the CPU oracle to the reference: every golden vector written by the reference's own modules
(`tests/golden/make_golden.py`) must be reproduced by the numpy restatement and by the C restatement."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import attention_oracle as ao
from oracle import c_oracle

FP32_TOL = 5e-5  # fp32 round-off of two matmuls and a softmax; outputs are O(1), the peaky case O(10)


def _bias_of(case: dict) -> tuple[np.ndarray | None, tuple | None]:
    if "bias" not in case:
        return None, None
    rel = ao.decomposed_terms(case["q"], case["rel_pos_h"], case["rel_pos_w"], case["hw"])
    return ao.decomposed_bias(*rel), rel


def test_numpy_oracle_matches_reference_modules(golden: dict) -> None:
    bias, _ = _bias_of(golden)
    out = ao.attention(golden["q"], golden["k"], golden["v"], float(golden["scale"]), bias)
    np.testing.assert_allclose(out, golden["out"], rtol=0, atol=FP32_TOL)


def test_c_oracle_matches_reference_modules(golden: dict) -> None:
    _, rel = _bias_of(golden)
    out = c_oracle.attention(golden["q"], golden["k"], golden["v"], float(golden["scale"]), rel=rel, threads=2)
    np.testing.assert_allclose(out, golden["out"], rtol=0, atol=FP32_TOL)


@pytest.mark.parametrize("name", ["sam_window_14x14", "sam_grid_8x16"])
def test_decomposed_bias_matches_reference_add_decomposed_rel_pos(name: str) -> None:
    from conftest import load_golden

    case = load_golden(name)
    bias, _ = _bias_of(case)
    np.testing.assert_allclose(bias, case["bias"], rtol=0, atol=5e-6)


def test_c_oracle_dense_bias_equals_decomposed() -> None:
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((1, 2, 35, 64), dtype=np.float32) for _ in range(3))
    rel_h = rng.standard_normal((1, 2, 35, 5), dtype=np.float32)
    rel_w = rng.standard_normal((1, 2, 35, 7), dtype=np.float32)
    dense = ao.decomposed_bias(rel_h, rel_w)
    a = c_oracle.attention(q, k, v, bias=dense)
    b = c_oracle.attention(q, k, v, rel=(rel_h, rel_w))
    c = ao.attention(q, k, v, bias=dense)
    np.testing.assert_allclose(a, b, rtol=0, atol=1e-6)
    np.testing.assert_allclose(a, c, rtol=0, atol=1e-5)


def test_oracle_properties() -> None:
    """Size-independent properties the GPU tests also use: rows of P sum to one (v = 1 -> out = 1), key
    permutation invariance, and a huge negative bias on a key removes it."""
    rng = np.random.default_rng(1)
    q, k, v = (rng.standard_normal((2, 3, 50, 64), dtype=np.float32) for _ in range(3))
    np.testing.assert_allclose(ao.attention(q, k, np.ones_like(v)), 1.0, atol=1e-5)
    perm = rng.permutation(50)
    np.testing.assert_allclose(ao.attention(q, k[:, :, perm], v[:, :, perm]), ao.attention(q, k, v), atol=1e-5)
    bias = np.zeros((1, 1, 50, 50), dtype=np.float32)
    bias[..., 10:] = -np.inf
    np.testing.assert_allclose(ao.attention(q, k, v, bias=bias), ao.attention(q, k[:, :, :10], v[:, :, :10]), atol=1e-5)


def test_get_rel_pos_rejects_interpolation() -> None:
    with pytest.raises(ValueError, match="interpolation"):
        ao.get_rel_pos(14, 14, np.zeros((5, 64), dtype=np.float32))


def test_gemm_oracle_matches_the_torch_calls_of_the_portable_blocks() -> None:
    """`oracle/gemm_oracle.py` against `tests/golden/gemm_epilogue.npz` (torch fp32 on the CPU: `F.linear`, `F.gelu`
    in both forms, `F.relu`, LayerScale + residual): every case of the fused epilogue's formula, at fp32 round-off."""
    from conftest import load_golden
    from oracle import gemm_oracle as go

    g = load_golden("gemm_epilogue")
    x, w, bias, scale, res = (g[k] for k in ("x", "w", "bias", "scale", "res"))
    cases = {
        "linear": go.gemm_epilogue(x, w, bias),
        "gelu": go.gemm_epilogue(x, w, bias, act=go.ACT_GELU),
        "gelu_tanh": go.gemm_epilogue(x, w, bias, act=go.ACT_GELU_TANH),
        "relu": go.gemm_epilogue(x, w, bias, act=go.ACT_RELU),
        "layerscale_residual": go.gemm_epilogue(x, w, bias, scale=scale, res=res),
        "no_bias_residual": go.gemm_epilogue(x, w, res=res),
    }
    for name, got in cases.items():
        np.testing.assert_allclose(got, g[name], rtol=0, atol=3e-5, err_msg=name)


def test_rope_oracle_matches_the_reference_portable_dinov3_attention() -> None:
    """`oracle/rope_oracle.py` against `tests/golden/dinov3_attention_6x5.npz` (the reference's `DINOv3ViT.attention` on
    a seeded layer): the half tables of `rope_table`, and q and k as they reach SDPA, in the kernel's form
    (`rope_qk`) and in the portable form (`rope_portable`); then the attention output from the rotated operands."""
    from conftest import load_golden
    from oracle import attention_oracle as ao
    from oracle import rope_oracle as ro

    g = load_golden("dinov3_attention_6x5")
    h, w = (int(x) for x in g["hw"])
    np.testing.assert_allclose(ro.rope_table(h, w, float(g["theta"])), g["cs"], rtol=0, atol=2e-6)
    to_bnhd = lambda a: a.transpose(0, 2, 1, 3)  # noqa: E731 - golden tensors are [B, heads, N, d]
    q_rot, k_rot = ro.rope_qk(to_bnhd(g["q"]), to_bnhd(g["k"]), g["cs"])
    np.testing.assert_allclose(to_bnhd(q_rot), g["q_rot"], rtol=0, atol=5e-6)
    np.testing.assert_allclose(to_bnhd(k_rot), g["k_rot"], rtol=0, atol=5e-6)
    np.testing.assert_allclose(ro.rope_portable(g["q"], g["cs"]), g["q_rot"], rtol=0, atol=5e-6)
    # the softmax scale on q commutes with the rotation and is exact for 2^-3
    q_scaled, _ = ro.rope_qk(to_bnhd(g["q"]), to_bnhd(g["k"]), g["cs"], q_scale=0.125)
    np.testing.assert_array_equal(q_scaled, q_rot * np.float32(0.125))
    out = ao.attention(g["q_rot"], g["k_rot"], g["v"], float(g["scale"]))
    np.testing.assert_allclose(out, g["out"], rtol=0, atol=5e-5)
