"""Parity of the rotary-embedding kernel (`b200_rope_qk`, through `fastforks_b200.rope_qk_`) with its CPU oracle on a
B200, and of the DINOv3 attention path built from it (rotate in place, then the attention kernel with scale 1).

The oracle (`oracle/rope_oracle.py`) restates the reference's `rope_qk_h` kernel and is pinned to the reference's
portable DINOv3 attention by `tests/test_oracle.py`. Both sides compute in fp32 on the 16-bit operands and round once;
the kernel may contract one product of `x1 c - x2 s` into a fused multiply-add (as the reference's kernel does), so a
result may differ from the oracle's by one unit in the last place of the 16-bit type.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import fastforks_b200 as ff
from conftest import assert_close, load_golden
from oracle import attention_oracle as ao
from oracle import rope_oracle as ro

pytestmark = pytest.mark.gpu
DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}
ULP = {"fp16": 2.0**-10, "bf16": 2.0**-7}  # relative size of one unit in the last place, upper bound


@pytest.fixture(autouse=True)
def _kernels_ran_to_the_end():  # noqa: ANN202
    yield
    assert ff.device_status() == 0


def within_one_ulp(got: torch.Tensor, ref: np.ndarray, dtype: str, what: str) -> None:
    got = got.float().cpu().numpy()
    rounded = torch.from_numpy(ref).to(DTYPES[dtype]).float().numpy()
    diff = np.abs(got - rounded)
    bound = ULP[dtype] * np.maximum(np.abs(rounded), 2.0**-14) * 1.01
    assert (diff <= bound).all(), f"{what}: {int((diff > bound).sum())} elements off by more than one ulp, worst {diff.max()}"
    assert (diff == 0).mean() > 0.98, f"{what}: only {(diff == 0).mean():.4f} of the elements are bit-equal"  # noqa: PLR2004


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_golden_dinov3_attention(dtype: str) -> None:
    """q, k, v of the reference's portable DINOv3 attention: rotate in place with the softmax scale on q, run the
    attention kernel with scale 1 (the call sequence of src/fastforks/features/models/dinov3/model.py:199-201)."""
    g = load_golden("dinov3_attention_6x5")
    dt = DTYPES[dtype]
    qkv = torch.stack([torch.from_numpy(g[x]).transpose(1, 2) for x in "qkv"], 2).to(dt).cuda().contiguous()  # [B, N, 3, H, 64]
    before = qkv.clone()
    cs = torch.from_numpy(g["cs"]).cuda()
    same = ff.rope_qk_(qkv, cs, q_scale=float(g["scale"]))
    assert same.data_ptr() == qkv.data_ptr()
    q_ref, k_ref = ro.rope_qk(before[:, :, 0].float().cpu().numpy(), before[:, :, 1].float().cpu().numpy(), g["cs"], float(g["scale"]))
    within_one_ulp(qkv[:, :, 0], q_ref, dtype, "q")
    within_one_ulp(qkv[:, :, 1], k_ref, dtype, "k")
    assert torch.equal(qkv[:, :, 2], before[:, :, 2]), "v must not change"
    prefix = qkv.shape[1] - cs.shape[0]
    assert torch.equal(qkv[:, :prefix, 1], before[:, :prefix, 1]), "k of the prefix tokens must not change"
    # against the reference's own rotated operands (fp32 there, 16-bit here)
    assert_close(qkv[:, :, 1].float().cpu().numpy().transpose(0, 2, 1, 3), g["k_rot"], unit_scale=True, what="k_rot vs reference")
    q, k, v = qkv.unbind(2)
    out = ff.attention(q, k, v, scale=1.0, layout="bnhd")
    assert_close(out.float().cpu().numpy().transpose(0, 2, 1, 3), g["out"], unit_scale=True, what=f"dinov3 attention {dtype}")


@pytest.mark.parametrize(("b", "heads", "hw"), [(4, 16, (32, 32)), (2, 6, (37, 23)), (1, 20, (14, 14))])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_full_size_against_the_oracle(b: int, heads: int, hw: tuple[int, int], dtype: str) -> None:
    """ViT-L/16 at 512 px (1029 tokens, 16 heads), an odd grid of ViT-S/16, ViT-H+/16 at 224 px: every element."""
    gen = torch.Generator().manual_seed(b * 100 + heads)
    n = 5 + hw[0] * hw[1]
    qkv = torch.randn(b, n, 3, heads, 64, generator=gen).to(DTYPES[dtype]).cuda()
    before = qkv.clone()
    cs = ff.rope_table(hw[0], hw[1], 100.0, "cuda")
    np.testing.assert_allclose(cs.cpu().numpy(), ro.rope_table(hw[0], hw[1], 100.0), rtol=0, atol=2e-6)
    ff.rope_qk_(qkv, cs, q_scale=0.125)
    q_ref, k_ref = ro.rope_qk(before[:, :, 0].float().cpu().numpy(), before[:, :, 1].float().cpu().numpy(), cs.cpu().numpy(), 0.125)
    within_one_ulp(qkv[:, :, 0], q_ref, dtype, "q")
    within_one_ulp(qkv[:, :, 1], k_ref, dtype, "k")
    assert torch.equal(qkv[:, :, 2], before[:, :, 2])


def test_strided_qkv_and_no_prefix() -> None:
    """A qkv tensor that is a view into a wider buffer (token rows padded), no prefix tokens at all."""
    gen = torch.Generator().manual_seed(3)
    b, heads, hw = 2, 3, (5, 4)
    n = hw[0] * hw[1]
    wide = torch.randn(b, n + 3, 3, heads + 1, 64, generator=gen).half().cuda()
    before = wide.clone()
    qkv = wide[:, 2 : 2 + n, :, :heads]
    cs = ff.rope_table(hw[0], hw[1], 100.0, "cuda")
    ff.rope_qk_(qkv, cs)
    view = before[:, 2 : 2 + n, :, :heads]
    q_ref, k_ref = ro.rope_qk(view[:, :, 0].float().cpu().numpy(), view[:, :, 1].float().cpu().numpy(), cs.cpu().numpy())
    within_one_ulp(qkv[:, :, 0], q_ref, "fp16", "q")
    within_one_ulp(qkv[:, :, 1], k_ref, "fp16", "k")
    canary = wide.clone()
    canary[:, 2 : 2 + n, :2, :heads] = before[:, 2 : 2 + n, :2, :heads]
    assert torch.equal(canary, before), "elements outside the q and k views changed"


def test_contract_violations_raise_before_launch() -> None:
    qkv = torch.zeros(1, 9, 3, 2, 64, dtype=torch.float16, device="cuda")
    cs = ff.rope_table(2, 2, 100.0, "cuda")
    with pytest.raises(ValueError, match="float32"):
        ff.rope_qk_(qkv, cs.half())
    with pytest.raises(ValueError, match="qkv must be"):
        ff.rope_qk_(qkv.float(), cs)
    with pytest.raises(ValueError, match="qkv must be"):
        ff.rope_qk_(qkv[:, :, :2], cs)
    with pytest.raises(ValueError, match="float32"):
        ff.rope_qk_(qkv, ff.rope_table(4, 4, 100.0, "cuda"))  # more patch tokens than the sequence has
    with pytest.raises(ValueError, match="q_scale"):
        ff.rope_qk_(qkv, cs, q_scale=0.0)
