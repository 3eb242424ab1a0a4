"""Parity of the fused-epilogue GEMM (`b200_gemm`, through `fastforks_b200.gemm`) with its CPU oracle on a B200.

The oracle (`oracle/gemm_oracle.py`) restates the epilogue formula of the reference's `dpt_fused` GEMMs and is pinned
to torch's `F.linear` / `F.gelu` / residual arithmetic by `tests/test_oracle.py`. Operands are rounded to 16 bits
first, accumulation is fp32 on both sides and the result is rounded to 16 bits once, so the bar is the reference's
relative form for this library's GEMMs: `|got - ref| <= 2e-2 * max|ref|`, mean within 2e-3 of that scale
(`conftest.assert_close`, reference tests/test_kernel_fuzz.py:63-83).
"""

from __future__ import annotations

import pytest
import torch

import fastforks_b200 as ff
from conftest import assert_close
from oracle import gemm_oracle as go

pytestmark = pytest.mark.gpu
DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}


@pytest.fixture(autouse=True)
def _kernels_ran_to_the_end():  # noqa: ANN202
    yield
    assert ff.device_status() == 0


def operands(m: int, n: int, k: int, dtype: torch.dtype, seed: int):  # noqa: ANN201
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=gen).to(dtype)
    w = (torch.randn(n, k, generator=gen) * k**-0.5).to(dtype)
    bias = torch.randn(n, generator=gen).to(dtype)
    scale = torch.rand(n, generator=gen) + 0.5
    res = torch.randn(m, n, generator=gen).to(dtype)
    return x, w, bias, scale, res


def check(got: torch.Tensor, x, w, bias=None, scale=None, res=None, act: int = 0, what: str = "") -> None:  # noqa: ANN001, PLR0913
    f = lambda t: None if t is None else t.float().cpu().numpy()  # noqa: E731
    ref = go.gemm_epilogue(f(x), f(w), f(bias), f(scale), f(res), act)
    assert_close(got.float().cpu().numpy(), ref, unit_scale=False, what=what)


# tile edges of the three tile shapes (128 x 128, 128 x 256, 256 x 256), k tails, the smallest problem, ViT shapes
SHAPES = [(1, 8, 8), (128, 128, 64), (129, 136, 72), (255, 256, 64), (257, 264, 200), (300, 1000, 520), (1370, 1152, 384),
          (5480, 1024, 1024), (2740, 3072, 1024), (700, 4096, 1024)]  # fmt: skip


@pytest.mark.parametrize(("m", "n", "k"), SHAPES)
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_linear_with_bias(m: int, n: int, k: int, dtype: str) -> None:
    x, w, bias, _, _ = (t.cuda() for t in operands(m, n, k, DTYPES[dtype], seed=m + n))
    out = torch.full((m, n), float("nan"), dtype=DTYPES[dtype], device="cuda")
    got = ff.gemm(x, w, bias, out=out)
    assert got is out and bool(torch.isfinite(out).all())
    check(got, x, w, bias, what=f"[{m},{n},{k}] {dtype}")


@pytest.mark.parametrize("act", [ff.ACT_RELU, ff.ACT_GELU, ff.ACT_GELU_TANH])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_activations(act: int, dtype: str) -> None:
    x, w, bias, _, _ = (t.cuda() for t in operands(777, 520, 264, DTYPES[dtype], seed=act))
    check(ff.gemm(x, w, bias, act=act), x, w, bias, act=act, what=f"act {act} {dtype}")


@pytest.mark.parametrize(("m", "n", "k"), [(300, 264, 136), (5480, 1024, 4096), (1370, 1536, 1536)])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_layerscale_and_in_place_residual(m: int, n: int, k: int, dtype: str) -> None:
    """`x += gamma * (o @ W^T + b)` as one call: scale = gamma (fp32), res = out = x, the block-output form of the
    reference's fused path (src/fastforks/shared/depth_anything_v2/fast_vit.py:199-208)."""
    x, w, bias, scale, res = (t.cuda() for t in operands(m, n, k, DTYPES[dtype], seed=k))
    before = res.clone()
    got = ff.gemm(x, w, bias, scale=scale, res=res, out=res)
    assert got.data_ptr() == res.data_ptr()
    check(got, x, w, bias, scale, before, what=f"in place [{m},{n},{k}] {dtype}")
    other = ff.gemm(x, w, None, res=before, act=ff.ACT_RELU)  # no bias, residual into a new tensor, then relu
    check(other, x, w, None, None, before, act=ff.ACT_RELU, what="no bias + residual + relu")


def test_row_strided_views_and_leading_dims() -> None:
    """x, res and out as 2-D views with a row stride (lda, lres, ldy) and x with leading batch dims."""
    gen = torch.Generator().manual_seed(5)
    big = torch.randn(200, 160, generator=gen).half().cuda()
    x = big[:, 8:80]  # [200, 72], row stride 160
    w = (torch.randn(48, 72, generator=gen) * 0.1).half().cuda()
    canvas = torch.full((200, 96), 7.0, dtype=torch.float16, device="cuda")
    out = canvas[:, 16:64]
    ff.gemm(x, w, out=out)
    check(out, x, w, what="strided")
    assert bool((canvas[:, :16] == 7.0).all()) and bool((canvas[:, 64:] == 7.0).all())  # nothing outside the view
    x3 = torch.randn(3, 50, 72, generator=gen).half().cuda()
    got = ff.gemm(x3, w)
    assert got.shape == (3, 50, 48)
    check(got.reshape(150, 48), x3.reshape(150, 72), w, what="leading dims")


def test_contract_violations_raise_before_launch() -> None:
    x = torch.zeros(16, 64, dtype=torch.float16, device="cuda")
    w = torch.zeros(32, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError, match="weight"):
        ff.gemm(x, w.t())
    with pytest.raises(ValueError, match="multiples of 8"):
        ff.gemm(x[:, :60].contiguous(), w[:, :60].contiguous())
    with pytest.raises(ValueError, match="bias"):
        ff.gemm(x, w, torch.zeros(31, dtype=torch.float16, device="cuda"))
    with pytest.raises(ValueError, match="scale"):
        ff.gemm(x, w, scale=torch.zeros(32, dtype=torch.float16, device="cuda"))
    with pytest.raises(ValueError, match="act"):
        ff.gemm(x, w, act=3)
    with pytest.raises(ValueError, match="requires grad"):
        ff.gemm(x.clone().requires_grad_(), w)
