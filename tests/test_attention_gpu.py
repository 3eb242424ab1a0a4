"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a B200.

Structure follows the reference's kernel fuzz test for this op (tests/test_kernel_fuzz.py:269-296): seeded random
shapes and magnitudes, q / k / v as strided views of one packed tensor, compared with fp32 attention on the same
fp16 / bf16-rounded operands. Here the fp32 side is the oracle (`oracle/`), pinned to the reference's own modules
by `tests/test_oracle.py`. Tolerances (`conftest.assert_close`): max-abs <= 2e-2 and mean-abs <= 2e-3 at unit scale,
the reference's relative 2e-2 form for other magnitudes.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import fastforks_b200 as ff
from conftest import assert_close, load_golden
from oracle import attention_oracle as ao
from oracle import c_oracle

pytestmark = pytest.mark.gpu

DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}


@pytest.fixture(autouse=True)
def _kernels_ran_to_the_end():  # noqa: ANN202
    """After every test the device error word must be clear: no kernel gave up a wait."""
    yield
    assert ff.device_status() == 0


def packed_qkv(b: int, n: int, h: int, dtype: torch.dtype, mag: float, seed: int) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(b, n, 3, h, 64, generator=gen) * mag).to(dtype).cuda()


def oracle_of_packed(qkv: torch.Tensor, scale: float, **kw: object) -> np.ndarray:
    """Oracle output `[B, N, H, 64]` from the rounded operands of a packed `[B, N, 3, H, 64]` tensor."""
    q, k, v = (t.float().cpu().numpy() for t in qkv.permute(2, 0, 3, 1, 4))  # [B, H, N, 64]
    big = q.shape[0] * q.shape[1] * q.shape[2] * k.shape[2] > 4_000_000
    out = ao.attention(q, k, v, scale, **kw) if big or kw else c_oracle.attention(q, k, v, scale, threads=4)
    return out.transpose(0, 2, 1, 3)


def test_library_is_the_cuda_build() -> None:
    """The loaded binary is the sm_100a build of the sources beside it: its version string carries their digest."""
    from fastforks_b200 import _lib

    assert ff.resolve_mode("kernels") == "kernels"
    assert "sm_100a" in ff.version()
    assert ff.version().endswith(f"b200attn-src:{_lib.source_hash()}")


@pytest.mark.parametrize("name", ["dinov2_n97", "dinov2_n257_peaky", "timm_n197"])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_golden_vectors_of_the_reference_modules(name: str, dtype: str) -> None:
    """Inputs captured inside the reference's DINOv2 / timm attention modules; output vs the module's own output.
    The operands are rounded to 16 bits first, so the tolerance is the op-level one, not fp32 round-off."""
    g = load_golden(name)
    dt = DTYPES[dtype]
    q, k, v = (torch.from_numpy(g[x]).to(dt).cuda() for x in "qkv")
    got = ff.scaled_dot_product_attention(q, k, v, scale=float(g["scale"]))
    assert_close(got.float().cpu().numpy(), g["out"], unit_scale=name != "dinov2_n257_peaky", what=f"{name} {dtype}")
    # and exactly the oracle on the rounded operands
    ref = ao.attention(*(t.float().cpu().numpy() for t in (q, k, v)), float(g["scale"]))
    assert_close(got.float().cpu().numpy(), ref, unit_scale=name != "dinov2_n257_peaky", what=f"{name} {dtype} oracle")


@pytest.mark.parametrize("name", ["sam_window_14x14", "sam_grid_8x16"])
@pytest.mark.parametrize("form", ["decomposed", "dense"])
def test_golden_vectors_of_the_reference_sam_attention(name: str, form: str) -> None:
    """SAM `Attention.forward` with `add_decomposed_rel_pos`: the bias goes in as rel_h / rel_w (never materialised)
    or as the dense `[B, H, N, N]` tensor the reference function produced."""
    g = load_golden(name)
    q, k, v = (torch.from_numpy(g[x]).half().cuda() for x in "qkv")
    if form == "dense":
        got = ff.scaled_dot_product_attention(q, k, v, attn_mask=torch.from_numpy(g["bias"]).cuda(), scale=float(g["scale"]))
    else:
        rel_h, rel_w = ao.decomposed_terms(g["q"], g["rel_pos_h"], g["rel_pos_w"], g["hw"])
        rel = (torch.from_numpy(rel_h).cuda(), torch.from_numpy(rel_w).cuda())
        got = ff.scaled_dot_product_attention(q, k, v, scale=float(g["scale"]), rel=rel)
    assert_close(got.float().cpu().numpy(), g["out"], unit_scale=True, what=f"{name} {form}")


@pytest.mark.parametrize("variant", ["hh", "fh", "ff"])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_flash64_fuzz(variant: str, seed: int) -> None:
    """The reference's fuzz of `Flash64` (tests/test_kernel_fuzz.py:284-296): b in {1,2}, n in {1, [2,63], [65,400]},
    heads in [1,6], magnitudes 1.0 / 0.05 / 4.0, strided views of packed qkv, new contiguous output."""
    rng = np.random.default_rng(seed)
    attn = ff.Flash64(variant)
    for mag in (1.0, 0.05, 4.0):
        for n in (1, int(rng.integers(2, 64)), int(rng.integers(65, 401))):
            b, h = int(rng.integers(1, 3)), int(rng.integers(1, 7))
            qkv = packed_qkv(b, n, h, torch.float16, mag, seed * 1000 + n)
            q, k, v = qkv.unbind(2)
            got = attn(q, k, v, 0.125)
            assert got.shape == (b, n, h, 64)
            assert got.is_contiguous()
            assert_close(got.float().cpu().numpy(), oracle_of_packed(qkv, 0.125), unit_scale=mag == 1.0, what=f"b{b} n{n} h{h} mag{mag}")


@pytest.mark.parametrize("n", [1, 2, 63, 64, 65, 127, 128, 129, 196, 197, 255, 256, 257, 383, 385, 512, 513, 1370])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_tile_boundaries(n: int, dtype: str) -> None:
    """Sequence lengths around every tile edge of the kernel (128-row query tiles, 128-key tiles, two tiles per CTA)."""
    qkv = packed_qkv(2, n, 3, DTYPES[dtype], 1.0, n)
    q, k, v = qkv.unbind(2)
    got = ff.attention(q, k, v, layout="bnhd")
    assert_close(got.float().cpu().numpy(), oracle_of_packed(qkv, 0.125), unit_scale=True, what=f"n{n} {dtype}")


def test_output_rows_past_the_sequence_are_untouched() -> None:
    """Canary rows and columns around the output view must survive: the kernel writes its rows only."""
    b, n, h = 2, 197, 3
    qkv = packed_qkv(b, n, h, torch.float16, 1.0, 5)
    q, k, v = qkv.unbind(2)
    big = torch.full((b, n + 7, h + 1, 64), 77.0, dtype=torch.float16, device="cuda")
    out = big[:, 3 : 3 + n, :h]
    ff.attention(q, k, v, layout="bnhd", out=out)
    assert_close(out.float().cpu().numpy(), oracle_of_packed(qkv, 0.125), unit_scale=True)
    canary = big.clone()
    canary[:, 3 : 3 + n, :h] = 77.0
    assert bool((canary == 77.0).all())


def test_sdpa_layout_and_free_transpose() -> None:
    """`[B, H, N, 64]` permuted views as in `_vit_kernels` (src/fastforks/_optimize/transformer.py:286-289); the result's
    `transpose(1, 2).reshape(B, N, C)` is a view."""
    b, n, h = 2, 197, 12
    qkv = packed_qkv(b, n, h, torch.float16, 1.0, 11)
    q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
    got = ff.scaled_dot_product_attention(q, k, v)
    assert got.shape == (b, h, n, 64)
    flat = got.transpose(1, 2).reshape(b, n, h * 64)
    assert flat.data_ptr() == got.data_ptr()
    assert_close(got.transpose(1, 2).float().cpu().numpy(), oracle_of_packed(qkv, 0.125), unit_scale=True)


def test_cross_lengths_and_scale() -> None:
    gen = torch.Generator().manual_seed(3)
    q = torch.randn(2, 3, 150, 64, generator=gen).half().cuda()
    k = torch.randn(2, 3, 77, 64, generator=gen).half().cuda()
    v = torch.randn(2, 3, 77, 64, generator=gen).half().cuda()
    got = ff.scaled_dot_product_attention(q, k, v, scale=0.2)
    ref = ao.attention(*(t.float().cpu().numpy() for t in (q, k, v)), 0.2)
    assert_close(got.float().cpu().numpy(), ref, unit_scale=True)


@pytest.mark.parametrize("bias_dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_dense_bias_broadcast_and_mask(bias_dtype: torch.dtype) -> None:
    """A Swin-style `[1, heads, N, N]` bias broadcast over the batch (`_swin_block`, transformer.py:476-479), with
    -inf entries acting as a mask."""
    gen = torch.Generator().manual_seed(4)
    b, h, n = 3, 4, 147
    q, k, v = (torch.randn(b, h, n, 64, generator=gen).half().cuda() for _ in range(3))
    bias = torch.randn(1, h, n, n, generator=gen).to(bias_dtype)
    bias[..., 100:] = float("-inf")
    got = ff.scaled_dot_product_attention(q, k, v, attn_mask=bias.cuda())
    ref = ao.attention(*(t.float().cpu().numpy() for t in (q, k, v)), 0.125, bias.float().numpy())
    assert_close(got.float().cpu().numpy(), ref, unit_scale=True)


@pytest.mark.parametrize(
    ("b", "h", "nq", "nk", "bias_shape", "pad"),
    [
        (3, 4, 144, 144, (1, 4, 144, 144), 0),  # short schedule, broadcast over the batch
        (2, 3, 200, 200, (2, 1, 200, 200), 0),  # broadcast over the heads, ragged last tile
        (2, 3, 150, 77, (2, 3, 150, 77), 3),  # cross lengths; rows padded to 80 columns in a wider buffer
        (1, 2, 700, 1000, (1, 1, 700, 1000), 0),  # long schedule, one bias for everything
        (2, 5, 1370, 1370, (1, 5, 1370, 1370), 6),  # 518-px token count, rows padded to 1376
        (1, 2, 1, 64, (1, 2, 1, 64), 0),  # a single query row
    ],
)
@pytest.mark.parametrize("bias_dtype", [torch.float16, torch.bfloat16])
def test_dense_bias_in_tiles(b: int, h: int, nq: int, nk: int, bias_shape: tuple[int, ...], pad: int, bias_dtype: torch.dtype) -> None:
    """A 16-bit bias whose rows start on 16-byte boundaries reaches the kernel as 128 x 64 tiles through TMA (the
    other layouts take the row-wise loads): every broadcast form, padded rows, -inf columns, short and long schedule."""
    gen = torch.Generator().manual_seed(nq * 7 + nk)
    q = torch.randn(b, h, nq, 64, generator=gen).half().cuda()
    k, v = (torch.randn(b, h, nk, 64, generator=gen).half().cuda() for _ in range(2))
    bias = torch.randn(*bias_shape, generator=gen).to(bias_dtype)
    bias[..., nk - nk // 5 :] = float("-inf")
    bias[..., 0, :] = 3.0  # a row without any masked key
    wide = torch.full((*bias_shape[:3], nk + pad), 9.0, dtype=bias_dtype).cuda()
    wide[..., :nk] = bias.cuda()
    dev_bias = wide[..., :nk]
    assert (dev_bias.stride(2) % 8 == 0 or nq == 1) and dev_bias.data_ptr() % 16 == 0
    got = ff.scaled_dot_product_attention(q, k, v, attn_mask=dev_bias)
    assert ff.device_status() == 0
    ref = ao.attention(*(t.float().cpu().numpy() for t in (q, k, v)), 0.125, bias.float().numpy())
    assert_close(got.float().cpu().numpy(), ref, unit_scale=True, what=f"tiles {bias_shape} {bias_dtype}")
    # the same numbers through the row-wise loads: float32 values, and the 16-bit rows at an odd stride taken as given
    rowwise = ff.scaled_dot_product_attention(q, k, v, attn_mask=dev_bias.float())
    assert_close(got.float().cpu().numpy(), rowwise.float().cpu().numpy(), unit_scale=True, what="tiles against float32 rows")
    odd = torch.empty((*bias_shape[:3], nk + 1), dtype=bias_dtype).cuda()[..., :nk]
    odd.copy_(dev_bias)
    rowwise = ff.attention(q, k, v, bias=odd, _bias_as_given=True)
    assert_close(got.float().cpu().numpy(), rowwise.float().cpu().numpy(), unit_scale=True, what="tiles against 16-bit rows")
    # and `attention` pads such rows itself
    padded = ff.attention(q, k, v, bias=odd)
    assert torch.equal(padded, got)
    assert ff.tile_layout(odd).stride(2) % 8 == 0 and torch.equal(ff.tile_layout(odd), odd)
    assert ff.tile_layout(dev_bias).data_ptr() == dev_bias.data_ptr()


def test_swin_window_bias_layout_of_the_reference() -> None:
    """`_swin_bias` + `_swin_block` (src/fastforks/_optimize/transformer.py:455-479): windows folded into the head
    dimension, one `[1, nw * heads, 49, 56]` table (relative-position bias plus the shift mask, rows padded to 8)
    sliced to 49 columns and broadcast over the images."""
    gen = torch.Generator().manual_seed(49)
    images, nw, heads, n = 3, 16, 3, 49
    q, k, v = (torch.randn(images, n, nw * heads, 64, generator=gen).half().cuda().transpose(1, 2) for _ in range(3))
    table = torch.randn(1, nw * heads, n, n, generator=gen).half()
    table[:, ::5, :7, 30:] = -100.0  # the shift mask of some windows
    padded = torch.zeros(1, nw * heads, n, 56, dtype=torch.float16).cuda()
    padded[..., :n] = table.cuda()
    got = ff.scaled_dot_product_attention(q, k, v, attn_mask=padded[..., :n], scale=0.125)
    ref = ao.attention(*(t.float().cpu().numpy() for t in (q, k, v)), 0.125, table.float().numpy())
    assert_close(got.float().cpu().numpy(), ref, unit_scale=True, what="swin windows")
    # the second call of a geometry is launched from its remembered description: new values, other memory
    other = padded.clone()
    other[..., :n] = 0.5 * table.cuda()
    again = ff.scaled_dot_product_attention(q, k, v, attn_mask=other[..., :n], scale=0.125)
    ref = ao.attention(*(t.float().cpu().numpy() for t in (q, k, v)), 0.125, 0.5 * table.float().numpy())
    assert_close(again.float().cpu().numpy(), ref, unit_scale=True, what="swin windows, remembered launch")


def test_bool_mask_like_sdpa() -> None:
    gen = torch.Generator().manual_seed(6)
    q, k, v = (torch.randn(1, 2, 70, 64, generator=gen).half().cuda() for _ in range(3))
    mask = torch.rand(1, 1, 70, 70, generator=gen) > 0.3
    mask[..., 0] = True
    got = ff.scaled_dot_product_attention(q, k, v, attn_mask=mask.cuda())
    bias = np.where(mask.numpy(), 0.0, -np.inf).astype(np.float32)
    ref = ao.attention(*(t.float().cpu().numpy() for t in (q, k, v)), 0.125, bias)
    assert_close(got.float().cpu().numpy(), ref, unit_scale=True)


@pytest.mark.parametrize(("hw", "b", "h"), [((14, 14), 25, 12), ((64, 64), 1, 2), ((5, 9), 2, 3)])
def test_decomposed_bias_sam_shapes(hw: tuple[int, int], b: int, h: int) -> None:
    """SAM-B's two attention shapes (25 windows of 14x14 tokens; the 64x64 global grid) and a ragged grid."""
    gen = torch.Generator().manual_seed(hw[0])
    n = hw[0] * hw[1]
    q, k, v = (torch.randn(b, h, n, 64, generator=gen).half().cuda() for _ in range(3))
    rel_h = torch.randn(b, h, n, hw[0], generator=gen).half()
    rel_w = torch.randn(b, h, n, hw[1], generator=gen).half()
    got = ff.scaled_dot_product_attention(q, k, v, rel=(rel_h.cuda(), rel_w.cuda()))
    args = [t.float().cpu().numpy() for t in (q, k, v)]
    if n > 1024:  # dense bias of the global grid would be 4096^2 per head: check two heads through the C oracle
        ref = c_oracle.attention(*args, 0.125, rel=(rel_h.float().numpy(), rel_w.float().numpy()), threads=8)
    else:
        ref = ao.attention(*args, 0.125, ao.decomposed_bias(rel_h.float().numpy(), rel_w.float().numpy()))
    assert_close(got.float().cpu().numpy(), ref, unit_scale=True)


@pytest.mark.parametrize(
    ("hw", "nq", "dtype", "rel_dtype"),
    [((14, 14), 77, "fp16", torch.float32), ((14, 14), 300, "bf16", torch.bfloat16), ((64, 64), 130, "bf16", torch.bfloat16),
     ((3, 64), 200, "fp16", torch.float16), ((1, 64), 64, "fp16", torch.float16),
     ((8, 64), 300, "bf16", torch.bfloat16), ((16, 64), 130, "fp16", torch.float16), ((24, 64), 257, "fp16", torch.bfloat16)],
)
def test_decomposed_bias_fast_paths_cross_length(hw: tuple[int, int], nq: int, dtype: str, rel_dtype: torch.dtype) -> None:
    """The 14 x 14 and 64-wide forms of the decomposed bias with a query count that differs from the key count
    (one-tile and three-tile items) and with tables of another type than q / k / v."""
    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(nq)
    b, h, nk = 2, 2, hw[0] * hw[1]
    q = torch.randn(b, h, nq, 64, generator=gen).to(dt).cuda()
    k, v = (torch.randn(b, h, nk, 64, generator=gen).to(dt).cuda() for _ in range(2))
    rel_h = torch.randn(b, h, nq, hw[0], generator=gen).to(rel_dtype)
    rel_w = torch.randn(b, h, nq, hw[1], generator=gen).to(rel_dtype)
    got = ff.scaled_dot_product_attention(q, k, v, rel=(rel_h.cuda(), rel_w.cuda()))
    args = [t.float().cpu().numpy() for t in (q, k, v)]
    ref = c_oracle.attention(*args, 0.125, rel=(rel_h.float().numpy(), rel_w.float().numpy()), threads=8)
    assert_close(got.float().cpu().numpy(), ref, unit_scale=True)


def test_extreme_range_inputs_give_the_fp32_result() -> None:
    """The reference's overflow case (tests/test_flash64_guard.py:175-199): q[..., 0] = k[..., 0] = 400 overflows fp16
    accumulators there and needs its fallback chain; here accumulation is fp32, so the first answer is the fp32 one."""
    qkv = packed_qkv(1, 300, 2, torch.float16, 1.0, 9)
    qkv[:, :, 0, :, 0] = 400.0
    qkv[:, :, 1, :, 0] = 400.0
    q, k, v = qkv.unbind(2)
    got = ff.Flash64("hh")(q, k, v, 0.125)
    assert bool(torch.isfinite(got).all())
    assert_close(got.float().cpu().numpy(), oracle_of_packed(qkv, 0.125), unit_scale=False)


@pytest.mark.parametrize(
    ("b", "h", "n", "dtype"),
    [(8, 6, 1370, "fp16"), (4, 16, 1370, "bf16"), (1, 12, 4096, "fp16"), (25, 12, 196, "fp16")],
)
def test_full_size_configs_by_properties(b: int, h: int, n: int, dtype: str) -> None:
    """The benchmark configurations at full size, checked by properties that need no N^2 oracle:
    v = const -> output = const (rows of P sum to one); permuting the keys leaves the output unchanged;
    plus an oracle check of a strided sample of heads."""
    dt = DTYPES[dtype]
    qkv = packed_qkv(b, n, h, dt, 1.0, n + b)
    q, k, v = qkv.unbind(2)
    got = ff.attention(q, k, v, layout="bnhd")
    ones = torch.full_like(v, 0.5)
    const = ff.attention(q, k, ones, layout="bnhd")
    assert float((const.float() - 0.5).abs().max()) <= 4e-3  # one 16-bit rounding of the output
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(1)).cuda()
    shuffled = ff.attention(q, k[:, perm], v[:, perm], layout="bnhd")
    assert float((shuffled.float() - got.float()).abs().max()) <= 2e-2
    sample = qkv[:: max(1, b // 2), :, :, :: max(1, h // 2)].contiguous()
    ref = oracle_of_packed(sample, 0.125)
    assert_close(got[:: max(1, b // 2), :, :: max(1, h // 2)].float().cpu().numpy(), ref, unit_scale=True)


def oracle_of_heads(qkv: torch.Tensor, picks: list[tuple[int, int]], scale: float, rel: tuple | None = None) -> np.ndarray:
    """Oracle output `[len(picks), N, 64]` for the chosen (batch, head) pairs of a packed `[B, N, 3, H, 64]` tensor,
    one head at a time (a dense 4096 x 4096 bias is 64 MB per head)."""
    rows = []
    for b, h in picks:
        q, k, v = (qkv[b, :, i, h].float().cpu().numpy()[None, None] for i in range(3))
        bias = None
        if rel is not None:
            bias = ao.decomposed_bias(rel[0][b, h].float().cpu().numpy()[None, None], rel[1][b, h].float().cpu().numpy()[None, None])
        rows.append(ao.attention(q, k, v, scale, bias)[0, 0])
    return np.stack(rows)


@pytest.mark.parametrize(
    ("b", "h", "n", "dtype", "stride"),
    [(32, 24, 1370, "bf16", 97), (256, 12, 197, "fp16", 61), (8, 6, 1370, "fp16", 5), (4, 16, 1370, "bf16", 7)],
)
def test_benchmarked_shapes_against_the_oracle(b: int, h: int, n: int, dtype: str, stride: int) -> None:
    """Every shape a benchmark number is quoted on, launched at full size (the work split and the grid are the
    benchmark's) and compared with the oracle on a strided sample of (batch, head) pairs that always contains the
    first and the last head. A NaN canary in the output shows any row the launch failed to write."""
    qkv = packed_qkv(b, n, h, DTYPES[dtype], 1.0, seed=b * 1000 + n)
    q, k, v = qkv.unbind(2)
    out = torch.full((b, n, h, 64), float("nan"), dtype=DTYPES[dtype], device="cuda")
    ff.attention(q, k, v, scale=0.125, layout="bnhd", out=out)
    assert bool(torch.isfinite(out).all())
    ids = sorted({*range(0, b * h, stride), b * h - 1})
    picks = [(i // h, i % h) for i in ids]
    ref = oracle_of_heads(qkv, picks, 0.125)
    got = np.stack([out[bi, :, hi].float().cpu().numpy() for bi, hi in picks])
    assert_close(got, ref, unit_scale=True, what=f"[{b},{h},{n},64] {dtype}, {len(picks)} heads")


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_sam_global_grid_with_decomposed_bias_all_heads(dtype: str) -> None:
    """SAM-B's global layers at full size, `[1, 12, 4096, 64]` with `rel_h`, `rel_w` `[1, 12, 4096, 64]`: all twelve
    heads in one launch (384 query tiles on 148 CTAs, the benchmark's work split), every head against the oracle."""
    dt = DTYPES[dtype]
    b, h, n = 1, 12, 4096
    qkv = packed_qkv(b, n, h, dt, 1.0, seed=4096)
    gen = torch.Generator().manual_seed(64)
    rel = tuple(torch.randn(b, h, n, 64, generator=gen).to(dt).cuda() for _ in range(2))
    q, k, v = qkv.unbind(2)
    out = torch.full((b, n, h, 64), float("nan"), dtype=dt, device="cuda")
    ff.attention(q, k, v, scale=0.125, layout="bnhd", out=out, rel=rel)
    assert bool(torch.isfinite(out).all())
    picks = [(0, i) for i in range(h)]
    ref = oracle_of_heads(qkv, picks, 0.125, rel=rel)
    got = np.stack([out[0, :, i].float().cpu().numpy() for i in range(h)])
    assert_close(got, ref, unit_scale=True, what=f"SAM global grid {dtype}")


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_sam_windows_with_decomposed_bias_full_size(dtype: str) -> None:
    """SAM-B's windowed layers at full size: 25 windows x 12 heads of 14 x 14 tokens with `rel_h`, `rel_w`
    `[25, 12, 196, 14]`, packed-qkv views in, every (window, head) against the oracle."""
    dt = DTYPES[dtype]
    b, h, n = 25, 12, 196
    qkv = packed_qkv(b, n, h, dt, 1.0, seed=196)
    gen = torch.Generator().manual_seed(14)
    rel = tuple(torch.randn(b, h, n, 14, generator=gen).to(dt).cuda() for _ in range(2))
    q, k, v = qkv.unbind(2)
    out = torch.full((b, n, h, 64), float("nan"), dtype=dt, device="cuda")
    ff.attention(q, k, v, scale=0.125, layout="bnhd", out=out, rel=rel)
    bias = ao.decomposed_bias(rel[0].float().cpu().numpy(), rel[1].float().cpu().numpy())
    ref = oracle_of_packed(qkv, 0.125, bias=bias)
    assert_close(out.float().cpu().numpy(), ref, unit_scale=True, what=f"SAM windows {dtype}")


def test_two_streams_equal_one_stream() -> None:
    """Launches on two torch streams give the same bits as on one (the reference checks its kernels the same way,
    tests/test_threads.py:58-332)."""
    qkv = packed_qkv(4, 500, 6, torch.float16, 1.0, 21)
    q, k, v = qkv.unbind(2)
    base = ff.attention(q, k, v, layout="bnhd")
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    with torch.cuda.stream(s1):
        a = ff.attention(q, k, v, layout="bnhd")
    with torch.cuda.stream(s2):
        b_ = ff.attention(q, k, v, layout="bnhd")
    torch.cuda.synchronize()
    assert torch.equal(a, base)
    assert torch.equal(b_, base)


def test_cuda_graph_replay_equals_eager() -> None:
    """The launch is capturable (families capture whole forwards, src/fastforks/shared/cuda_graphs.py:1-17). The
    workspace of the capture stream is reserved before the capture, so the captured launch may split along the keys
    like the eager one; replays with new contents in the same buffers must follow them (the kernel leaves the
    workspace ready for its next launch, whatever launched it)."""
    qkv = packed_qkv(2, 1370, 6, torch.float16, 1.0, 22)
    q, k, v = qkv.unbind(2)
    out = torch.empty(2, 1370, 6, 64, dtype=torch.float16, device="cuda")
    eager = ff.attention(q, k, v, layout="bnhd").clone()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ff.reserve_workspace()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        ff.attention(q, k, v, layout="bnhd", out=out)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    for seed in (23, 24):
        qkv.copy_(packed_qkv(2, 1370, 6, torch.float16, 1.0, seed))
        graph.replay()
        torch.cuda.synchronize()
        assert_close(out.float().cpu().numpy(), oracle_of_packed(qkv, 0.125), unit_scale=True, what=f"replay seed {seed}")


def test_capture_without_a_reserved_workspace_runs_unsplit() -> None:
    """Nothing is allocated during a capture: a capture on a stream that never reserved a workspace launches the
    unsplit form, which must give the oracle's result too."""
    qkv = packed_qkv(1, 1370, 6, torch.float16, 1.0, 25)
    q, k, v = qkv.unbind(2)
    out = torch.empty(1, 1370, 6, 64, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):  # torch captures on a side stream of its own: no workspace there
        ff.attention(q, k, v, layout="bnhd", out=out)
    graph.replay()
    torch.cuda.synchronize()
    assert_close(out.float().cpu().numpy(), oracle_of_packed(qkv, 0.125), unit_scale=True)


SPLIT_SHAPES = [(1, 6, 1370, None), (8, 6, 1370, None), (1, 12, 4096, None), (3, 7, 900, None), (1, 2, 300, 1000), (1, 1, 129, 20000), (2, 16, 1370, None)]


@pytest.mark.parametrize(("b", "h", "n", "nk"), SPLIT_SHAPES)
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_key_split_launches_match_the_oracle_on_both_merge_routes(b: int, h: int, n: int, nk: int | None, dtype: str) -> None:
    """Long sequences whose query tiles level badly over 148 SMs are cut along the keys (`workspace` in
    include/b200_attn.h). Runs of two to twenty key tiles per CTA, items cut into up to five parts: the result must
    be the oracle's, on the usual route (the owner of a cut item folds the later parts in) and on the general one
    (a store warp folds them), with the same bits on both and on every repeat (the workspace is left ready)."""
    dt = DTYPES[dtype]
    nk = n if nk is None else nk
    gen = torch.Generator().manual_seed(n + nk)
    q = torch.randn(b, n, h, 64, generator=gen).to(dt).cuda()
    k, v = (torch.randn(b, nk, h, 64, generator=gen).to(dt).cuda() for _ in range(2))
    ref = ao.attention(*(t.float().cpu().numpy().transpose(0, 2, 1, 3) for t in (q, k, v)), 0.125).transpose(0, 2, 1, 3)
    outs = []
    for general in (False, True, False, True):
        out = torch.full((b, n, h, 64), float("nan"), dtype=dt, device="cuda")
        ff.attention(q, k, v, scale=0.125, layout="bnhd", out=out, _general_merge=general)
        assert_close(out.float().cpu().numpy(), ref, unit_scale=True, what=f"[{b},{h},{n}x{nk}] {dtype} general={general}")
        outs.append(out)
    assert all(torch.equal(outs[0], o) for o in outs[1:])


def test_key_split_with_decomposed_and_dense_bias() -> None:
    """The bias forms walk absolute key positions: a part that begins in the middle of the keys must read the
    right columns of a dense bias and the right rows of the decomposed tables (SAM's 64-wide form fetches `rel_h`
    in groups of four key tiles)."""
    gen = torch.Generator().manual_seed(77)
    b, h, n = 1, 3, 2048
    q, k, v = (torch.randn(b, n, h, 64, generator=gen).half().cuda() for _ in range(3))
    rel = tuple(torch.randn(b, h, n, 64 if i else 32, generator=gen).half().cuda() for i in range(2))
    args = [t.float().cpu().numpy().transpose(0, 2, 1, 3) for t in (q, k, v)]
    ref = ao.attention(*args, 0.125, ao.decomposed_bias(rel[0].float().cpu().numpy(), rel[1].float().cpu().numpy()))
    for general in (False, True):
        got = ff.attention(q, k, v, scale=0.125, layout="bnhd", rel=rel, _general_merge=general)
        assert_close(got.float().cpu().numpy().transpose(0, 2, 1, 3), ref, unit_scale=True, what=f"rel 32x64 general={general}")
    n = 1000
    q, k, v = (torch.randn(b, n, h, 64, generator=gen).half().cuda() for _ in range(3))
    bias = torch.randn(1, h, n, n, generator=gen).half()
    args = [t.float().cpu().numpy().transpose(0, 2, 1, 3) for t in (q, k, v)]
    ref = ao.attention(*args, 0.125, bias.float().numpy())
    got = ff.attention(q, k, v, scale=0.125, layout="bnhd", bias=bias.cuda())
    assert_close(got.float().cpu().numpy().transpose(0, 2, 1, 3), ref, unit_scale=True, what="dense bias, split")


def test_contract_violations_raise_before_launch() -> None:
    q = torch.zeros(1, 5, 2, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError, match="head dim"):
        ff.attention(q[..., :32], q[..., :32], q[..., :32], layout="bnhd")
    with pytest.raises(ValueError, match="unit last stride"):
        ff.attention(q.transpose(2, 3).contiguous().transpose(2, 3), q, q, layout="bnhd")
    odd = torch.zeros(1, 5, 2, 68, dtype=torch.float16, device="cuda")[..., 4:]  # token stride 136, base offset 8 bytes
    with pytest.raises(ValueError, match="aligned|multiple of 8"):
        ff.attention(odd, odd, odd, layout="bnhd")
    with pytest.raises(ValueError, match="requires grad"):
        ff.attention(q.clone().requires_grad_(), q, q, layout="bnhd")
    with pytest.raises(ValueError, match="exclusive"):
        ff.attention(q, q, q, layout="bnhd", bias=torch.zeros(5, 5, device="cuda"), rel=(q, q))


def test_a_wait_that_runs_out_sets_the_status_word_and_the_context_survives() -> None:
    """Every wait in the kernels is bounded. The self-test kernel waits 2 ms on a barrier nothing completes, gives up
    like the attention kernels do, and the next attention call still runs and is correct."""
    import ctypes

    from fastforks_b200 import _lib

    assert ff.device_status() == 0
    stream = torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())  # noqa: SLF001
    assert _lib.library().b200_attn_selftest_wait_limit(2000, ctypes.c_void_p(stream)) == 0
    assert ff.device_status() == 8  # read and cleared
    assert ff.device_status() == 0
    qkv = packed_qkv(1, 130, 2, torch.float16, 1.0, 3)
    q, k, v = qkv.unbind(2)
    got = ff.attention(q, k, v, layout="bnhd")
    assert_close(got.float().cpu().numpy(), oracle_of_packed(qkv, 0.125), unit_scale=True)


@pytest.mark.parametrize("depth", [1, 2, 3])
def test_host_operands_pipeline_matches_the_device_call(depth: int) -> None:
    """`HostAttention`: five packed tensors in pinned host memory through `depth` staging buffers, twice in a row
    (staging buffers are reused across calls); every output equals the plain device call bit for bit."""
    gen = torch.Generator().manual_seed(5)
    host_qkv = [torch.randn(2, 300, 3, 3, 64, generator=gen).half().pin_memory() for _ in range(5)]
    host_out = [torch.full((2, 300, 3, 64), float("nan"), dtype=torch.float16).pin_memory() for _ in range(5)]
    pipe = ff.HostAttention(depth=depth)
    for _ in range(2):
        pipe(host_qkv, host_out, 0.125)
        for x, o in zip(host_qkv, host_out):
            q, k, v = x.cuda().unbind(2)
            want = ff.attention(q, k, v, scale=0.125, layout="bnhd")
            assert torch.equal(o, want.cpu())
        for o in host_out:
            o.fill_(float("nan"))


def test_repeated_geometry_takes_the_remembered_launch_and_still_checks() -> None:
    """The second call with the same views goes through the remembered description: same result, new pointers are
    used, and a call that breaks the contract is still rejected before the launch."""
    qkv = packed_qkv(2, 197, 4, torch.float16, 1.0, seed=3)
    q, k, v = qkv.unbind(2)
    first = ff.attention(q, k, v, layout="bnhd")
    second = ff.attention(q, k, v, layout="bnhd")
    assert first.data_ptr() != second.data_ptr() and torch.equal(first, second)
    other = packed_qkv(2, 197, 4, torch.float16, 1.0, seed=4)
    third = ff.attention(*other.unbind(2), layout="bnhd")
    assert_close(third.float().cpu().numpy(), oracle_of_packed(other, 0.125), unit_scale=True, what="remembered launch")
    with pytest.raises(ValueError, match="requires grad"):
        ff.attention(q.clone().requires_grad_(), k, v, layout="bnhd")
    base = torch.zeros(100 * 4 * 64 + 8, device="cuda", dtype=torch.float16)
    aligned = base[: 100 * 4 * 64].view(1, 100, 4, 64)
    ff.attention(aligned, aligned, aligned, layout="bnhd")
    shifted = base[4 : 4 + 100 * 4 * 64].view(1, 100, 4, 64)  # same geometry, 8 bytes off: the library checks
    with pytest.raises(ValueError, match="16-byte"):
        ff.attention(shifted, shifted, shifted, layout="bnhd")


@pytest.mark.parametrize(("b", "n", "h"), [(1, 4096, 12), (2, 1370, 16), (1, 1370, 6), (3, 900, 7), (1, 197, 12), (5, 640, 31)])
def test_mixed_one_and_two_tile_items_cover_every_query_tile_once(b: int, n: int, h: int) -> None:
    """Grids smaller than, about equal to and larger than the SM count, where the host splits each head's query
    tiles into two-tile and one-tile items to level the CTAs' loads: every output row must be written, once, with
    the right head's result (NaN canary in the output buffer, oracle on the whole tensor)."""
    qkv = packed_qkv(b, n, h, torch.float16, 1.0, seed=n + b)
    out = torch.full((b, n, h, 64), float("nan"), dtype=torch.float16, device="cuda")
    q, k, v = qkv.unbind(2)
    ff.attention(q, k, v, scale=0.125, layout="bnhd", out=out)
    assert_close(out.float().cpu().numpy(), oracle_of_packed(qkv, 0.125), unit_scale=True, what=f"[{b},{h},{n},64]")


@pytest.mark.parametrize("schedule", ["auto", "long", "short"])
@pytest.mark.parametrize("n", [197, 160, 225, 256, 130, 1370])
def test_both_schedules_give_the_same_result(schedule: str, n: int) -> None:
    """The short schedule skips the exponentials of a last key tile's final 32 columns when they hold no key (197,
    160, 130 keys: taken; 225, 256: tile too full; 1370: only on request). Any hint must give the oracle's result,
    and the two schedules the same bits."""
    qkv = packed_qkv(2, n, 3, torch.float16, 1.0, seed=n)
    q, k, v = qkv.unbind(2)
    got = ff.attention(q, k, v, scale=0.125, layout="bnhd", schedule=schedule)
    assert_close(got.float().cpu().numpy(), oracle_of_packed(qkv, 0.125), unit_scale=True, what=f"{schedule} n={n}")
    other = ff.attention(q, k, v, scale=0.125, layout="bnhd", schedule="long")
    assert torch.equal(got, other)
