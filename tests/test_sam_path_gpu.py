"""SAM's attention with the decomposed relative-position term, side by side with the path the reference runs.

For SAM the reference's kernels mode does not call `flash64_*`: it folds the bias into the dot product by widening
q and k ("augmented", `src/fastforks/promptable_segmentation/models/sam/fast.py:92-113`: `q' = [q * scale | rel_h |
rel_w | 0]`, `k' = [k | onehot(kh) | onehot(kw) | 0]`, `v' = [v | 0]`, head dim 96 for 14 x 14 windows and 192 for the
64 x 64 grid) and calls `F.scaled_dot_product_attention(..., scale=1.0)[..., :64]` (`fused.py:80-86`). This file
restates that construction (test infrastructure: torch ops only) and

  * checks this library's `rel=(rel_h, rel_w)` call against it on the same packed qkv and tables (same operands, two
    different routes to the same logits: the bar is the path's op-level tolerance), and
  * times both, each including the two einsums that produce `rel_h`, `rel_w` from q and the tables (both routes
    need them) and, for the reference's route, the three concatenations it needs on top; and this library once more
    with its own producer kernel (`b200_sam_rel_terms`) in place of the einsums, which is also checked against the
    oracle on its own.

Speed is reported (JSON to $B200_SAM_SIDE_BY_SIDE when set), not gated.
"""

from __future__ import annotations

import json
import os

import pytest
import torch

import fastforks_b200 as ff
from conftest import assert_close

pytestmark = pytest.mark.gpu

HEADS, DIM = 12, 64
SHAPES = {"sam-vit-b windows [25,12,196,64]": (25, 14), "sam-vit-b global [1,12,4096,64]": (1, 64)}


def onehot_keys(side: int) -> torch.Tensor:
    """`[side * side, 2 * side]`: key (a, c) has a one in column a and in column side + c (fast.py:85-89)."""
    eye = torch.eye(side, device="cuda", dtype=torch.float16)
    return torch.cat([eye.repeat_interleave(side, 0), eye.repeat(side, 1)], 1)


def rel_terms(qkv: torch.Tensor, rh: torch.Tensor, rw: torch.Tensor, side: int) -> tuple[torch.Tensor, torch.Tensor]:
    """`rel_h`, `rel_w` `[B, heads, N, side]` from the unscaled q and the tables `[side, side, 64]` (fast.py:104-106)."""
    b, n = qkv.shape[:2]
    r_q = qkv[:, :, 0].reshape(b, side, side, HEADS, DIM)
    rel_h = torch.einsum("bhwnc,hkc->bnhwk", r_q, rh).reshape(b, HEADS, n, side)
    rel_w = torch.einsum("bhwnc,wkc->bnhwk", r_q, rw).reshape(b, HEADS, n, side)
    return rel_h, rel_w


def reference_route(qkv: torch.Tensor, rh: torch.Tensor, rw: torch.Tensor, onehot: torch.Tensor, side: int) -> torch.Tensor:
    """Widened operands + SDPA with scale 1, sliced back to 64 columns: `[B, heads, N, 64]` (fast.py:92-113, 128-135)."""
    b, n = qkv.shape[:2]
    q, k, v = qkv.unbind(2)
    rel_h, rel_w = rel_terms(qkv, rh, rw, side)
    pad = -(DIM + 2 * side) % 8
    qt = q.transpose(1, 2)
    zeros = qt.new_zeros(b, HEADS, n, pad)
    qa = torch.cat([qt * DIM**-0.5, rel_h, rel_w, zeros], -1)
    ka = torch.cat([k.transpose(1, 2), onehot.expand(b, HEADS, n, 2 * side), zeros], -1)
    va = torch.cat([v.transpose(1, 2), qt.new_zeros(b, HEADS, n, 2 * side + pad)], -1)
    return torch.nn.functional.scaled_dot_product_attention(qa, ka, va, scale=1.0)[..., :DIM]


def this_library(qkv: torch.Tensor, rh: torch.Tensor, rw: torch.Tensor, side: int) -> torch.Tensor:
    """The same attention through `rel=`: q, k, v stay 64 wide views of the packed tensor. `[B, N, heads, 64]`."""
    q, k, v = qkv.unbind(2)
    return ff.attention(q, k, v, scale=DIM**-0.5, layout="bnhd", rel=rel_terms(qkv, rh, rw, side))


def this_library_with_producer(qkv: torch.Tensor, pos_h: torch.Tensor, pos_w: torch.Tensor, side: int) -> torch.Tensor:
    """The same with `rel_h`, `rel_w` from this library's producer kernel, which reads q in place and the module's
    `[2 * side - 1, 64]` parameters instead of gathered tables."""
    q, k, v = qkv.unbind(2)
    return ff.attention(q, k, v, scale=DIM**-0.5, layout="bnhd", rel=ff.sam_rel_terms(q, pos_h, pos_w, side))


def gathered(pos: torch.Tensor, side: int) -> torch.Tensor:
    """`[side, side, 64]` table of a `[2 * side - 1, 64]` parameter (upstream `get_rel_pos`, equal sizes)."""
    idx = torch.arange(side, device=pos.device)
    return pos[(idx[:, None] - idx[None, :]) + (side - 1)]


@pytest.mark.parametrize(("b", "side", "dtype"), [(25, 14, torch.float16), (1, 64, torch.float16), (3, 14, torch.bfloat16), (2, 8, torch.bfloat16), (1, 64, torch.bfloat16)])
def test_producer_kernel_matches_the_oracle(b: int, side: int, dtype: torch.dtype) -> None:
    """`b200_sam_rel_terms` against the oracle's restatement of the two einsums of `add_decomposed_rel_pos`
    (oracle/attention_oracle.py: decomposed_terms) on the rounded operands; results are rounded to 16 bits once."""
    from oracle import attention_oracle as ao

    gen = torch.Generator().manual_seed(side + b)
    qkv = torch.randn(b, side * side, 3, HEADS, DIM, generator=gen).to(dtype).cuda()
    pos_h, pos_w = ((torch.randn(2 * side - 1, DIM, generator=gen) * 0.1).to(dtype).cuda() for _ in range(2))
    rel_h, rel_w = ff.sam_rel_terms(qkv[:, :, 0], pos_h, pos_w, side)
    q = qkv[:, :, 0].float().cpu().numpy().transpose(0, 2, 1, 3)
    want_h, want_w = ao.decomposed_terms(q, pos_h.float().cpu().numpy(), pos_w.float().cpu().numpy(), (side, side))
    assert_close(rel_h.float().cpu().numpy(), want_h, unit_scale=False, what=f"rel_h side {side} {dtype}")
    assert_close(rel_w.float().cpu().numpy(), want_w, unit_scale=False, what=f"rel_w side {side} {dtype}")


def test_producer_kernel_rejects_what_it_cannot_take() -> None:
    q = torch.zeros(1, 25, 2, 64, dtype=torch.float16, device="cuda")
    pos = torch.zeros(9, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError, match="grid"):
        ff.sam_rel_terms(q, pos, pos, 4)
    with pytest.raises(ValueError, match="even"):
        ff.sam_rel_terms(q, pos, pos, 5)
    with pytest.raises(ValueError, match="rel_pos_h"):
        ff.sam_rel_terms(q[:, :16], pos, pos, 4)


def operands(b: int, side: int, seed: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    qkv = torch.randn(b, side * side, 3, HEADS, DIM, generator=gen).half().cuda()
    rh, rw = ((torch.randn(side, side, DIM, generator=gen) * 0.1).half().cuda() for _ in range(2))
    return qkv, rh, rw


def parameters(side: int, seed: int) -> tuple[torch.Tensor, torch.Tensor]:
    gen = torch.Generator().manual_seed(1000 + seed)
    return tuple((torch.randn(2 * side - 1, DIM, generator=gen) * 0.1).half().cuda() for _ in range(2))


@pytest.mark.parametrize("name", list(SHAPES))
def test_same_result_as_the_reference_route(name: str) -> None:
    b, side = SHAPES[name]
    qkv, _, _ = operands(b, side, seed=side)
    pos_h, pos_w = parameters(side, side)
    rh, rw = gathered(pos_h, side), gathered(pos_w, side)
    theirs = reference_route(qkv, rh, rw, onehot_keys(side), side).transpose(1, 2)
    ours = this_library(qkv, rh, rw, side)
    assert_close(ours.float().cpu().numpy(), theirs.float().cpu().numpy(), unit_scale=True, what=name)
    fused = this_library_with_producer(qkv, pos_h, pos_w, side)
    assert_close(fused.float().cpu().numpy(), theirs.float().cpu().numpy(), unit_scale=True, what=name + " (producer kernel)")
    assert ff.device_status() == 0


def _time_us(fn, reps: int = 20) -> float:  # noqa: ANN001
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / reps * 1e3)
    return best


def test_times_side_by_side_with_the_reference_route() -> None:
    rows = {}
    for name, (b, side) in SHAPES.items():
        sets = [operands(b, side, seed=i) for i in range(8)]  # 8 x 19-30 MB of qkv: rotating, larger than L2 together
        onehot = onehot_keys(side)
        state = {"i": 0}

        def nxt() -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
            state["i"] = (state["i"] + 1) % len(sets)
            return sets[state["i"]]

        pos_h, pos_w = parameters(side, 0)
        rel_only = _time_us(lambda: rel_terms(*nxt(), side))
        producer_only = _time_us(lambda: ff.sam_rel_terms(nxt()[0][:, :, 0], pos_h, pos_w, side))
        ours = _time_us(lambda: this_library(*nxt(), side))
        ours_producer = _time_us(lambda: this_library_with_producer(nxt()[0], pos_h, pos_w, side))
        theirs = _time_us(lambda: reference_route(*nxt(), onehot, side))
        rows[name] = {"rel_einsums_us": rel_only, "producer_kernel_us": producer_only, "this_library_with_einsums_us": ours,
                      "this_library_with_producer_kernel_us": ours_producer,
                      "reference_augmented_sdpa_with_einsums_us": theirs, "speedup": theirs / ours_producer}  # fmt: skip
        print(name, json.dumps(rows[name]))
    assert all(r["this_library_with_einsums_us"] > 0 for r in rows.values())
    assert ff.device_status() == 0
    path = os.environ.get("B200_SAM_SIDE_BY_SIDE")
    if path:
        with open(path, "w") as f:
            json.dump(rows, f, indent=1)
