"""SAM's attention with the decomposed relative-position term, side by side with the path the reference runs.

For SAM the reference's kernels mode does not call `flash64_*`: it folds the bias into the dot product by widening
q and k ("augmented", `src/fastforks/promptable_segmentation/models/sam/fast.py:92-113`: `q' = [q * scale | rel_h |
rel_w | 0]`, `k' = [k | onehot(kh) | onehot(kw) | 0]`, `v' = [v | 0]`, head dim 96 for 14 x 14 windows and 192 for the
64 x 64 grid) and calls `F.scaled_dot_product_attention(..., scale=1.0)[..., :64]` (`fused.py:80-86`). This file
restates that construction (test infrastructure: torch ops only) and

  * checks this library's `rel=(rel_h, rel_w)` call against it on the same packed qkv and tables (same operands, two
    different routes to the same logits: the bar is the path's op-level tolerance), and
  * times both, each including the two einsums that produce `rel_h`, `rel_w` from q and the tables (both routes
    need them) and, for the reference's route, the three concatenations it needs on top.

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


def operands(b: int, side: int, seed: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    qkv = torch.randn(b, side * side, 3, HEADS, DIM, generator=gen).half().cuda()
    rh, rw = ((torch.randn(side, side, DIM, generator=gen) * 0.1).half().cuda() for _ in range(2))
    return qkv, rh, rw


@pytest.mark.parametrize("name", list(SHAPES))
def test_same_result_as_the_reference_route(name: str) -> None:
    b, side = SHAPES[name]
    qkv, rh, rw = operands(b, side, seed=side)
    theirs = reference_route(qkv, rh, rw, onehot_keys(side), side).transpose(1, 2)
    ours = this_library(qkv, rh, rw, side)
    assert_close(ours.float().cpu().numpy(), theirs.float().cpu().numpy(), unit_scale=True, what=name)
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

        rel_only = _time_us(lambda: rel_terms(*nxt(), side))
        ours = _time_us(lambda: this_library(*nxt(), side))
        theirs = _time_us(lambda: reference_route(*nxt(), onehot, side))
        rows[name] = {"rel_einsums_us": rel_only, "this_library_with_einsums_us": ours,
                      "reference_augmented_sdpa_with_einsums_us": theirs, "speedup": theirs / ours}  # fmt: skip
        print(name, json.dumps(rows[name]))
    assert all(r["this_library_with_einsums_us"] > 0 for r in rows.values())
    assert ff.device_status() == 0
    path = os.environ.get("B200_SAM_SIDE_BY_SIDE")
    if path:
        with open(path, "w") as f:
            json.dump(rows, f, indent=1)
