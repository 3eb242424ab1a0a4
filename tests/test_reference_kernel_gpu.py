"""Side by side with the reference's own CUDA kernel (`flash64_*`, compiled for sm_100 from the reference checkout
into `oracle/_ref/`, see `oracle/Makefile`): the results of the two kernels on the same operands, and their times.

The reference kernel is test infrastructure, loaded only here. Where `oracle/_ref/libref_flash64.so` was not built
(no reference checkout at build time) these tests are skipped with that reason.
"""

from __future__ import annotations

import json
import os

import pytest
import torch

import fastforks_b200 as ff
from conftest import assert_close
from oracle import ref_flash64

pytestmark = [
    pytest.mark.gpu,
    pytest.mark.skipif(not ref_flash64.available(), reason="oracle/_ref/libref_flash64.so is not built"),
]


def packed(b: int, n: int, h: int, mag: float, seed: int) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(b, n, 3, h, 64, generator=gen) * mag).half().cuda()


@pytest.mark.parametrize("variant", ["hh", "fh", "ff"])
@pytest.mark.parametrize(("b", "n", "h"), [(1, 197, 12), (2, 1370, 6), (3, 64, 2), (1, 577, 5), (2, 130, 3)])
@pytest.mark.parametrize("mag", [1.0, 0.05, 4.0])
def test_same_results_as_the_reference_kernel(variant: str, b: int, n: int, h: int, mag: float) -> None:
    """Magnitudes and layout of the reference's fuzz test (tests/test_kernel_fuzz.py:284-296). Both kernels round
    P to fp16 and differ in accumulation order and width, so the bar is the path's op-level tolerance."""
    qkv = packed(b, n, h, mag, seed=n + h)
    q, k, v = qkv.unbind(2)
    theirs = ref_flash64.run(variant, q, k, v, 0.125)
    ours = ff.Flash64(variant)(q, k, v, 0.125)
    assert ours.shape == theirs.shape and ours.is_contiguous()
    assert_close(ours.float().cpu().numpy(), theirs.float().cpu().numpy(), unit_scale=mag == 1.0,
                 what=f"{variant} [{b},{n},{h},64] mag {mag}")
    assert ff.device_status() == 0


def _time_us(fn, reps: int = 30) -> float:  # noqa: ANN001
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


SHAPES = {
    "dinov2-vits14 [8,6,1370,64]": (8, 1370, 6),
    "depth-anything-v2-l [4,16,1370,64]": (4, 1370, 16),
    "dinov2-vitg14 [32,24,1370,64]": (32, 1370, 24),
    "sam-vit-b global, no bias [1,12,4096,64]": (1, 4096, 12),
    "vit-b16 [256,12,197,64]": (256, 197, 12),
    "vit-b16 [1,12,197,64]": (1, 197, 12),
}


def test_times_side_by_side() -> None:
    """Device time per launch (CUDA events, best of 5 runs of 30 back-to-back launches over rotating buffers larger
    than L2) of this library, of the reference kernel under the reference's launch rule, and of torch's SDPA, which
    the reference's kernels mode calls for timm ViTs and SAM. Written as JSON to $B200_SIDE_BY_SIDE when set.
    Asserts only that every kernel ran; speed is reported, not gated."""
    rows = {}
    for name, (b, n, h) in SHAPES.items():
        copies = max(2, min(32, int(300e6 // (b * n * h * 64 * 8)) + 1))
        qkvs = [packed(b, n, h, 1.0, seed=i) for i in range(copies)]
        out = torch.empty(b, n, h, 64, device="cuda", dtype=torch.float16)
        state = {"i": 0}

        def nxt() -> tuple[torch.Tensor, ...]:
            state["i"] = (state["i"] + 1) % copies
            return qkvs[state["i"]].unbind(2)

        ours = _time_us(lambda: ff.attention(*nxt(), scale=0.125, layout="bnhd", out=out))
        ref = {v: _time_us(lambda v=v: ref_flash64.run(v, *nxt(), 0.125, out=out)) for v in ("hh", "ff")}

        def sdpa() -> None:
            q, k, v = (t.transpose(1, 2) for t in nxt())
            torch.nn.functional.scaled_dot_product_attention(q, k, v, scale=0.125)

        lib = _time_us(sdpa)
        flops = 4.0 * b * h * n * n * 64
        rows[name] = {
            "ours_us": ours, "reference_flash64_hh_us": ref["hh"], "reference_flash64_ff_us": ref["ff"],
            "torch_sdpa_us": lib, "ours_tflops": flops / ours / 1e6, "reference_hh_tflops": flops / ref["hh"] / 1e6,
        }  # fmt: skip
        print(name, json.dumps(rows[name]))
        del qkvs
    assert all(r["ours_us"] > 0 and r["reference_flash64_hh_us"] > 0 for r in rows.values())
    assert ff.device_status() == 0
    path = os.environ.get("B200_SIDE_BY_SIDE")
    if path:
        with open(path, "w") as f:
            json.dump(rows, f, indent=1)
