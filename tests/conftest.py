"""Shared test set-up: the `gpu` marker, import path, golden-vector loader and the error metrics.

`-m "not gpu"` runs on a machine without a GPU (oracle vs golden vectors, host-side contract checks, ABI symbols,
two-process gloo sharding). `-m gpu` tests are the parity tests proper: they call the CUDA library through its C ABI
and skip nowhere silently: without a CUDA device they are skipped by marker, with one they fail loudly if the
library is missing.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"
GOLDEN_CASES = ("dinov2_n97", "dinov2_n257_peaky", "timm_n197", "sam_window_14x14", "sam_grid_8x16")

# Per-op tolerances of the path for unit-scale inputs, and the reference's own relative form for scaled inputs
# (reference tests/test_kernel_fuzz.py:63-83: |got - ref| <= 2e-2 * max|ref| + 2^-24).
MAX_ABS = 2e-2
MEAN_ABS = 2e-3
REL = 2e-2


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config: pytest.Config, items: list[pytest.Item]) -> None:
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict[str, np.ndarray]:
    with np.load(GOLDEN / f"{name}.npz") as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(params=GOLDEN_CASES)
def golden(request: pytest.FixtureRequest) -> dict[str, np.ndarray]:
    case = load_golden(request.param)
    case["name"] = request.param
    return case


def assert_close(got: np.ndarray, ref: np.ndarray, *, unit_scale: bool, what: str = "") -> None:
    """The path's parity bar: finite where the reference is finite, max-abs and mean-abs within tolerance.

    `unit_scale=True`: absolute max-abs <= 2e-2 and mean-abs <= 2e-3 (inputs ~ N(0, 1)). Otherwise the reference's
    relative form, `|got - ref| <= 2e-2 * max|ref| + 2^-24`, with the mean bound scaled the same way.
    """
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.array_equal(np.isfinite(got), np.isfinite(ref)), f"{what}: finiteness differs"
    diff = np.abs(got - ref)
    diff = diff[np.isfinite(diff)]
    peak = float(np.abs(ref[np.isfinite(ref)]).max()) if diff.size else 0.0
    scale = 1.0 if unit_scale else max(peak, 1e-30)
    max_tol = MAX_ABS if unit_scale else REL * scale + 2.0**-24
    mean_tol = MEAN_ABS * scale
    assert diff.max() <= max_tol, f"{what}: max-abs {diff.max():.3e} > {max_tol:.3e} (max|ref| {peak:.3g})"
    assert diff.mean() <= mean_tol, f"{what}: mean-abs {diff.mean():.3e} > {mean_tol:.3e}"
