"""The CUDA-graph cache around launch-bound forwards (`fastforks_b200.GraphCache`), on a B200: a replayed forward
gives the bits of the eager one, geometries are captured after the stated number of eager calls, a forward that
cannot be captured stays eager, and the ViT-B/16 forward of one image is reported eager against replayed."""

from __future__ import annotations

import time

import pytest
import torch

import fastforks_b200 as ff
from fastforks_b200.vit import CONFIGS, ViTEncoder, seeded_state

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _kernels_ran_to_the_end():  # noqa: ANN202
    yield
    assert ff.device_status() == 0


def encoder(name: str = "vit-b16", dtype: torch.dtype = torch.float16) -> ViTEncoder:
    cfg = CONFIGS[name]
    return ViTEncoder(cfg, seeded_state(cfg, seed=3, qk_gain=4.0), device="cuda", dtype=dtype)


def test_replay_equals_eager_and_geometries_get_their_own_graphs() -> None:
    enc = encoder()
    cache = ff.GraphCache(enc, capture_after=1)
    gen = torch.Generator().manual_seed(0)
    one = torch.rand(1, 3, 224, 224, generator=gen).half().cuda()
    two = torch.rand(2, 3, 224, 224, generator=gen).half().cuda()
    want_one, want_two = enc(one), enc(two)
    assert torch.equal(cache(one), want_one) and cache.stats == {"eager": 1, "captured": 0, "replayed": 0, "failed": 0, "evicted": 0}
    assert torch.equal(cache(one), want_one) and cache.stats["captured"] == 1 and cache.stats["replayed"] == 1
    other = torch.rand(1, 3, 224, 224, generator=gen).half().cuda()
    assert torch.equal(cache(other), enc(other)) and cache.stats["replayed"] == 2  # new values through the static buffers
    assert torch.equal(cache(two), want_two) and cache.stats["eager"] == 2  # a new geometry starts eager
    assert torch.equal(cache(two), want_two) and cache.stats["captured"] == 2
    first = cache(one)
    second = cache(other)  # must not change `first`: callers get copies
    assert torch.equal(first, want_one) and not torch.equal(first, second)
    cache.release()
    assert torch.equal(cache(one), want_one) and cache.stats["eager"] == 3


def test_long_sequences_replay_with_the_key_split_plan() -> None:
    """518 px, batch 2 of ViT-S/14: 1370 tokens, a launch the planner splits along the keys when it has scratch memory.
    The cache reserves that memory for the capture stream before it captures."""
    enc = encoder("dinov2-vits14", torch.bfloat16)
    cache = ff.GraphCache(enc)
    images = torch.rand(2, 3, 518, 518, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
    want = enc(images)
    cache(images)
    for _ in range(3):
        assert torch.equal(cache(images), want)
    assert cache.stats["replayed"] == 3


@pytest.mark.filterwarnings("ignore:The CUDA Graph is empty")
def test_a_forward_that_cannot_be_captured_stays_eager() -> None:
    calls = []

    def forward(x: torch.Tensor) -> torch.Tensor:
        calls.append(1)
        if torch.cuda.is_current_stream_capturing():
            msg = "this forward refuses to be captured"
            raise RuntimeError(msg)
        return x * 2

    cache = ff.GraphCache(forward)
    x = torch.ones(4, device="cuda")
    for _ in range(4):
        assert torch.equal(cache(x), x * 2)
    assert cache.stats["failed"] == 1 and cache.stats["captured"] == 0 and cache.stats["eager"] == 4


def test_the_cache_holds_at_most_max_graphs() -> None:
    cache = ff.GraphCache(lambda x: x + 1, max_graphs=2)
    for n in (1, 2, 3):
        x = torch.zeros(n, device="cuda")
        cache(x)
        assert torch.equal(cache(x), x + 1)
    assert cache.stats["captured"] == 3 and cache.stats["evicted"] == 1
    with pytest.raises(ValueError, match="at least 1"):
        ff.GraphCache(lambda x: x, capture_after=0)


def test_one_image_of_vit_b16_eager_against_replayed(capsys: pytest.CaptureFixture[str]) -> None:
    """The launch-bound configuration (one image, 197 tokens): wall time per forward, eager and replayed."""
    enc = encoder()
    cache = ff.GraphCache(enc)
    image = torch.rand(1, 3, 224, 224).half().cuda()
    cache(image)
    cache(image)

    def per_call(fn) -> float:  # noqa: ANN001
        for _ in range(3):
            fn(image)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(20):
            fn(image)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / 20 * 1e3

    eager, replayed = per_call(enc), per_call(cache)
    with capsys.disabled():
        print(f"\nvit-b16, one image: {eager:.3f} ms per forward eager, {replayed:.3f} ms replayed from a graph")
    assert replayed < eager
