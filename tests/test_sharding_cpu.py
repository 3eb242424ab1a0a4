"""The multi-GPU path on CPU: two gloo ranks shard a batch image-wise, each computes its shard independently,
rank 0 gathers. No collective runs between the shard computations, as on the GPUs."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fastforks_b200.sharding import gather_to_rank0, image_range

ROOT = Path(__file__).resolve().parent.parent


def test_image_range_partitions_exactly() -> None:
    for total in (0, 1, 7, 8, 255, 256, 257):
        for world in (1, 2, 3, 4, 8):
            ranges = [image_range(total, world, r) for r in range(world)]
            flat = [i for r in ranges for i in r]
            assert flat == list(range(total))
            sizes = [len(r) for r in ranges]
            assert max(sizes) - min(sizes) <= 1
            assert sizes == sorted(sizes, reverse=True)
    assert [len(image_range(256, 8, r)) for r in range(8)] == [32] * 8
    with pytest.raises(ValueError, match="invalid"):
        image_range(4, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, total: int, out_path: str) -> None:
    sys.path.insert(0, str(ROOT))
    from oracle import attention_oracle as ao  # the checker stands in for the GPU kernel on CPU ranks

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(0)  # identical seeded inputs on every rank, no broadcast
        qkv = torch.randn(total, 3, 2, 33, 64, generator=gen)
        mine = image_range(total, world, rank)
        local = qkv[mine.start : mine.stop]
        out = torch.from_numpy(ao.attention(local[:, 0].numpy(), local[:, 1].numpy(), local[:, 2].numpy()))
        full = gather_to_rank0(out, total)
        if rank == 0:
            np.save(out_path, full.numpy())
        else:
            assert full is None
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [5, 8])
def test_two_ranks_shard_and_gather(tmp_path: Path, total: int) -> None:
    from oracle import attention_oracle as ao

    out_path = str(tmp_path / "gathered.npy")
    mp.spawn(_worker, args=(2, _free_port(), total, out_path), nprocs=2, join=True)
    gen = torch.Generator().manual_seed(0)
    qkv = torch.randn(total, 3, 2, 33, 64, generator=gen)
    ref = ao.attention(qkv[:, 0].numpy(), qkv[:, 1].numpy(), qkv[:, 2].numpy())
    np.testing.assert_allclose(np.load(out_path), ref, rtol=0, atol=1e-6)


def _leaver_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    """Two steps of independent shard work, a barrier after each. Rank 1 leaves between the steps (it returns without
    joining the second barrier and without destroying the group, as a process that is gone would); rank 0's second
    barrier must end with an error within the group's timeout instead of waiting for ever."""
    import time
    from datetime import timedelta

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=5))
    dist.barrier()  # step 1: everybody is here
    if rank == 1:
        os._exit(0)  # noqa: SLF001 - leaves between steps, nothing of it in flight
    t0 = time.monotonic()
    outcome = "completed"
    try:
        dist.barrier()  # step 2: rank 1 never comes
    except Exception as e:  # noqa: BLE001 - gloo reports the lost peer or the timeout as RuntimeError / DistBackendError
        outcome = f"error after {time.monotonic() - t0:.1f} s: {type(e).__name__}"
    Path(out_dir, f"rank{rank}.txt").write_text(outcome)
    os._exit(0)  # noqa: SLF001 - the group is broken: no orderly shutdown to wait for


def test_a_rank_that_leaves_between_steps_ends_the_others_barrier_with_an_error(tmp_path: Path) -> None:
    """The host-side failure form of the multi-GPU harness: no collective runs while a model runs, so a lost rank
    shows at the next barrier, which has a finite limit (bench.py gives its process group one too)."""
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_leaver_worker, args=(r, 2, port, str(tmp_path))) for port in [_free_port()] for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank is still waiting: the barrier has no limit"
    outcome = (tmp_path / "rank0.txt").read_text()
    assert outcome.startswith("error after"), outcome
    assert float(outcome.split()[2]) < 30.0
