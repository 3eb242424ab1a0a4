"""Image-wise sharding of a batch over one-process-per-GPU replicas.

The reference runs multi-GPU as independent processes, one CUDA device each, with images split between them and no
communication while a model runs (`docs/usage.md:658-662`, `src/fastforks/_core/model.py:1006-1015`). These helpers
give every rank its contiguous image range and, after the work is done, collect the per-rank outputs on rank 0.
The gather is the only collective and is never inside a timed or hot region.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def image_range(total: int, world_size: int, rank: int) -> range:
    """Contiguous range of image indices owned by `rank`: sizes differ by at most one, earlier ranks get the extra.

    Raises:
        ValueError: Negative total, non-positive world size or a rank outside it.
    """
    if total < 0 or world_size < 1 or not 0 <= rank < world_size:
        msg = f"image_range(total={total}, world_size={world_size}, rank={rank}): invalid arguments"
        raise ValueError(msg)
    base, extra = divmod(total, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def gather_to_rank0(local: torch.Tensor, total: int, group: dist.ProcessGroup | None = None) -> torch.Tensor | None:
    """Collect per-rank outputs `[n_local, ...]` (ranges of `image_range`) into `[total, ...]` on rank 0.

    Every rank must call it; ranks other than 0 get None. Shards may differ in size by one image, so shards are
    padded to the largest before the collective and trimmed afterwards.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    sizes = [len(image_range(total, world, r)) for r in range(world)]
    if local.shape[0] != sizes[rank]:
        msg = f"rank {rank} holds {local.shape[0]} images, its range has {sizes[rank]}"
        raise ValueError(msg)
    biggest = max(sizes)
    padded = local
    if local.shape[0] < biggest:
        pad = local.new_zeros((biggest - local.shape[0], *local.shape[1:]))
        padded = torch.cat([local, pad])
    padded = padded.contiguous()
    bucket = [torch.empty_like(padded) for _ in range(world)] if rank == 0 else None
    dist.gather(padded, bucket, dst=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    if rank != 0:
        return None
    return torch.cat([t[:s] for t, s in zip(bucket, sizes)])
