"""A small cache of CUDA graphs for launch-bound forwards: one graph per input geometry.

One image of ViT-B/16 is some 150 kernel launches of a few microseconds each; replayed from a graph the forward is
bound by the kernels instead of by the launches. The conventions follow the reference's graph cache
(`src/fastforks/shared/cuda_graphs.py:1-17`): a geometry is captured only after `capture_after` eager calls (so a
one-off size never captures), a full cache evicts the graph unused for longest, a failed capture marks the geometry
eager for good, calls are serialised per device (graphs share static buffers and the attention workspace of the capture
stream, so two replays must never overlap), and every warm-up and capture runs on one stream per device.

The attention kernels are capturable as they are: they allocate nothing, and the scratch memory of long sequences is
reserved for the capture stream before the capture begins (`reserve_workspace`).
"""

from __future__ import annotations

import functools
import threading
from collections import OrderedDict
from typing import TYPE_CHECKING, Any

import torch

from .attention import reserve_workspace

if TYPE_CHECKING:
    from collections.abc import Callable, Hashable

CAPTURE_LOCK = threading.RLock()  # serialises warm-ups, captures and replays (static buffers are shared)
_LAST_REPLAY: dict[int, torch.cuda.Event] = {}  # per device: the end of the last replay, which the next one waits for


@functools.cache
def capture_stream(index: int) -> torch.cuda.Stream:
    """The stream of every graph warm-up and capture on device `index` (hold `CAPTURE_LOCK` while using it)."""
    return torch.cuda.Stream(index)


def geometry_key(inputs: tuple[torch.Tensor, ...]) -> Hashable:
    """What a graph is valid for: dtype, device, shape and strides of every input."""
    return tuple((t.dtype, t.device, tuple(t.shape), tuple(t.stride())) for t in inputs)


def _map(out: Any, fn: Callable[[torch.Tensor], torch.Tensor]) -> Any:  # noqa: ANN401 - a tensor or a list / tuple / dict of them
    if isinstance(out, torch.Tensor):
        return fn(out)
    if isinstance(out, dict):
        return {k: _map(v, fn) for k, v in out.items()}
    if isinstance(out, (list, tuple)):
        return type(out)(_map(v, fn) for v in out)
    return out


class _Graph:
    def __init__(self, graph: torch.cuda.CUDAGraph, static_in: tuple[torch.Tensor, ...], static_out: Any) -> None:  # noqa: ANN401
        self.graph, self.static_in, self.static_out = graph, static_in, static_out


class GraphCache:
    """`cache(*tensors)` = `forward(*tensors)`, replayed from a CUDA graph once the geometry has been seen often enough.

    Args:
        forward: A function of CUDA tensors that returns a tensor or a list / tuple / dict of tensors, launches on the
            current stream, never synchronises and keeps no tensor it returns (its outputs are overwritten by the
            next replay; callers get copies).
        capture_after: Eager calls of a geometry before it is captured (at least 1).
        max_graphs: Graphs held; the one unused for longest makes room.
    """

    def __init__(self, forward: Callable[..., Any], *, capture_after: int = 1, max_graphs: int = 8) -> None:
        if capture_after < 1 or max_graphs < 1:
            msg = f"GraphCache: capture_after {capture_after} and max_graphs {max_graphs} must be at least 1"
            raise ValueError(msg)
        self.forward, self.capture_after, self.max_graphs = forward, capture_after, max_graphs
        self._graphs: OrderedDict[Hashable, _Graph] = OrderedDict()
        self._seen: dict[Hashable, int] = {}
        self._failed: set[Hashable] = set()
        self.stats = {"eager": 0, "captured": 0, "replayed": 0, "failed": 0, "evicted": 0}

    def __call__(self, *inputs: torch.Tensor) -> Any:  # noqa: ANN401
        if not inputs or not all(isinstance(t, torch.Tensor) and t.is_cuda for t in inputs) or torch.cuda.is_current_stream_capturing():
            self.stats["eager"] += 1
            return self.forward(*inputs)
        key = geometry_key(inputs)
        with CAPTURE_LOCK:
            held = self._graphs.get(key)
            if held is None and key not in self._failed:
                self._seen[key] = self._seen.get(key, 0) + 1
                if self._seen[key] > self.capture_after:
                    held = self._capture(key, inputs)
            if held is None:
                self.stats["eager"] += 1
                return self.forward(*inputs)
            self._graphs.move_to_end(key)
            index = inputs[0].device.index
            stream = torch.cuda.current_stream(index)
            last = _LAST_REPLAY.get(index)
            if last is not None:
                stream.wait_event(last)  # the replay before (of any cache) has finished with the shared buffers
            for dst, src in zip(held.static_in, inputs, strict=True):
                dst.copy_(src, non_blocking=True)
            held.graph.replay()
            out = _map(held.static_out, torch.clone)
            done = torch.cuda.Event()
            done.record(stream)
            _LAST_REPLAY[index] = done
            self.stats["replayed"] += 1
            return out

    def _capture(self, key: Hashable, inputs: tuple[torch.Tensor, ...]) -> _Graph | None:
        index = inputs[0].device.index
        side = capture_stream(index)
        side.wait_stream(torch.cuda.current_stream(index))
        static_in: tuple[torch.Tensor, ...] = ()
        try:
            with torch.cuda.stream(side):
                static_in = tuple(torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=t.device).copy_(t) for t in inputs)
                reserve_workspace(index)  # for this stream, before the capture: a capture allocates nothing
                self.forward(*static_in)  # warm-up: lazy initialisation happens outside the capture
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    static_out = self.forward(*static_in)
        except RuntimeError:
            self._failed.add(key)
            self.stats["failed"] += 1
            torch.cuda.current_stream(index).wait_stream(side)
            return None
        torch.cuda.current_stream(index).wait_stream(side)
        while len(self._graphs) >= self.max_graphs:
            self._graphs.popitem(last=False)
            self.stats["evicted"] += 1
        held = self._graphs[key] = _Graph(graph, static_in, static_out)
        self.stats["captured"] += 1
        return held

    def release(self) -> None:
        """Drop every graph and its static buffers; geometries are counted anew."""
        with CAPTURE_LOCK:
            self._graphs.clear()
            self._seen.clear()
