"""Attention over operands that live in HOST memory: copies in, kernel and copies out overlapped on three streams.

The reference's kernels keep everything on the device and its callers upload one batch of images per call
(`src/fastforks/_core/model.py:142-148` serialises those calls). A caller that holds packed qkv tensors in pinned host
memory (a benchmark of the operator end to end, or a pipeline stage fed from another process) would otherwise pay
upload + kernel + download one after the other for every tensor. `HostAttention` keeps `depth` device staging
buffers and runs the upload of tensor i+1 and the download of tensor i-1 beside the kernel of tensor i; PCIe carries
both directions at once, so a sequence of calls costs about the larger of the two copy times.
"""

from __future__ import annotations

from typing import TYPE_CHECKING

import torch

from .attention import HEAD_DIM, attention

if TYPE_CHECKING:
    from collections.abc import Sequence

PACKED_DIMS = 5  # [B, N, 3, heads, 64]


class HostAttention:
    """`softmax(scale * q k^T) v` for packed `[B, N, 3, heads, 64]` qkv tensors in pinned host memory."""

    def __init__(self, device: torch.device | int | str | None = None, depth: int = 2) -> None:
        """`device`: the CUDA device to run on (default: current); `depth`: staging buffers in flight (>= 2 overlaps)."""
        if depth < 1:
            msg = f"HostAttention: depth {depth} must be at least 1"
            raise ValueError(msg)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if self.device.type != "cuda":
            msg = f"HostAttention: device {self.device} is not a CUDA device"
            raise ValueError(msg)
        self.depth = depth
        with torch.cuda.device(self.device):
            self._upload, self._compute, self._download = (torch.cuda.Stream() for _ in range(3))
        self._slots: list[dict] = []
        self._geometry: tuple | None = None

    @staticmethod
    def check(host_qkv: Sequence[torch.Tensor], host_out: Sequence[torch.Tensor]) -> None:
        """Check the host-side contract before anything is copied or launched.

        Raises:
            ValueError: Lists of different length, CUDA or unpinned tensors, a shape other than packed
                `[B, N, 3, heads, 64]` in / `[B, N, heads, 64]` out, non-contiguous memory, a dtype other than
                fp16 / bf16, or tensors of different geometry in one call.
        """
        if len(host_qkv) != len(host_out):
            msg = f"HostAttention: {len(host_qkv)} qkv tensors but {len(host_out)} outputs"
            raise ValueError(msg)
        for i, (x, o) in enumerate(zip(host_qkv, host_out)):
            if x.is_cuda or o.is_cuda:
                msg = f"HostAttention: tensor {i} is on {x.device} / {o.device}; operands must be in host memory"
                raise ValueError(msg)
            if x.dim() != PACKED_DIMS or x.shape[2] != 3 or x.shape[-1] != HEAD_DIM:  # noqa: PLR2004
                msg = f"HostAttention: qkv {i} has shape {tuple(x.shape)}, expected packed [B, N, 3, heads, {HEAD_DIM}]"
                raise ValueError(msg)
            if x.dtype not in (torch.float16, torch.bfloat16) or o.dtype != x.dtype:
                msg = f"HostAttention: tensor {i} is {x.dtype} / {o.dtype}; expected one of float16, bfloat16 for both"
                raise ValueError(msg)
            b, n, _, h, d = x.shape
            if tuple(o.shape) != (b, n, h, d):
                msg = f"HostAttention: output {i} has shape {tuple(o.shape)}, expected {(b, n, h, d)}"
                raise ValueError(msg)
            if not x.is_contiguous() or not o.is_contiguous():
                msg = f"HostAttention: tensor {i} is not contiguous"
                raise ValueError(msg)
            if x.shape != host_qkv[0].shape or x.dtype != host_qkv[0].dtype:
                msg = f"HostAttention: qkv {i} {tuple(x.shape)} {x.dtype} differs from qkv 0 in one call"
                raise ValueError(msg)
            if x.numel() == 0:
                msg = f"HostAttention: qkv {i} is empty"
                raise ValueError(msg)
            if torch.cuda.is_available() and not (x.is_pinned() and o.is_pinned()):
                msg = f"HostAttention: tensor {i} is not in pinned memory (asynchronous copies need it)"
                raise ValueError(msg)

    def _staging(self, like: torch.Tensor) -> list[dict]:
        geometry = (tuple(like.shape), like.dtype)
        if geometry != self._geometry:
            b, n, _, h, d = like.shape
            self._slots = [
                {
                    "qkv": torch.empty(like.shape, dtype=like.dtype, device=self.device),
                    "out": torch.empty((b, n, h, d), dtype=like.dtype, device=self.device),
                    "uploaded": torch.cuda.Event(),
                    "computed": torch.cuda.Event(),
                    "downloaded": torch.cuda.Event(),
                    "used": False,
                }
                for _ in range(self.depth)
            ]
            self._geometry = geometry
        return self._slots

    def __call__(self, host_qkv: Sequence[torch.Tensor], host_out: Sequence[torch.Tensor], scale: float | None = None) -> None:
        """Fill `host_out[i]` (`[B, N, heads, 64]`) with the attention of `host_qkv[i]`; returns when all are written.

        Raises:
            ValueError: See `check`.
            KernelUnavailableError / RuntimeError: As `attention`.
        """
        self.check(host_qkv, host_out)
        if not host_qkv:
            return
        slots = self._staging(host_qkv[0])
        caller = torch.cuda.current_stream(self.device)
        for s in (self._upload, self._compute, self._download):
            s.wait_stream(caller)  # host tensors written by work queued on the caller's stream are complete first
        for i, (x, o) in enumerate(zip(host_qkv, host_out)):
            slot = slots[i % self.depth]
            with torch.cuda.stream(self._upload):
                if slot["used"]:
                    self._upload.wait_event(slot["computed"])  # the kernel that read this staging buffer is done
                slot["qkv"].copy_(x, non_blocking=True)
                slot["uploaded"].record(self._upload)
            with torch.cuda.stream(self._compute):
                self._compute.wait_event(slot["uploaded"])
                if slot["used"]:
                    self._compute.wait_event(slot["downloaded"])  # the previous result has left this output buffer
                q, k, v = slot["qkv"].unbind(2)
                attention(q, k, v, scale=scale, layout="bnhd", out=slot["out"])
                slot["computed"].record(self._compute)
            with torch.cuda.stream(self._download):
                self._download.wait_event(slot["computed"])
                o.copy_(slot["out"], non_blocking=True)
                slot["downloaded"].record(self._download)
            slot["used"] = True
        self._download.synchronize()
        caller.wait_stream(self._download)
