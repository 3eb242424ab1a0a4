"""Typed errors of the B200 attention backend.

Same names and meaning as the reference's `src/fastforks/_core/errors.py:40-60`: asking for the kernels
backend where it cannot run raises, it never falls back silently.
"""

from __future__ import annotations


class BackendUnavailableError(RuntimeError):
    """The requested backend (`mode="kernels"`) cannot run here. There is no silent fallback."""


class KernelUnavailableError(BackendUnavailableError):
    """The kernel library cannot be loaded on this machine.

    Attributes:
        library: Kernel library name.
        reason: Why it cannot be loaded (no binary, no GPU, wrong architecture, ...).
    """

    def __init__(self, library: str, reason: str) -> None:
        super().__init__(f"kernel library {library!r} is unavailable: {reason}")
        self.library = library
        self.reason = reason
