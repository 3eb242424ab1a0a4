"""Typed errors of the B200 attention backend.

The class names and their meaning are the reference's (`src/fastforks/_core/errors.py:40-66`), so code written
against it catches the same things: the kernels backend either runs or raises, it never quietly does something else.
"""

from __future__ import annotations


class BackendUnavailableError(RuntimeError):
    """Raised when a backend was asked for by name (`mode="kernels"`) on a machine where it cannot run."""


class KernelUnavailableError(BackendUnavailableError):
    """Raised when the compiled kernel library is missing, stale or does not load.

    Attributes:
        library: Which library (`"b200attn"`).
        reason: What is wrong with it and, where there is one, the command that fixes it.
    """

    def __init__(self, library: str, reason: str) -> None:
        super().__init__(f"kernel library {library!r} is unavailable: {reason}")
        self.library = library
        self.reason = reason
