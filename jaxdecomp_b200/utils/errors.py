"""Exception types and diagnostic messages.

The reference aborts the process on CUDA/MPI errors and throws an untyped
exception for cuFFT/cuDecomp ones (``src/csrc/include/checks.h:29-72``); its only
Python-level diagnostics are two messages raised when a Jacobian is requested on
an unsharded operand (``src/jaxdecomp/_src/error.py:1-18``).  Here every failure,
including a device-side wait that ran out of time, surfaces as a Python
exception and never ends the process.
"""
from __future__ import annotations


class DecompError(RuntimeError):
    """Base class of every error raised by this package."""


class ShardingError(DecompError, ValueError):
    """A spec, mesh or global shape is not usable for the requested operation."""


class NativeExtensionError(DecompError):
    """The CUDA extension is missing or failed to load on a machine with a GPU."""


class PeerTimeoutError(DecompError):
    """A bounded device-side wait on a peer's signal expired.

    Attributes mirror the status block written by the kernel: which peer was
    awaited, the epoch that was expected and the epoch that was last seen.
    """

    def __init__(self, message: str, peer: int = -1, expected: int = -1, seen: int = -1):
        super().__init__(message)
        self.peer = peer
        self.expected = expected
        self.seen = seen


class StaleEpochError(DecompError):
    """A peer's signal was more than one barrier ahead of the barrier this rank was waiting in: the
    ranks no longer count the same barriers (a replayed or skipped barrier, a corrupted flag)."""


class PeerAbortedError(DecompError):
    """Another rank's bounded wait failed and it marked the whole group as aborted; the exchange
    buffers hold incomplete data, every later kernel of this rank returned without computing, and the
    arena must be re-created (``finalize()`` then the next call) before the mesh is used again."""

    def __init__(self, message: str, peer: int = -1):
        super().__init__(message)
        self.peer = peer


class KernelStatusError(DecompError):
    """A kernel reported a non-zero status word (bounds check, bad argument)."""


def error_unsharded_operand(op: str) -> ShardingError:
    """Message used when an op that needs a sharded operand receives a plain,
    fully replicated tensor while a multi-rank mesh is active (the analogue of
    the reference's jacfwd/jacrev diagnostics)."""
    return ShardingError(
        f"{op}: the operand is a plain tensor without sharding information, no mesh is active, and this "
        "process is one of several ranks. Wrap the local block in a ShardedTensor, or call the op under "
        "`with mesh:` with the local block in the layout the op expects; use `with jd.single_rank_mesh():` "
        "to transform a replicated array on every rank on purpose."
    )
