"""Library-wide configuration object and the enumerated constants of the API.

Covers the reference's ``JAXDecompConfig`` (``src/jaxdecomp/__init__.py:94-110``)
and the constants it re-exports from its native module
(``src/csrc/include/jaxdecomp.h:10-49``, ``src/csrc/jaxdecomp.cc:574-606``).
Unlike the reference, the configuration is read at call time: there is no
trace cache to clear after changing it.
"""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass, fields


class HaloCommBackend(enum.IntEnum):
    """Transport used for halo exchange.  Values match the reference's enum."""

    HALO_COMM_MPI = 1
    HALO_COMM_MPI_BLOCKING = 2
    HALO_COMM_NCCL = 3
    HALO_COMM_NVSHMEM = 4
    HALO_COMM_NVSHMEM_BLOCKING = 5
    # transports native to this package
    HALO_COMM_P2P = 16


class TransposeCommBackend(enum.IntEnum):
    """Transport used for the pencil transposes.  Values match the reference."""

    TRANSPOSE_COMM_MPI_P2P = 1
    TRANSPOSE_COMM_MPI_P2P_PL = 2
    TRANSPOSE_COMM_MPI_A2A = 3
    TRANSPOSE_COMM_NCCL = 4
    TRANSPOSE_COMM_NCCL_PL = 5
    TRANSPOSE_COMM_NVSHMEM = 6
    TRANSPOSE_COMM_NVSHMEM_PL = 7
    # transports native to this package: fused peer-store kernels, each exchange pass followed by its
    # barrier (P2P) or cut into chunks that overlap with the local pass that consumes them (P2P_PL)
    TRANSPOSE_COMM_P2P = 16
    TRANSPOSE_COMM_P2P_PL = 17


class TransposeType(enum.IntEnum):
    TRANSPOSE_XY = 0
    TRANSPOSE_YZ = 1
    TRANSPOSE_ZY = 2
    TRANSPOSE_YX = 3
    TRANSPOSE_XZ = 4
    TRANSPOSE_ZX = 5


class Decomposition(enum.IntEnum):
    SLAB_XY = 0
    SLAB_YZ = 1
    PENCILS = 2
    NO_DECOMP = 3


HALO_COMM_MPI = HaloCommBackend.HALO_COMM_MPI
HALO_COMM_MPI_BLOCKING = HaloCommBackend.HALO_COMM_MPI_BLOCKING
HALO_COMM_NCCL = HaloCommBackend.HALO_COMM_NCCL
HALO_COMM_NVSHMEM = HaloCommBackend.HALO_COMM_NVSHMEM
HALO_COMM_NVSHMEM_BLOCKING = HaloCommBackend.HALO_COMM_NVSHMEM_BLOCKING
HALO_COMM_P2P = HaloCommBackend.HALO_COMM_P2P
TRANSPOSE_COMM_MPI_P2P = TransposeCommBackend.TRANSPOSE_COMM_MPI_P2P
TRANSPOSE_COMM_MPI_P2P_PL = TransposeCommBackend.TRANSPOSE_COMM_MPI_P2P_PL
TRANSPOSE_COMM_MPI_A2A = TransposeCommBackend.TRANSPOSE_COMM_MPI_A2A
TRANSPOSE_COMM_NCCL = TransposeCommBackend.TRANSPOSE_COMM_NCCL
TRANSPOSE_COMM_NCCL_PL = TransposeCommBackend.TRANSPOSE_COMM_NCCL_PL
TRANSPOSE_COMM_NVSHMEM = TransposeCommBackend.TRANSPOSE_COMM_NVSHMEM
TRANSPOSE_COMM_NVSHMEM_PL = TransposeCommBackend.TRANSPOSE_COMM_NVSHMEM_PL
TRANSPOSE_COMM_P2P = TransposeCommBackend.TRANSPOSE_COMM_P2P
TRANSPOSE_COMM_P2P_PL = TransposeCommBackend.TRANSPOSE_COMM_P2P_PL
TRANSPOSE_XY = TransposeType.TRANSPOSE_XY
TRANSPOSE_YZ = TransposeType.TRANSPOSE_YZ
TRANSPOSE_ZY = TransposeType.TRANSPOSE_ZY
TRANSPOSE_YX = TransposeType.TRANSPOSE_YX
TRANSPOSE_XZ = TransposeType.TRANSPOSE_XZ
TRANSPOSE_ZX = TransposeType.TRANSPOSE_ZX
SLAB_XY = Decomposition.SLAB_XY
SLAB_YZ = Decomposition.SLAB_YZ
PENCILS = Decomposition.PENCILS
NO_DECOMP = Decomposition.NO_DECOMP

_BACKEND_ALIASES = {
    "auto": "auto",
    "b200": "b200",
    "native": "b200",
    "cudecomp": "b200",  # drop-in for code written against the reference's native backend
    "torch": "torch",
    "jax": "torch",  # drop-in for the reference's default backend name
    "nccl": "torch",
}


def canonical_backend(name: str) -> str:
    """Map a user-facing backend string (case-insensitive) to 'auto', 'b200' or 'torch'."""
    key = str(name).lower()
    if key not in _BACKEND_ALIASES:
        raise ValueError(f"Invalid backend {name!r}; expected one of {sorted(_BACKEND_ALIASES)}")
    return _BACKEND_ALIASES[key]


@dataclass
class DecompConfig:
    """Mutable configuration state.

    ``halo_comm_backend`` / ``transpose_comm_backend`` keep the reference's
    field names.  With the per-call ``backend`` argument at ``'auto'``, the
    NCCL/MPI/NVSHMEM values select the all_to_all / send-recv baseline backend
    and the P2P values the fused peer-store kernels.  As in the reference
    (``src/csrc/include/jaxdecomp.h:13-18``) the ``*_PL`` transposes are the
    pipelined ones: on the native backend every exchange pass that is followed
    by a local pass is cut into ``pipeline_chunks`` chunks, and the local pass
    works on chunk k while chunk k+1 crosses NVLink.  ``pipeline_ctas`` limits
    the thread blocks of an exchange chunk (0: no limit) so that the local pass
    finds free SMs; the default, -1, picks the limit from the number of peers
    of the exchange (96 of the 148 SMs for two peers, 112 for more: the best
    settings measured on 2, 4 and 8 GPUs).
    """

    halo_comm_backend: HaloCommBackend = HALO_COMM_P2P
    transpose_comm_backend: TransposeCommBackend = TRANSPOSE_COMM_P2P_PL
    transpose_axis_contiguous: bool = True
    backend: str = "auto"
    wait_timeout_ms: int = int(os.environ.get("JD_B200_WAIT_TIMEOUT_MS", "10000"))
    reference_compat_halo_grad: bool = False
    pipeline_chunks: int = int(os.environ.get("JD_B200_PIPE_CHUNKS", "4"))
    pipeline_ctas: int = int(os.environ.get("JD_B200_PIPE_CTAS", "-1"))

    def update(self, key, value):
        names = {f.name for f in fields(self)}
        if key not in names:
            raise ValueError(f"key {key} is not a valid configuration key")
        if key == "backend":
            value = canonical_backend(value)
        elif key == "transpose_comm_backend":
            value = TransposeCommBackend(int(value))
        elif key == "halo_comm_backend":
            value = HaloCommBackend(int(value))
        elif key in ("pipeline_chunks", "pipeline_ctas", "wait_timeout_ms"):
            value = int(value)
            if value < (-1 if key == "pipeline_ctas" else 0):
                raise ValueError(f"{key} must not be negative" + (" (-1: automatic)" if key == "pipeline_ctas" else ""))
        setattr(self, key, value)

    @property
    def pipelined(self) -> bool:
        """True when the configured transpose transport is one of the pipelined (``*_PL``) ones."""
        return TransposeCommBackend(int(self.transpose_comm_backend)).name.endswith("_PL")

    def snapshot(self) -> tuple:
        """Hashable view of every field; the native backend puts it into its plan-cache keys, so a plan
        built under one configuration is never reused under another."""
        return tuple(getattr(self, f.name) for f in fields(self))


config = DecompConfig()
