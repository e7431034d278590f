"""Backend selection shared by all ops.

``backend='auto'`` picks the native sm_100a kernels for CUDA tensors and the
library baseline for CPU tensors.  A CUDA tensor never falls back silently:
if the native extension cannot be loaded the op raises, so that a GPU run
cannot pass on library code by accident.
"""
from __future__ import annotations

import torch

from ..utils.config import (
    HALO_COMM_P2P,
    TRANSPOSE_COMM_P2P,
    TRANSPOSE_COMM_P2P_PL,
    canonical_backend,
    config,
)
from ..utils.errors import NativeExtensionError


def resolve_backend(backend: str, x: torch.Tensor, family: str = "transpose") -> str:
    b = canonical_backend(backend)
    if b == "auto":
        b = config.backend
    if b == "auto":
        if x.is_cuda:
            comm = config.halo_comm_backend if family == "halo" else config.transpose_comm_backend
            native = (HALO_COMM_P2P,) if family == "halo" else (TRANSPOSE_COMM_P2P, TRANSPOSE_COMM_P2P_PL)
            b = "b200" if comm in native else "torch"
        else:
            b = "torch"
    if b == "b200":
        if not x.is_cuda:
            raise NativeExtensionError("backend 'b200' needs CUDA tensors; use backend='torch' for CPU ranks")
        from .. import native

        native.require()
    return b
