"""jaxdecomp_b200 -- domain decomposition, distributed FFTs and halo exchange
for NVIDIA B200, with PyTorch as the framework layer.

The public names mirror the reference library's ``__all__``
(``src/jaxdecomp/__init__.py:52-91``): ``pfft3d``/``pifft3d``, the six pencil
transposes, ``halo_exchange``, ``fftfreq3d``/``rfftfreq3d``, the spec helpers,
``config`` and the enumerated constants, plus ``init``/``finalize``,
``get_pencil_info``, ``get_autotuned_config`` and ``make_config``.  Arrays are
:class:`ShardedTensor` objects (one process per GPU holds one block); the
same functions accept plain tensors as the local block under an active mesh.

Two backends implement every op: ``'b200'`` (hand-written sm_100a kernels that
fuse each collective with its compute; default for CUDA tensors) and
``'torch'`` (``torch.fft`` + NCCL/gloo collectives; default for CPU tensors and
the oracle/baseline).  The strings ``'jax'`` and ``'cudecomp'`` are accepted as
aliases so that code written against the reference runs unchanged.
"""
from __future__ import annotations

from . import fft, halo, transpose  # noqa: F401  (module paths of the reference: jaxdecomp.fft.pfft3d, ...)
from .ops.fft import fftfreq3d, pfft3d, pifft3d, pirfft3d, prfft3d, rfftfreq3d
from .ops.halo import halo_accumulate, halo_exchange, halo_exchange_, halo_reduce, pad_halo, unpad_halo
from .ops.peer import empty_peer_visible, empty_sharded, free_peer_visible
from .ops.transpose import (
    transpose_shard,
    transposeXtoY,
    transposeXtoZ,
    transposeYtoX,
    transposeYtoZ,
    transposeZtoX,
    transposeZtoY,
)
from .parallel.mesh import Mesh, current_mesh, init_distributed, make_mesh, set_mesh, single_rank_mesh
from .parallel.sharding import (
    NamedSharding,
    P,
    PartitionSpec,
    PencilInfo,
    ShardedTensor,
    get_fft_output_sharding,
    get_output_specs,
    shard,
    validate_spec_matches_mesh,
)
from .utils.api import (
    GridConfig,
    autotune,
    finalize,
    check_peers,
    get_autotuned_config,
    get_fft_workspace_size,
    get_halo_workspace_size,
    get_pencil_info,
    get_transpose_workspace_size,
    init,
    make_config,
    reserve_workspace,
)
from .utils.checkpoint import load_sharded, save_sharded
from .utils.config import (
    HALO_COMM_MPI,
    HALO_COMM_MPI_BLOCKING,
    HALO_COMM_NCCL,
    HALO_COMM_NVSHMEM,
    HALO_COMM_NVSHMEM_BLOCKING,
    HALO_COMM_P2P,
    NO_DECOMP,
    PENCILS,
    SLAB_XY,
    SLAB_YZ,
    TRANSPOSE_COMM_MPI_A2A,
    TRANSPOSE_COMM_MPI_P2P,
    TRANSPOSE_COMM_MPI_P2P_PL,
    TRANSPOSE_COMM_NCCL,
    TRANSPOSE_COMM_NCCL_PL,
    TRANSPOSE_COMM_NVSHMEM,
    TRANSPOSE_COMM_NVSHMEM_PL,
    TRANSPOSE_COMM_P2P,
    TRANSPOSE_COMM_P2P_PL,
    TRANSPOSE_XY,
    TRANSPOSE_XZ,
    TRANSPOSE_YX,
    TRANSPOSE_YZ,
    TRANSPOSE_ZX,
    TRANSPOSE_ZY,
    Decomposition,
    HaloCommBackend,
    TransposeCommBackend,
    TransposeType,
    config,
)

__version__ = "0.1.0"

__all__ = [
    "config", "init", "finalize", "get_pencil_info", "get_autotuned_config", "make_config", "autotune",
    "get_fft_workspace_size", "get_transpose_workspace_size", "get_halo_workspace_size", "reserve_workspace", "check_peers",
    "halo_exchange", "halo_exchange_", "halo_accumulate", "halo_reduce", "pad_halo", "unpad_halo",
    "pfft3d", "pifft3d", "prfft3d", "pirfft3d", "fftfreq3d", "rfftfreq3d", "fft", "halo", "transpose",
    "transposeXtoY", "transposeYtoX", "transposeYtoZ", "transposeZtoY", "transposeXtoZ", "transposeZtoX",
    "transpose_shard",
    "TRANSPOSE_XY", "TRANSPOSE_YX", "TRANSPOSE_YZ", "TRANSPOSE_ZY", "TRANSPOSE_XZ", "TRANSPOSE_ZX",
    "SLAB_XY", "SLAB_YZ", "PENCILS", "NO_DECOMP",
    "get_fft_output_sharding", "get_output_specs", "validate_spec_matches_mesh",
    "HALO_COMM_MPI", "HALO_COMM_MPI_BLOCKING", "HALO_COMM_NCCL", "HALO_COMM_NVSHMEM", "HALO_COMM_NVSHMEM_BLOCKING",
    "HALO_COMM_P2P",
    "TRANSPOSE_COMM_MPI_A2A", "TRANSPOSE_COMM_MPI_P2P", "TRANSPOSE_COMM_MPI_P2P_PL", "TRANSPOSE_COMM_NCCL",
    "TRANSPOSE_COMM_NCCL_PL", "TRANSPOSE_COMM_NVSHMEM", "TRANSPOSE_COMM_NVSHMEM_PL", "TRANSPOSE_COMM_P2P", "TRANSPOSE_COMM_P2P_PL",
    "HaloCommBackend", "TransposeCommBackend", "TransposeType", "Decomposition",
    "Mesh", "make_mesh", "set_mesh", "current_mesh", "single_rank_mesh", "init_distributed",
    "ShardedTensor", "shard", "PartitionSpec", "P", "NamedSharding", "PencilInfo", "GridConfig",
    "save_sharded", "load_sharded", "empty_sharded", "empty_peer_visible", "free_peer_visible",
]
