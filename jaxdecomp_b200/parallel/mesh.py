"""Device mesh: one process per GPU arranged on an N-D grid.

The last two mesh axes are the decomposition axes ``(a0, a1)`` with sizes
``pdims = (P0, P1)``; any leading axes are independent batch groups (the
reference's "nested parallelism": a leading mesh axis plus ``vmap``,
``src/jaxdecomp/_src/pencil_utils.py:47-99``).  Ranks map to coordinates in
row-major order, which is also the default device order of ``jax.make_mesh``.

A mesh owns the ``torch.distributed`` sub-groups along each decomposition axis
(the row / column communicators of a pencil decomposition).  With a single rank
no process group is needed at all.
"""
from __future__ import annotations

import itertools
import threading
from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..utils.config import NO_DECOMP, PENCILS, SLAB_XY, SLAB_YZ, Decomposition

_tls = threading.local()


def _dist_ready() -> bool:
    return dist.is_available() and dist.is_initialized()


def pencil_type_from_pdims(pdims: Sequence[int]) -> Decomposition:
    """Name the decomposition after the mesh shape (reference:
    ``pencil_utils.py:81-92``): (1,1) none, P0==1 slab-YZ, P1==1 slab-XY, else pencils."""
    if pdims is None:
        return NO_DECOMP
    pdims = tuple(int(p) for p in pdims)
    if len(pdims) != 2:
        raise ValueError("Only one or two-dimensional meshes are supported.")
    if pdims == (1, 1):
        return NO_DECOMP
    if pdims[0] == 1:
        return SLAB_YZ
    if pdims[1] == 1:
        return SLAB_XY
    return PENCILS


class Mesh:
    """An N-D process mesh.

    Parameters
    ----------
    shape : sizes of the mesh axes; ``prod(shape)`` must equal the world size.
    axis_names : one name per mesh axis.
    rank, world_size : override for unit tests that only need the arithmetic
        (no process group is created when ``create_groups=False``).
    """

    def __init__(
        self,
        shape: Sequence[int],
        axis_names: Sequence[str],
        *,
        rank: Optional[int] = None,
        world_size: Optional[int] = None,
        create_groups: bool = True,
    ):
        shape = tuple(int(s) for s in shape)
        axis_names = tuple(axis_names)
        if len(shape) != len(axis_names):
            raise ValueError(f"mesh shape {shape} and axis names {axis_names} differ in length")
        if len(set(axis_names)) != len(axis_names):
            raise ValueError(f"duplicate mesh axis names {axis_names}")
        if len(shape) == 0:
            raise ValueError("empty mesh")
        if len(shape) == 1:  # a 1-D mesh shards array axis 1 (reference: get_pencil_type)
            shape = (1,) + shape
            axis_names = (None,) + axis_names
        n = 1
        for s in shape:
            if s < 1:
                raise ValueError(f"invalid mesh shape {shape}")
            n *= s
        if world_size is None:
            world_size = dist.get_world_size() if _dist_ready() else 1
        if rank is None:
            rank = dist.get_rank() if _dist_ready() else 0
        if n != world_size:
            raise ValueError(f"mesh shape {shape} needs {n} ranks but the world has {world_size}")
        self.shape = shape
        self.axis_names = axis_names
        self.rank = int(rank)
        self.world_size = int(world_size)
        self.coords = self.coords_of(self.rank)
        self._groups = {}
        if create_groups and self.world_size > 1:
            if not _dist_ready():
                raise RuntimeError("torch.distributed must be initialised before creating a multi-rank Mesh")
            self._build_groups()

    # ---- arithmetic ---------------------------------------------------------------------
    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def pdims(self) -> Tuple[int, int]:
        return (self.shape[-2], self.shape[-1])

    @property
    def decomp_axis_names(self) -> Tuple[Optional[str], Optional[str]]:
        return (self.axis_names[-2], self.axis_names[-1])

    @property
    def batch_axis_names(self) -> tuple:
        return self.axis_names[:-2]

    @property
    def pencil_type(self) -> Decomposition:
        return pencil_type_from_pdims(self.pdims)

    @property
    def empty(self) -> bool:
        return False

    def axis_size(self, axis) -> int:
        return self.shape[self._axis_index(axis)]

    def _axis_index(self, axis) -> int:
        if isinstance(axis, int):
            # 0 / 1 address the two decomposition axes
            return self.ndim - 2 + axis
        return self.axis_names.index(axis)

    def coords_of(self, rank: int) -> tuple:
        out = []
        for s in reversed(self.shape):
            out.append(rank % s)
            rank //= s
        return tuple(reversed(out))

    def rank_of(self, coords: Sequence[int]) -> int:
        r = 0
        for c, s in zip(coords, self.shape):
            r = r * s + (c % s)
        return r

    def axis_coord(self, axis) -> int:
        return self.coords[self._axis_index(axis)]

    def axis_ranks(self, axis, rank: Optional[int] = None) -> list:
        """Global ranks of the sub-group along ``axis`` that contains ``rank``
        (default: this rank), ordered by their coordinate on that axis."""
        ai = self._axis_index(axis)
        coords = list(self.coords if rank is None else self.coords_of(rank))
        out = []
        for c in range(self.shape[ai]):
            coords[ai] = c
            out.append(self.rank_of(coords))
        return out

    def neighbor(self, d0: int, d1: int, periodic=(True, True)) -> Optional[int]:
        """Rank at offset (d0, d1) on the two decomposition axes, or None when
        the offset leaves a non-periodic mesh."""
        coords = list(self.coords)
        for k, d, per in ((self.ndim - 2, d0, periodic[0]), (self.ndim - 1, d1, periodic[1])):
            c = coords[k] + d
            if c < 0 or c >= self.shape[k]:
                if not per:
                    return None
                c %= self.shape[k]
            coords[k] = c
        return self.rank_of(coords)

    def submesh_ranks(self) -> list:
        """Ranks of this rank's 2-D decomposition mesh (same batch coordinates), row-major."""
        lead = self.coords[:-2]
        return [self.rank_of(lead + (i, j)) for i in range(self.shape[-2]) for j in range(self.shape[-1])]

    # ---- process groups -----------------------------------------------------------------
    def _build_groups(self):
        # every rank must create every group, in the same order
        for ai in range(self.ndim):
            if self.shape[ai] == 1:
                continue
            others = [range(s) for k, s in enumerate(self.shape) if k != ai]
            for combo in itertools.product(*others):
                coords = list(combo)
                coords.insert(ai, 0)
                ranks = []
                for c in range(self.shape[ai]):
                    coords[ai] = c
                    ranks.append(self.rank_of(coords))
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self._groups[ai] = g
        if self.ndim > 2:
            lead_shapes = [range(s) for s in self.shape[:-2]]
            for lead in itertools.product(*lead_shapes):
                ranks = [
                    self.rank_of(tuple(lead) + (i, j)) for i in range(self.shape[-2]) for j in range(self.shape[-1])
                ]
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self._groups["submesh"] = g
        else:
            self._groups["submesh"] = dist.group.WORLD

    def axis_group(self, axis):
        """Process group along a mesh axis (None for a size-1 axis)."""
        return self._groups.get(self._axis_index(axis))

    def submesh_group(self):
        return self._groups.get("submesh")

    def barrier(self):
        if self.world_size > 1:
            dist.barrier()

    # ---- context manager: default mesh for ops called with plain tensors -------------------
    def __enter__(self):
        stack = getattr(_tls, "stack", None)
        if stack is None:
            stack = _tls.stack = []
        stack.append(self)
        return self

    def __exit__(self, *exc):
        _tls.stack.pop()
        return False

    def __repr__(self):
        return f"Mesh(shape={self.shape}, axis_names={self.axis_names}, rank={self.rank})"

    def __eq__(self, other):
        return (
            isinstance(other, Mesh)
            and self.shape == other.shape
            and self.axis_names == other.axis_names
            and self.world_size == other.world_size
        )

    def __hash__(self):
        return hash((self.shape, self.axis_names, self.world_size))


_default_mesh: Optional[Mesh] = None


def set_mesh(mesh: Optional[Mesh]) -> None:
    """Install a process-wide default mesh used when ops receive plain tensors."""
    global _default_mesh
    _default_mesh = mesh


def current_mesh() -> Optional[Mesh]:
    stack = getattr(_tls, "stack", None)
    if stack:
        return stack[-1]
    return _default_mesh


def make_mesh(pdims: Sequence[int], axis_names: Sequence[str] = ("z", "y")) -> Mesh:
    """Create a mesh with the given shape; the analogue of ``jax.make_mesh``."""
    return Mesh(pdims, axis_names)


def single_rank_mesh(axis_names=("z", "y")) -> Mesh:
    return Mesh((1, 1), axis_names, rank=0, world_size=1, create_groups=False)


def init_distributed(backend: Optional[str] = None, device: Optional[torch.device] = None) -> torch.device:
    """Initialise ``torch.distributed`` from the torchrun environment (RANK,
    WORLD_SIZE, LOCAL_RANK, MASTER_ADDR, MASTER_PORT) and bind this process to
    its GPU.  Plays the role of ``jax.distributed.initialize()`` in the
    reference's benchmark (``benchmarks/bench.py:13``)."""
    import os

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if device is None:
        if torch.cuda.is_available():
            device = torch.device("cuda", local_rank % torch.cuda.device_count())
        else:
            device = torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
        # keep the rank (and the pinned buffers it allocates from now on) on the GPU's NUMA node
        from ..utils.affinity import bind_to_device_cpus

        bind_to_device_cpus(device.index if device.index is not None else torch.cuda.current_device())
    if world > 1 and not _dist_ready():
        if backend is None:
            backend = "nccl" if device.type == "cuda" else "gloo"
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = device
        dist.init_process_group(backend=backend, **kwargs)
    return device
