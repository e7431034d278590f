"""Peer-visible tensors: blocks that every GPU of a mesh can address directly.

An ordinary ``torch`` tensor lives in memory that only its own GPU can reach, so an exchange has to go
through the library's peer-visible workspace: the sender stores into a staging slab there and the
receiver copies the slab into its block.  A block allocated here is itself mapped on every rank of the
mesh (``cudaMalloc`` + CUDA IPC, like the workspace), so kernels can store straight into the
neighbour's copy at the final address: ``halo_exchange_`` on such a block is one push kernel between
two barriers, with no staging and no unpack pass -- the in-place update that the reference's native
backend gets from cuDecomp (``src/jaxdecomp/_src/cudecomp/halo.py:146-151``,
``src/csrc/halo.cu:45-73``).

Allocation and release are collective over the ranks of the mesh's decomposition group, and every rank
must allocate the same shape (the blocks are addressed by the same offsets everywhere).  The memory is
returned to the driver by :func:`free_peer_visible` (collective) or at :func:`finalize`; it is not
managed by PyTorch's caching allocator.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import native as _native
from ..parallel.mesh import Mesh
from ..parallel.sharding import ShardedTensor

_TYPESTR = {torch.float32: "<f4", torch.float64: "<f8", torch.complex64: "<c8", torch.complex128: "<c16",
            torch.float16: "<f2", torch.int32: "<i4", torch.int64: "<i8", torch.uint8: "|u1"}


class _DeviceBuffer:
    """Exposes raw device memory to ``torch.as_tensor`` through the CUDA array interface; the tensor made
    from it keeps this object, and with it the allocation, alive."""

    def __init__(self, ptr: int, shape: Sequence[int], dtype: torch.dtype, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": tuple(int(s) for s in shape), "typestr": _TYPESTR[dtype],
                                         "data": (int(ptr), False), "version": 2, "strides": None}


class PeerAllocation:
    """One collective allocation: the native block, the tensor that views this rank's copy, and the base
    address of every rank's copy (indexed by rank within the decomposition group)."""

    def __init__(self, block, tensor: torch.Tensor, ptrs: List[int], nbytes: int, group, world: int):
        self.block, self.tensor, self.ptrs, self.nbytes, self.group, self.world = block, tensor, ptrs, nbytes, group, world
        self.closed = False

    def contains(self, t: torch.Tensor) -> bool:
        p = t.data_ptr()
        return self.ptrs_me <= p and p + t.numel() * t.element_size() <= self.ptrs_me + self.nbytes

    @property
    def ptrs_me(self) -> int:
        return self.tensor.data_ptr()


# allocations by (ranks of the group, device)
_allocations: Dict[tuple, List[PeerAllocation]] = {}


def _key(mesh: Mesh) -> tuple:
    return (tuple(mesh.submesh_ranks()), torch.cuda.current_device())


def empty_peer_visible(mesh: Mesh, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Collective: allocate an uninitialised block of ``shape`` on every rank of ``mesh``'s decomposition
    group, addressable by all of them.  Returns this rank's block as an ordinary tensor (slicing and views
    work; the halo ops recognise it by its address)."""
    if dtype not in _TYPESTR:
        raise TypeError(f"unsupported dtype {dtype}")
    nat = _native.require()
    ranks = mesh.submesh_ranks()
    world = len(ranks)
    me = ranks.index(mesh.rank)
    numel = 1
    for s in shape:
        numel *= int(s)
    nbytes = max(1, numel) * torch.empty((), dtype=dtype).element_size()
    torch.cuda.synchronize()
    block = nat.PeerBlock(nbytes, world, me)
    if world > 1:
        group = mesh.submesh_group()
        blobs: List[bytes] = [b""] * world
        dist.all_gather_object(blobs, block.export_handles(), group=group)
        block.open_peers(blobs)
        dist.barrier(group=group)
    else:
        group = None
    ptrs = [int(block.ptr(p)) for p in range(world)]
    t = torch.as_tensor(_DeviceBuffer(ptrs[me], shape, dtype, block), device=torch.device("cuda", torch.cuda.current_device()))
    alloc = PeerAllocation(block, t, ptrs, nbytes, group, world)
    _allocations.setdefault(_key(mesh), []).append(alloc)
    return t


def empty_sharded(mesh: Mesh, local_shape: Sequence[int], dtype: torch.dtype = torch.float32, spec=None,
                  peer_visible: bool = True) -> ShardedTensor:
    """An uninitialised :class:`ShardedTensor` with the given local block shape; with ``peer_visible`` the
    block can be written by the other ranks of the mesh directly (see the module docstring)."""
    if peer_visible and torch.cuda.is_available():
        local = empty_peer_visible(mesh, local_shape, dtype)
    else:
        local = torch.empty(tuple(local_shape), dtype=dtype)
    return ShardedTensor(local, mesh, spec)


def lookup(mesh: Mesh, t: torch.Tensor) -> Optional[Tuple[PeerAllocation, int]]:
    """The allocation that holds tensor ``t`` and the byte offset of ``t`` inside it, or ``None``."""
    for a in _allocations.get(_key(mesh), ()):
        if not a.closed and a.contains(t):
            return a, t.data_ptr() - a.ptrs_me
    return None


def free_peer_visible(mesh: Optional[Mesh] = None, collective: bool = True) -> None:
    """Release the peer-visible blocks of ``mesh`` (all meshes when ``None``).  Collective unless
    ``collective=False`` (a rank leaving alone only unmaps the other ranks' blocks; its own are left to
    process tear-down, because a peer may still be writing to them).  Tensors made from the blocks must
    not be used afterwards."""
    keys = [_key(mesh)] if mesh is not None else list(_allocations)
    for k in keys:
        for a in _allocations.pop(k, []):
            if a.closed:
                continue
            a.closed = True
            torch.cuda.synchronize()
            met = False
            if a.world > 1 and collective and dist.is_initialized():
                a.block.close_peers()
                dist.barrier(group=a.group)
                met = True
            a.block.close(met or a.world == 1)
