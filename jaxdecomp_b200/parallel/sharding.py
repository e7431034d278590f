"""Partition specs, named shardings, the sharded-tensor handle and the spec
algebra of the distributed FFT.

Parity targets in the reference: ``validate_spec_matches_mesh``
(``src/jaxdecomp/_src/pencil_utils.py:114-142``), ``get_output_specs``
(``pencil_utils.py:235-330``), ``get_fft_output_sharding``
(``pencil_utils.py:218-232``) and ``PencilInfo``
(``src/csrc/include/jaxdecomp.h:90-97``).

A :class:`ShardedTensor` is what a global ``jax.Array`` is in the reference,
seen from one process: the local block, the mesh, the spec and the global shape.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch

from ..utils.config import NO_DECOMP, PENCILS, SLAB_XY, SLAB_YZ, Decomposition, config
from ..utils.errors import ShardingError
from .mesh import Mesh, current_mesh


class PartitionSpec(tuple):
    """Tuple of mesh-axis names (or None), one per array dimension."""

    def __new__(cls, *names):
        return super().__new__(cls, names)

    def __repr__(self):
        return "PartitionSpec" + tuple.__repr__(self)

    def padded(self, n: int) -> "PartitionSpec":
        return PartitionSpec(*(tuple(self) + (None,) * (n - len(self))))


P = PartitionSpec


@dataclass(frozen=True)
class NamedSharding:
    mesh: Mesh
    spec: PartitionSpec

    def shard_shape(self, global_shape: Sequence[int]) -> tuple:
        return local_shape(global_shape, self.spec, self.mesh)


def _spec_tuple(spec) -> tuple:
    if spec is None:
        return ()
    return tuple(spec)


def local_shape(global_shape: Sequence[int], spec, mesh: Mesh) -> tuple:
    spec = _spec_tuple(spec)
    spec = spec + (None,) * (len(global_shape) - len(spec))
    out = []
    for n, name in zip(global_shape, spec):
        p = 1 if name is None else mesh.axis_size(name)
        if n % p:
            raise ShardingError(
                f"global extent {n} is not divisible by the size {p} of mesh axis {name!r}; "
                "uneven decompositions are not supported"
            )
        out.append(n // p)
    return tuple(out)


def global_shape_of(local: Sequence[int], spec, mesh: Mesh) -> tuple:
    spec = _spec_tuple(spec)
    spec = spec + (None,) * (len(local) - len(spec))
    return tuple(n * (1 if name is None else mesh.axis_size(name)) for n, name in zip(local, spec))


def shard_offsets(global_shape: Sequence[int], spec, mesh: Mesh, rank: Optional[int] = None) -> tuple:
    """Global index of the first local element along every array dimension."""
    spec = _spec_tuple(spec)
    spec = spec + (None,) * (len(global_shape) - len(spec))
    coords = mesh.coords if rank is None else mesh.coords_of(rank)
    out = []
    for n, name in zip(global_shape, spec):
        if name is None:
            out.append(0)
        else:
            ai = mesh.axis_names.index(name)
            out.append(coords[ai] * (n // mesh.shape[ai]))
    return tuple(out)


def validate_spec_matches_mesh(spec, mesh: Mesh) -> None:
    """Check that ``spec`` names the two decomposition axes in mesh order.

    Position ``i`` of the (3-padded) spec must hold the name of decomposition
    axis ``i``, or ``None`` when that mesh axis has size one or when ``i`` is
    past the mesh axes.  Raises ``ValueError`` naming the offending position.
    """
    spec = _spec_tuple(spec)
    spec = spec + (None,) * (3 - len(spec))
    names = tuple(mesh.decomp_axis_names)
    sizes = mesh.pdims
    for i in range(3):
        want = names[i] if i < len(names) else None
        if spec[i] is not None:
            if want is None or spec[i] != want:
                raise ValueError(
                    f"Spec {spec} does not match mesh axis names {names}. At position {i}: spec has "
                    f"'{spec[i]}' but mesh expects '{want if want is not None else 'nothing (trailing)'}'. "
                    "Ensure the array is sharded with a spec matching the mesh axis order."
                )
        elif i < len(names) and sizes[i] > 1:
            raise ValueError(
                f"Spec {spec} does not match mesh axis names {names}. At position {i}: spec has None "
                f"but mesh axis '{names[i]}' has size {sizes[i]} (> 1). "
                "An unsharded dimension cannot correspond to a distributed mesh axis."
            )


def _as_decomp(pencil_type) -> Decomposition:
    if isinstance(pencil_type, str):
        return Decomposition[pencil_type.upper()]
    return Decomposition(int(pencil_type))


def get_output_specs(fft_type, pencil_type, spec, backend: str = "JAX") -> tuple:
    """Spec of the result of a distributed FFT.

    ``fft_type`` is ``'fft'``/``'ifft'`` (any case; ``'rfft'``/``'irfft'`` are
    treated like their complex counterparts).  In contiguous mode the output
    array is rotated, so only slabs change their spec; in non-contiguous mode
    the array keeps its axis order and the sharded dimensions migrate.
    """
    kind = str(getattr(fft_type, "name", fft_type)).lower()
    if kind not in ("fft", "ifft", "rfft", "irfft"):
        raise TypeError("only complex FFTs are currently supported through pfft.")
    forward = kind in ("fft", "rfft")
    pt = _as_decomp(pencil_type)
    spec = _spec_tuple(spec)
    spec = spec + (None,) * (3 - len(spec))
    if config.transpose_axis_contiguous:
        if pt == SLAB_XY:
            return (spec[1], spec[0], spec[2])
        if pt == SLAB_YZ:
            return (spec[2], spec[1], spec[0])
        if pt in (PENCILS, NO_DECOMP):
            return tuple(spec)
        raise TypeError("Unknown pencil type")
    if forward:
        if spec[2] is not None:
            raise ValueError(
                "Distributed FFTs with non-contiguous axes do not support a third distributed axis; "
                f"make sure the device mesh is 1-D or 2-D, got spec {spec}"
            )
        if pt == SLAB_XY:
            return (spec[2], spec[1], spec[0])
        if pt == SLAB_YZ:
            return (spec[0], spec[2], spec[1])
        if pt in (PENCILS, NO_DECOMP):
            return (spec[2], spec[0], spec[1])
        raise TypeError("Unknown pencil type")
    if pt == SLAB_XY:
        return (spec[2], spec[1], spec[0])
    if pt == SLAB_YZ:
        if spec[0] is not None or spec[1] is not None:
            raise ValueError(
                "Distributed IFFT with a YZ slab is not compatible with the current sharding, "
                f"got {spec}; apply the inverse to the output of a distributed forward FFT"
            )
        return (spec[0], spec[2], spec[1])
    if pt in (PENCILS, NO_DECOMP):
        if spec[0] is not None:
            raise ValueError(
                "Distributed IFFT with a PENCILS decomposition is not compatible with the current "
                f"sharding, got {spec}; apply the inverse to the output of a distributed forward FFT"
            )
        return (spec[1], spec[2], spec[0])
    raise TypeError("Unknown pencil type")


def get_fft_output_sharding(sharding: NamedSharding) -> NamedSharding:
    """Sharding of ``pfft3d``'s result for an input with the given sharding;
    a leading batch entry of a 4-D spec passes through unchanged."""
    spec = _spec_tuple(sharding.spec)
    mesh = sharding.mesh
    batched = len(spec) >= 4 or (len(spec) >= 1 and spec[0] is not None and spec[0] in mesh.batch_axis_names)
    if batched:
        out = get_output_specs("fft", mesh.pencil_type, spec[1:])
        return NamedSharding(mesh, P(spec[0], *out))
    out = get_output_specs("fft", mesh.pencil_type, spec)
    return NamedSharding(mesh, P(*out))


@dataclass(frozen=True)
class PencilInfo:
    """Geometry of this rank's pencil for one of the three pencil orientations.

    ``shape``/``lo``/``hi`` are given in the pencil's memory order (slowest
    first); ``order[i]`` is the global axis stored at memory position ``i``;
    ``hi`` is inclusive, as in the reference's native struct.
    """

    shape: Tuple[int, int, int]
    lo: Tuple[int, int, int]
    hi: Tuple[int, int, int]
    order: Tuple[int, int, int]
    halo_extents: Tuple[int, int, int]
    size: int


def pencil_info(gdims: Sequence[int], pdims: Sequence[int], axis: int, coords: Sequence[int],
                halo_extents: Sequence[int] = (0, 0, 0), contiguous: Optional[bool] = None) -> PencilInfo:
    """Pencil geometry for ``axis`` (0 = X-pencil: the input layout, 1 = Y-pencil,
    2 = Z-pencil: the layout of the forward FFT's output).

    ``gdims`` is the global shape of the X-pencil array ``(N0, N1, N2)``; the
    decomposition axes ``(a0, a1)`` have sizes ``pdims`` and this rank sits at
    ``coords`` on them.
    """
    if contiguous is None:
        contiguous = config.transpose_axis_contiguous
    n0, n1, n2 = (int(g) for g in gdims)
    p0, p1 = (int(p) for p in pdims)
    c0, c1 = (int(c) for c in coords)
    g = (n0, n1, n2)
    # (global axis -> (mesh axis index or None)) for the three pencil orientations
    if axis == 0:
        shard = {0: 0, 1: 1}
        order = (0, 1, 2)
    elif axis == 1:
        shard = {0: 0, 2: 1}
        order = (2, 0, 1) if contiguous else (0, 1, 2)
    elif axis == 2:
        shard = {1: 0, 2: 1}
        order = (1, 2, 0) if contiguous else (0, 1, 2)
    else:
        raise ValueError("axis must be 0, 1 or 2")
    psz = (p0, p1)
    pc = (c0, c1)
    shape, lo, hi, halos = [], [], [], []
    for gax in order:
        n = g[gax]
        if gax in shard:
            p = psz[shard[gax]]
            if n % p:
                raise ShardingError(f"global extent {n} of axis {gax} is not divisible by {p}")
            ln = n // p
            start = pc[shard[gax]] * ln
        else:
            ln, start = n, 0
        h = int(halo_extents[gax])
        shape.append(ln + 2 * h)
        lo.append(start)
        hi.append(start + ln - 1)
        halos.append(h)
    size = shape[0] * shape[1] * shape[2]
    return PencilInfo(tuple(shape), tuple(lo), tuple(hi), tuple(order), tuple(halos), size)


class ShardedTensor:
    """Local block of a globally sharded array plus the metadata to interpret it.

    Arithmetic is done on ``.local`` (a regular ``torch.Tensor`` that takes
    part in autograd); the distributed ops of this package accept and return
    ``ShardedTensor``.
    """

    __slots__ = ("local", "mesh", "spec", "global_shape")

    def __init__(self, local: torch.Tensor, mesh: Mesh, spec=None, global_shape: Optional[Sequence[int]] = None):
        nd = local.dim()
        if nd not in (3, 4):
            raise ShardingError(f"expected a 3-D array (or 4-D with a leading batch), got {nd}-D")
        if spec is None:
            a0, a1 = mesh.decomp_axis_names
            spec = (None,) * (nd - 3) + (a0 if mesh.pdims[0] > 1 else None, a1 if mesh.pdims[1] > 1 else None, None)
        spec = _spec_tuple(spec)
        spec = spec + (None,) * (nd - len(spec))
        self.local = local
        self.mesh = mesh
        self.spec = PartitionSpec(*spec)
        if global_shape is None:
            global_shape = global_shape_of(local.shape, spec, mesh)
        self.global_shape = tuple(int(s) for s in global_shape)
        want = local_shape(self.global_shape, spec, mesh)
        if tuple(local.shape) != want:
            raise ShardingError(
                f"local block {tuple(local.shape)} does not match global shape {self.global_shape} "
                f"sharded as {self.spec} on mesh {mesh.shape} (expected {want})"
            )

    # --- conveniences ---------------------------------------------------------------------
    @property
    def sharding(self) -> NamedSharding:
        return NamedSharding(self.mesh, self.spec)

    @property
    def shape(self) -> tuple:
        return self.global_shape

    @property
    def dtype(self):
        return self.local.dtype

    @property
    def device(self):
        return self.local.device

    @property
    def spatial_spec(self) -> tuple:
        return tuple(self.spec[-3:])

    @property
    def offsets(self) -> tuple:
        return shard_offsets(self.global_shape, self.spec, self.mesh)

    def with_local(self, local: torch.Tensor, spec=None, global_shape=None) -> "ShardedTensor":
        return ShardedTensor(local, self.mesh, self.spec if spec is None else spec, global_shape)

    def is_complex(self) -> bool:
        return self.local.is_complex()

    def detach(self) -> "ShardedTensor":
        return ShardedTensor(self.local.detach(), self.mesh, self.spec, self.global_shape)

    def requires_grad_(self, flag: bool = True) -> "ShardedTensor":
        self.local.requires_grad_(flag)
        return self

    def _binary(self, other, fn):
        o = other.local if isinstance(other, ShardedTensor) else other
        return ShardedTensor(fn(self.local, o), self.mesh, self.spec, self.global_shape)

    def __mul__(self, o):
        return self._binary(o, torch.mul)

    __rmul__ = __mul__

    def __add__(self, o):
        return self._binary(o, torch.add)

    __radd__ = __add__

    def __sub__(self, o):
        return self._binary(o, torch.sub)

    def __truediv__(self, o):
        return self._binary(o, torch.div)

    def abs(self):
        return ShardedTensor(self.local.abs(), self.mesh, self.spec, self.global_shape)

    def global_sum(self) -> torch.Tensor:
        """Sum over the whole global array (differentiable all-reduce)."""
        s = self.local.sum()
        if self.mesh.world_size > 1:
            from ..ops.collectives import all_reduce_sum

            s = all_reduce_sum(s, self.mesh.submesh_group())
        return s

    def gather(self) -> torch.Tensor:
        """Assemble the global array on every rank (test/debug helper; the
        counterpart of ``process_allgather(tiled=True)`` in the reference's tests)."""
        from ..ops.collectives import gather_global

        return gather_global(self)

    def __repr__(self):
        return (
            f"ShardedTensor(global_shape={self.global_shape}, spec={tuple(self.spec)}, "
            f"local={tuple(self.local.shape)}, dtype={self.local.dtype}, mesh={self.mesh.shape})"
        )


def shard(global_array: torch.Tensor, mesh: Mesh, spec=None) -> ShardedTensor:
    """Slice this rank's block out of a replicated global array."""
    nd = global_array.dim()
    if spec is None:
        a0, a1 = mesh.decomp_axis_names
        spec = (None,) * (nd - 3) + (a0 if mesh.pdims[0] > 1 else None, a1 if mesh.pdims[1] > 1 else None, None)
    spec = _spec_tuple(spec) + (None,) * (nd - len(_spec_tuple(spec)))
    lshape = local_shape(global_array.shape, spec, mesh)
    offs = shard_offsets(global_array.shape, spec, mesh)
    idx = tuple(slice(o, o + n) for o, n in zip(offs, lshape))
    return ShardedTensor(global_array[idx].contiguous(), mesh, spec, tuple(global_array.shape))


def as_sharded(x, mesh: Optional[Mesh] = None, spec=None) -> Tuple[ShardedTensor, bool]:
    """Normalise an op input.  Returns ``(sharded, was_plain)``: plain tensors
    are interpreted as the local block under the active mesh (``with mesh:`` or
    :func:`set_mesh`), in the layout the op expects.  Without an active mesh a
    plain tensor is a complete array on a mesh of one rank -- unless the process
    belongs to a job of several ranks: a tensor without sharding information
    would then be transformed by every rank on its own, which is never what a
    distributed op is called for, so this raises (the analogue of the reference's
    diagnostics for unsharded operands, ``src/jaxdecomp/_src/error.py:1-18``).
    Use ``with jd.single_rank_mesh():`` to transform a replicated array on purpose."""
    if isinstance(x, ShardedTensor):
        return x, False
    if not isinstance(x, torch.Tensor):
        raise TypeError(f"expected a torch.Tensor or ShardedTensor, got {type(x)}")
    if mesh is None:
        mesh = current_mesh()
    if mesh is None:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            from ..utils.errors import error_unsharded_operand

            raise error_unsharded_operand("distributed op")
        from .mesh import single_rank_mesh

        mesh = single_rank_mesh()
    return ShardedTensor(x, mesh, spec), True
