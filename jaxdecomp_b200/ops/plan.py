"""Declarative pipelines for the distributed FFT and the pencil transposes.

Every distributed op of this package is described once, as a short list of
steps over the *local* block of a rank:

* ``Fft(axis)``          un-normalised 1-D transform along a local axis,
* ``A2A(mesh_axis, split, concat)``  tiled all-to-all over one decomposition
  axis of the mesh (0 = ``a0``, 1 = ``a1``),
* ``Perm(order)``        local axis permutation.

The baseline backend executes the steps literally (``torch.fft`` +
``all_to_all_single`` + ``permute``).  The native backend compiles runs of
``Fft [A2A] [Perm...]`` into single kernel passes whose stores land directly in
the destination layout on the destination rank.  Both therefore share one
source of truth for data movement, and output specs/shapes are derived
mechanically from the same lists.

The step lists restate the behaviour of the reference's per-shard pipelines
(``src/jaxdecomp/_src/jax/fft.py:28-264``) and transposes
(``src/jaxdecomp/_src/jax/transpose.py:76-108``).  Two identities keep the
table small: the pencil pipeline run on a mesh with ``P0 == 1`` produces
exactly the slab-YZ result, and with ``P0 == P1 == 1`` the single-device
result, so only slab-XY needs lists of its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple, Union

from ..utils.config import SLAB_XY, Decomposition


@dataclass(frozen=True)
class Fft:
    axis: int


@dataclass(frozen=True)
class A2A:
    mesh_axis: int  # 0 -> a0 (size P0), 1 -> a1 (size P1)
    split: int
    concat: int


@dataclass(frozen=True)
class Perm:
    order: Tuple[int, int, int]


Step = Union[Fft, A2A, Perm]

ROT_FWD = (2, 0, 1)  # new[i] = old[order[i]]: brings the last axis to the front
ROT_BWD = (1, 2, 0)


def fft_steps(pencil_type: Decomposition, inverse: bool, contiguous: bool, native: bool = False) -> List[Step]:
    """Step list of ``pfft3d`` (``inverse=False``) or ``pifft3d`` for a decomposition.

    ``native=True`` returns an equivalent list in which every transform is
    followed by at most a two-axis re-layout (what one kernel pass can do); it
    differs from the literal list only for the forward slab-XY pipeline, where
    the local rotation is moved in front of the second transform.
    """
    pt = Decomposition(int(pencil_type))
    xy = pt == SLAB_XY
    if contiguous:
        if not inverse:
            if xy and native:
                return [Fft(2), Perm(ROT_FWD), Fft(2), A2A(0, 0, 1), Perm(ROT_FWD), Fft(2)]
            if xy:
                return [Fft(2), Fft(1), A2A(0, 2, 0), Perm(ROT_BWD), Fft(2)]
            return [Fft(2), A2A(1, 2, 1), Perm(ROT_FWD), Fft(2), A2A(0, 2, 1), Perm(ROT_FWD), Fft(2)]
        if xy:
            return [Fft(2), A2A(0, 2, 1), Perm(ROT_FWD), Fft(2), Fft(1)]
        return [Fft(2), A2A(0, 2, 0), Perm(ROT_BWD), Fft(2), A2A(1, 2, 0), Perm(ROT_BWD), Fft(2)]
    if not inverse:
        if xy:
            return [Fft(2), Fft(1), A2A(0, 2, 0), Fft(0)]
        return [Fft(2), A2A(1, 2, 1), Fft(1), A2A(0, 1, 0), Fft(0)]
    if xy:
        return [Fft(0), A2A(0, 0, 2), Fft(2), Fft(1)]
    return [Fft(0), A2A(0, 0, 1), Fft(1), A2A(1, 1, 2), Fft(2)]


_TRANSPOSE_CONTIG = {
    "x_y": [A2A(1, 2, 1), Perm(ROT_FWD)],
    "y_z": [A2A(0, 2, 1), Perm(ROT_FWD)],
    "z_y": [A2A(0, 2, 0), Perm(ROT_BWD)],
    "y_x": [A2A(1, 2, 0), Perm(ROT_BWD)],
    "x_z": [A2A(0, 2, 0), Perm(ROT_BWD)],
    "z_x": [A2A(0, 2, 1), Perm(ROT_FWD)],
}
_TRANSPOSE_NONCONTIG = {
    "x_y": [A2A(1, 2, 1)],
    "y_z": [A2A(0, 1, 0)],
    "z_y": [A2A(0, 0, 1)],
    "y_x": [A2A(1, 1, 2)],
    "x_z": [A2A(0, 2, 0)],
    "z_x": [A2A(0, 0, 2)],
}
TRANSPOSE_KINDS = tuple(_TRANSPOSE_CONTIG)
INVERSE_KIND = {"x_y": "y_x", "y_x": "x_y", "y_z": "z_y", "z_y": "y_z", "x_z": "z_x", "z_x": "x_z"}


def transpose_steps(kind: str, contiguous: bool) -> List[Step]:
    table = _TRANSPOSE_CONTIG if contiguous else _TRANSPOSE_NONCONTIG
    if kind not in table:
        raise ValueError(f"Invalid transpose kind {kind!r}; expected one of {TRANSPOSE_KINDS}")
    return list(table[kind])


def propagate(steps: Sequence[Step], local_shape: Sequence[int], spec: Sequence, pdims: Sequence[int],
              axis_names: Sequence) -> Tuple[tuple, tuple]:
    """Push a local shape and a spec through a step list.

    An all-to-all over mesh axis ``m`` un-shards the concat dimension and
    shards the split dimension by ``m``; a permutation reorders both.
    Returns ``(local_shape, spec)`` after the last step and raises
    ``ValueError`` when an extent cannot be split evenly.
    """
    shape = list(int(s) for s in local_shape)
    spec = list(spec) + [None] * (3 - len(spec))
    for st in steps:
        if isinstance(st, A2A):
            p = int(pdims[st.mesh_axis])
            if p == 1:
                continue
            if shape[st.split] % p:
                raise ValueError(
                    f"local extent {shape[st.split]} of axis {st.split} cannot be split over the {p} ranks of "
                    f"mesh axis {axis_names[st.mesh_axis]!r}"
                )
            shape[st.split] //= p
            shape[st.concat] *= p
            name = axis_names[st.mesh_axis]
            if spec[st.concat] == name:
                spec[st.concat] = None
            spec[st.split] = name
        elif isinstance(st, Perm):
            shape = [shape[i] for i in st.order]
            spec = [spec[i] for i in st.order]
    return tuple(shape), tuple(spec)


def check_input_spec(steps: Sequence[Step], spec: Sequence, pdims: Sequence[int], axis_names: Sequence) -> None:
    """Verify that every all-to-all of the list finds its concat dimension
    sharded by the mesh axis it runs over (i.e. the op is applied to an array
    in the layout it expects)."""
    spec = list(spec) + [None] * (3 - len(spec))
    for st in steps:
        if isinstance(st, A2A):
            if int(pdims[st.mesh_axis]) == 1:
                continue
            name = axis_names[st.mesh_axis]
            if spec[st.concat] != name:
                raise ValueError(
                    f"operand spec {tuple(spec)} is not the layout this operation expects: dimension "
                    f"{st.concat} should be sharded over mesh axis {name!r}"
                )
            spec[st.concat] = None
            if spec[st.split] is not None:
                raise ValueError(
                    f"operand spec {tuple(spec)}: dimension {st.split} is already sharded and cannot "
                    f"receive mesh axis {name!r}"
                )
            spec[st.split] = name
        elif isinstance(st, Perm):
            spec = [spec[i] for i in st.order]
