"""Baseline backend: the step lists executed literally with library calls.

``torch.fft`` (cuFFT on GPU), ``torch.distributed.all_to_all_single`` (NCCL on
GPU, gloo on CPU ranks) and ``permute().contiguous()``; halos with batched
``isend``/``irecv``.  This is what XLA lowers the reference's default backend
to (``src/jaxdecomp/_src/jax/fft.py:94-135``: cuFFT + NCCL all-to-all + copy
kernels), so it serves both as the elementwise oracle for the native kernels
and as the same-machine performance baseline.  It is not the product path.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from ..parallel.mesh import Mesh
from .collectives import all_to_all_tiled
from .plan import A2A, Fft, Perm, Step


def run_steps(x: torch.Tensor, steps: Sequence[Step], mesh: Mesh, inverse: bool) -> torch.Tensor:
    """Execute a step list on a local block with optional leading batch dims.
    Transforms are un-normalised in both directions (the inverse is multiplied
    back by its length), matching ``_un_normalize_fft`` of the reference
    (``src/jaxdecomp/_src/fft_utils.py:60-73``)."""
    nb = x.dim() - 3
    for st in steps:
        if isinstance(st, Fft):
            ax = nb + st.axis
            if inverse:
                x = torch.fft.ifft(x, dim=ax, norm="forward")  # norm='forward' on ifft == no scaling
            else:
                x = torch.fft.fft(x, dim=ax)
        elif isinstance(st, A2A):
            p = mesh.pdims[st.mesh_axis]
            if p > 1:
                x = all_to_all_tiled(x, mesh.axis_group(st.mesh_axis), p, nb + st.split, nb + st.concat)
        elif isinstance(st, Perm):
            order = tuple(range(nb)) + tuple(nb + o for o in st.order)
            x = x.permute(order).contiguous()
        else:  # pragma: no cover
            raise TypeError(st)
    return x


def fft_single_device(x: torch.Tensor, inverse: bool, contiguous: bool) -> torch.Tensor:
    """The transform on a mesh of one rank, the way the reference does it there: one ``fftn`` over the
    three axes plus, in contiguous mode, one axis rotation (``src/jaxdecomp/_src/jax/fft.py:285-288``) --
    not three 1-D transforms with a copy after each.  Un-normalised in both directions."""
    nb = x.dim() - 3
    dims = (nb, nb + 1, nb + 2)
    lead = tuple(range(nb))
    if not inverse:
        y = torch.fft.fftn(x, dim=dims)
        return y.permute(lead + (nb + 1, nb + 2, nb)).contiguous() if contiguous else y
    if contiguous:
        x = x.permute(lead + (nb + 2, nb, nb + 1))
    return torch.fft.ifftn(x, dim=dims, norm="forward").contiguous()


def halo_exchange(x: torch.Tensor, halo_extents, halo_periods, mesh: Mesh) -> torch.Tensor:
    """Ghost-cell exchange on the two sharded axes of an already padded block.

    For a sharded axis with extent ``h`` and padded local size ``S``: rows
    ``[S-2h, S-h)`` go to the next rank's ``[0, h)`` and rows ``[h, 2h)`` go to
    the previous rank's ``[S-h, S)``; face slabs span the full padded width of
    the other axis and the four corners are then overwritten with the diagonal
    neighbours' blocks.  A rank at the edge of a non-periodic axis receives
    zeros.  Axes whose mesh size is one are left untouched.  (Reference:
    ``src/jaxdecomp/_src/jax/halo.py:18-196``.)
    """
    nb = x.dim() - 3
    h0, h1 = int(halo_extents[0]), int(halo_extents[1])
    per0, per1 = bool(halo_periods[0]), bool(halo_periods[1])
    p0, p1 = mesh.pdims
    if p0 == 1:
        h0 = 0
    if p1 == 1:
        h1 = 0
    if h0 == 0 and h1 == 0:
        return x.clone()
    a0, a1 = nb, nb + 1
    s0, s1 = x.shape[a0], x.shape[a1]
    if (h0 and s0 < 2 * h0) or (h1 and s1 < 2 * h1):
        raise ValueError(f"padded block {tuple(x.shape)} is smaller than twice the halo extents {(h0, h1)}")

    def sl(lo0, hi0, lo1, hi1):
        idx = [slice(None)] * x.dim()
        idx[a0] = slice(lo0, hi0)
        idx[a1] = slice(lo1, hi1)
        return tuple(idx)

    # (offset on a0, offset on a1) -> (send region of the sender, receive region of the receiver)
    def send_rng(d, h, s):  # data travelling in direction d along an axis
        if d == 0:
            return (0, s)
        return (s - 2 * h, s - h) if d > 0 else (h, 2 * h)

    def recv_rng(d, h, s):
        if d == 0:
            return (0, s)
        return (0, h) if d > 0 else (s - h, s)

    out = x.clone()
    dirs = []
    if h0:
        dirs += [(1, 0), (-1, 0)]
    if h1:
        dirs += [(0, 1), (0, -1)]
    if h0 and h1:
        dirs += [(1, 1), (1, -1), (-1, 1), (-1, -1)]
    ops = []
    updates = []  # (receive region, payload) in application order; payload None -> zeros
    for tag, (d0, d1) in enumerate(dirs):
        dst = mesh.neighbor(d0, d1, (per0, per1))
        src = mesh.neighbor(-d0, -d1, (per0, per1))
        sreg = sl(*send_rng(d0, h0, s0), *send_rng(d1, h1, s1))
        rreg = sl(*recv_rng(d0, h0, s0), *recv_rng(d1, h1, s1))
        if src is None:
            updates.append((rreg, None))
        elif src == mesh.rank:
            updates.append((rreg, x[sreg]))
        else:
            buf = torch.empty_like(x[rreg])
            ops.append(dist.P2POp(dist.irecv, buf, src, tag=tag))
            updates.append((rreg, buf))
        if dst is not None and dst != mesh.rank:
            ops.append(dist.P2POp(dist.isend, x[sreg].contiguous(), dst, tag=tag))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    # faces first, corners last (the order of ``dirs``), so that later writes win
    for rreg, payload in updates:
        if payload is None:
            out[rreg] = 0
        else:
            out[rreg] = payload
    return out


def halo_regions(shape0: int, shape1: int, h0: int, h1: int):
    """The (up to) eight disjoint exchange regions of a padded block.

    Yields ``(d0, d1, send, recv)`` where ``send``/``recv`` are
    ``((lo0, hi0), (lo1, hi1))`` index ranges on the two sharded axes: data in
    the sender's ``send`` range travels by ``(d0, d1)`` mesh steps into the
    receiver's ``recv`` range.  Faces exclude the corner columns/rows, which
    makes the eight receive ranges disjoint; the result equals the
    faces-then-corners overwrite order of the reference.
    """
    def send_rng(d, h, s):
        if d == 0:
            return (h, s - h)
        return (s - 2 * h, s - h) if d > 0 else (h, 2 * h)

    def recv_rng(d, h, s):
        if d == 0:
            return (h, s - h)
        return (0, h) if d > 0 else (s - h, s)

    for d0 in (1, -1, 0):
        for d1 in (1, -1, 0):
            if d0 == 0 and d1 == 0:
                continue
            if (d0 and not h0) or (d1 and not h1):
                continue
            yield d0, d1, (send_rng(d0, h0, shape0), send_rng(d1, h1, shape1)), (
                recv_rng(d0, h0, shape0), recv_rng(d1, h1, shape1))


def halo_accumulate(g: torch.Tensor, halo_extents, halo_periods, mesh: Mesh) -> torch.Tensor:
    """Adjoint of :func:`halo_exchange`: the content of every halo region is
    sent back to the rank it would have been copied from and *added* into that
    rank's send region; the halo regions of the result are zero.

    Besides being the exact gradient rule, this is the reduction needed after
    painting particles onto a padded mesh: mass deposited in a rank's pad
    belongs to the neighbour's interior edge.
    """
    nb = g.dim() - 3
    h0, h1 = int(halo_extents[0]), int(halo_extents[1])
    per = (bool(halo_periods[0]), bool(halo_periods[1]))
    p0, p1 = mesh.pdims
    if p0 == 1:
        h0 = 0
    if p1 == 1:
        h1 = 0
    out = g.clone()
    if h0 == 0 and h1 == 0:
        return out
    a0, a1 = nb, nb + 1
    s0, s1 = g.shape[a0], g.shape[a1]

    def sl(r):
        idx = [slice(None)] * g.dim()
        idx[a0] = slice(*r[0])
        idx[a1] = slice(*r[1])
        return tuple(idx)

    regions = list(halo_regions(s0, s1, h0, h1))
    ops, adds = [], []
    for tag, (d0, d1, send, recv) in enumerate(regions):
        # forward data moved me -> neighbor(d); the adjoint moves neighbor(d)'s recv block back to me
        back_to = mesh.neighbor(-d0, -d1, per)   # rank my recv block came from
        comes_from = mesh.neighbor(d0, d1, per)  # rank that holds the copy of my send block
        payload = g[sl(recv)]
        if comes_from is not None:
            if comes_from == mesh.rank:
                adds.append((sl(send), payload.clone()))
            else:
                buf = torch.empty_like(g[sl(send)])
                ops.append(dist.P2POp(dist.irecv, buf, comes_from, tag=tag))
                adds.append((sl(send), buf))
        if back_to is not None and back_to != mesh.rank:
            ops.append(dist.P2POp(dist.isend, payload.contiguous(), back_to, tag=tag))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    for _, _, _, recv in regions:
        out[sl(recv)] = 0
    for reg, buf in adds:  # fixed order -> deterministic sums
        out[reg] += buf
    return out
