"""Cloud-in-cell painting and read-out on the local mesh block of a rank.

Replaces the chunked XLA scatter of the reference's example
(``examples/scatter.py:59-153``).  Positions are in cell units relative to the
origin of the local, already padded block; along an axis flagged in ``wrap``
neighbour cells are taken modulo the extent, otherwise contributions outside
the block are dropped.  ``lattice=(g0, g1, g2)`` with ``origin`` selects grid
mode: particle ``i`` starts on lattice site ``(i // (g1*g2), (i // g2) % g1,
i % g2) + origin`` and ``pos`` holds displacements.

Both ops are differentiable with respect to positions, weights and the mesh.
CUDA tensors use the native kernels; CPU tensors a plain PyTorch restatement,
which is also the oracle of the tests.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch


def _positions(pos: torch.Tensor, lattice, origin, planar: bool = False) -> torch.Tensor:
    p = pos.reshape(3, -1).t() if planar else pos.reshape(-1, 3)
    if lattice is not None:
        g0, g1, g2 = lattice
        dev = p.device
        a = torch.arange(g0, device=dev, dtype=p.dtype).view(-1, 1, 1) + origin[0]
        b = torch.arange(g1, device=dev, dtype=p.dtype).view(1, -1, 1) + origin[1]
        c = torch.arange(g2, device=dev, dtype=p.dtype).view(1, 1, -1) + origin[2]
        base = torch.stack(torch.broadcast_tensors(a, b, c), dim=-1).reshape(-1, 3)
        p = p + base
    return p


def _neighbours(p: torch.Tensor, shape, wrap):
    """Yield (flat index, weight, validity mask, per-axis weights, signs) for the 8 cells."""
    fl = torch.floor(p)
    i0 = fl.to(torch.long)
    d = p - fl
    for c in range(8):
        bits = [(c >> k) & 1 for k in range(3)]
        idx, ok, w = [], torch.ones(p.shape[0], dtype=torch.bool, device=p.device), []
        for k in range(3):
            j = i0[:, k] + bits[k]
            if wrap[k]:
                j = j % shape[k]
            else:
                ok = ok & (j >= 0) & (j < shape[k])
                j = j.clamp(0, shape[k] - 1)
            idx.append(j)
            w.append(d[:, k] if bits[k] else 1.0 - d[:, k])
        flat = (idx[0] * shape[1] + idx[1]) * shape[2] + idx[2]
        yield flat, ok, w, bits


def _paint_torch(p, weight, shape, wrap):
    mesh = torch.zeros(shape[0] * shape[1] * shape[2], dtype=p.dtype, device=p.device)
    for flat, ok, w, _ in _neighbours(p, shape, wrap):
        val = w[0] * w[1] * w[2] * weight * ok
        mesh.index_add_(0, flat, val)
    return mesh.view(*shape)


def _readout_torch(p, mesh, wrap):
    shape = mesh.shape
    flatmesh = mesh.reshape(-1)
    out = torch.zeros(p.shape[0], dtype=p.dtype, device=p.device)
    for flat, ok, w, _ in _neighbours(p, shape, wrap):
        out = out + flatmesh[flat] * w[0] * w[1] * w[2] * ok
    return out


def _grad_pos_torch(p, weight, gmesh, wrap):
    shape = gmesh.shape
    flatmesh = gmesh.reshape(-1)
    g = torch.zeros_like(p)
    for flat, ok, w, bits in _neighbours(p, shape, wrap):
        v = flatmesh[flat] * weight * ok
        sgn = [1.0 if b else -1.0 for b in bits]
        g[:, 0] += v * sgn[0] * w[1] * w[2]
        g[:, 1] += v * w[0] * sgn[1] * w[2]
        g[:, 2] += v * w[0] * w[1] * sgn[2]
    return g


def _native_call(op, pos, weight, mesh_or_g, out, shape, wrap, lattice, origin, wscalar, planar=False):
    from .. import native

    nat = native.require()
    n = pos.numel() // 3
    nat.cic(op, n, [int(s) for s in shape], [int(bool(w)) for w in wrap],
            [int(g) for g in (lattice or (0, 0, 0))], [float(o) for o in origin], float(wscalar),
            pos.data_ptr(), 0 if weight is None else weight.data_ptr(), mesh_or_g.data_ptr(),
            0 if out is None else out.data_ptr(), torch.cuda.current_stream().cuda_stream, bool(planar))


def _use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.float32


def _paint_impl(pos, weight, wscalar, shape, wrap, lattice, origin, planar=False):
    if _use_native(pos):
        mesh = torch.zeros(shape, dtype=torch.float32, device=pos.device)
        _native_call(0, pos.contiguous(), None if weight is None else weight.contiguous(), mesh, None, shape, wrap,
                     lattice, origin, wscalar, planar)
        return mesh
    w = weight.reshape(-1) if weight is not None else torch.as_tensor(wscalar, dtype=pos.dtype, device=pos.device)
    return _paint_torch(_positions(pos, lattice, origin, planar), w, tuple(shape), wrap)


def _readout_impl(pos, mesh, wrap, lattice, origin, planar=False):
    if _use_native(pos):
        out = torch.empty(pos.numel() // 3, dtype=torch.float32, device=pos.device)
        _native_call(1, pos.contiguous(), None, mesh.contiguous(), out, mesh.shape, wrap, lattice, origin, 1.0, planar)
        return out
    return _readout_torch(_positions(pos, lattice, origin, planar), mesh, wrap)


def _grad_pos_impl(pos, weight, wscalar, gmesh, wrap, lattice, origin, planar=False):
    if _use_native(pos):
        g = torch.empty_like(pos, memory_format=torch.contiguous_format)
        _native_call(2, pos.contiguous(), None if weight is None else weight.contiguous(), gmesh.contiguous(), g,
                     gmesh.shape, wrap, lattice, origin, wscalar, planar)
        return g
    w = weight.reshape(-1) if weight is not None else torch.as_tensor(wscalar, dtype=pos.dtype, device=pos.device)
    g = _grad_pos_torch(_positions(pos, lattice, origin, planar), w, gmesh, wrap)
    return (g.t() if planar else g).reshape(pos.shape)


class _Paint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pos, weight, wscalar, shape, wrap, lattice, origin, planar=False):
        ctx.save_for_backward(pos, weight if weight is not None else pos.new_empty(0))
        ctx.meta = (wscalar, tuple(shape), tuple(wrap), lattice, tuple(origin), weight is not None, planar)
        return _paint_impl(pos, weight, wscalar, shape, wrap, lattice, origin, planar)

    @staticmethod
    def backward(ctx, g):
        pos, weight = ctx.saved_tensors
        wscalar, shape, wrap, lattice, origin, has_w, planar = ctx.meta
        weight = weight if has_w else None
        g = g.contiguous()
        gpos = gw = None
        if ctx.needs_input_grad[0]:
            gpos = _grad_pos_impl(pos, weight, wscalar, g, wrap, lattice, origin, planar)
        if has_w and ctx.needs_input_grad[1]:
            gw = _readout_impl(pos, g, wrap, lattice, origin, planar).reshape(weight.shape)
        return gpos, gw, None, None, None, None, None, None


class _Readout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pos, mesh, wrap, lattice, origin, planar=False):
        ctx.save_for_backward(pos, mesh)
        ctx.meta = (tuple(wrap), lattice, tuple(origin), planar)
        return _readout_impl(pos, mesh, wrap, lattice, origin, planar)

    @staticmethod
    def backward(ctx, g):
        pos, mesh = ctx.saved_tensors
        wrap, lattice, origin, planar = ctx.meta
        g = g.contiguous()
        gpos = gmesh = None
        if ctx.needs_input_grad[0]:
            gpos = _grad_pos_impl(pos, g, 1.0, mesh, wrap, lattice, origin, planar)
        if ctx.needs_input_grad[1]:
            gmesh = _paint_impl(pos, g, 1.0, mesh.shape, wrap, lattice, origin, planar)
        return gpos, gmesh, None, None, None, None


def cic_paint(pos: torch.Tensor, mesh_shape: Sequence[int], weight: Optional[torch.Tensor] = None, value: float = 1.0,
              wrap: Sequence[bool] = (False, False, True), lattice: Optional[Sequence[int]] = None,
              origin: Sequence[float] = (0.0, 0.0, 0.0), planar: bool = False) -> torch.Tensor:
    """Deposit particles onto a zero-initialised mesh of ``mesh_shape`` with trilinear weights.

    ``pos`` is ``[..., 3]``, or with ``planar=True`` three planes ``[3, ...]`` -- the layout in which a
    batched inverse FFT returns the three displacement fields, so that they can be painted without
    interleaving them first."""
    if (pos.shape[0] if planar else pos.shape[-1]) != 3:
        raise ValueError("pos must have a leading (planar) or trailing dimension of 3")
    lat = tuple(int(g) for g in lattice) if lattice is not None else None
    if lat is not None and lat[0] * lat[1] * lat[2] != pos.numel() // 3:
        raise ValueError("lattice does not match the number of particles")
    return _Paint.apply(pos, weight, float(value), tuple(int(s) for s in mesh_shape), tuple(bool(w) for w in wrap), lat,
                        tuple(float(o) for o in origin), bool(planar))


def cic_readout(pos: torch.Tensor, mesh: torch.Tensor, wrap: Sequence[bool] = (False, False, True),
                lattice: Optional[Sequence[int]] = None, origin: Sequence[float] = (0.0, 0.0, 0.0),
                planar: bool = False) -> torch.Tensor:
    """Interpolate the mesh at the particle positions (adjoint of :func:`cic_paint`)."""
    lat = tuple(int(g) for g in lattice) if lattice is not None else None
    out = _Readout.apply(pos, mesh, tuple(bool(w) for w in wrap), lat, tuple(float(o) for o in origin), bool(planar))
    return out.reshape(pos.shape[1:] if planar else pos.shape[:-1])
