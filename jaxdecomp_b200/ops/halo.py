"""Halo (ghost-cell) exchange and the helpers around it.

``halo_exchange`` follows ``src/jaxdecomp/halo.py:8-80`` of the reference: the
operand's local blocks are already padded, extents and periodicity are given
for the two sharded axes, and the result has the same shape and sharding.  The
reference leaves padding to the user (``shard_map(jnp.pad)``,
``docs/01-basic_usage.md:80-96``); since PyTorch has no ``shard_map`` the
helpers ``pad_halo``, ``unpad_halo`` and ``halo_reduce`` (accumulate overflow
into the neighbours and crop) are provided here.

Gradient: by default the exact adjoint (halo cotangents are added into the
interior edge of the rank the values came from, and the halo cotangent of the
input is zero).  The reference instead applies ``halo_exchange`` to the
cotangent (``src/jaxdecomp/_src/jax/halo.py:401-420``); set
``config.reference_compat_halo_grad = True`` to reproduce that rule.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.nn.functional as F

from ..parallel.sharding import ShardedTensor, as_sharded
from ..utils.config import config
from .dispatch import resolve_backend


def _exchange(x, mesh, extents, periods, backend):
    if backend == "b200":
        from . import b200_backend

        return b200_backend.halo_exchange(x, extents, periods, mesh)
    from . import torch_backend

    return torch_backend.halo_exchange(x, extents, periods, mesh)


def _accumulate(g, mesh, extents, periods, backend):
    if backend == "b200":
        from . import b200_backend

        return b200_backend.halo_accumulate(g, extents, periods, mesh)
    from . import torch_backend

    return torch_backend.halo_accumulate(g, extents, periods, mesh)


class _HaloExchange(torch.autograd.Function):
    @staticmethod
    def forward(x, mesh, extents, periods, backend, compat):
        return _exchange(x, mesh, extents, periods, backend)

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.args = tuple(inputs[1:])

    @staticmethod
    def backward(ctx, g):
        mesh, extents, periods, backend, compat = ctx.args
        if compat:
            gx = _HaloExchange.apply(g.contiguous(), mesh, extents, periods, backend, compat)
        else:
            gx = _HaloAccumulate.apply(g.contiguous(), mesh, extents, periods, backend)
        return gx, None, None, None, None, None

    @staticmethod
    def jvp(ctx, t, *_):
        mesh, extents, periods, backend, compat = ctx.args
        return _HaloExchange.apply(t.contiguous(), mesh, extents, periods, backend, compat)

    @staticmethod
    def vmap(info, in_dims, x, *args):
        from .fft import _vmap_leading

        return _vmap_leading(_HaloExchange.apply, in_dims, x, args)


class _HaloAccumulate(torch.autograd.Function):
    @staticmethod
    def forward(g, mesh, extents, periods, backend):
        return _accumulate(g, mesh, extents, periods, backend)

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.args = tuple(inputs[1:])

    @staticmethod
    def backward(ctx, gg):
        mesh, extents, periods, backend = ctx.args
        # the adjoint of the adjoint is the exchange itself
        y = _HaloExchange.apply(gg.contiguous(), mesh, extents, periods, backend, False)
        return y, None, None, None, None

    @staticmethod
    def jvp(ctx, t, *_):
        mesh, extents, periods, backend = ctx.args
        return _HaloAccumulate.apply(t.contiguous(), mesh, extents, periods, backend)

    @staticmethod
    def vmap(info, in_dims, x, *args):
        from .fft import _vmap_leading

        return _vmap_leading(_HaloAccumulate.apply, in_dims, x, args)


def _effective_extents(mesh, extents):
    h0, h1 = int(extents[0]), int(extents[1])
    if mesh.pdims[0] == 1:
        h0 = 0
    if mesh.pdims[1] == 1:
        h1 = 0
    return h0, h1


def _check(extents, periods):
    if len(extents) != 2 or len(periods) != 2:
        raise ValueError("halo_extents and halo_periods take one entry per sharded axis: (h0, h1), (p0, p1)")
    if any(int(h) < 0 for h in extents):
        raise ValueError(f"negative halo extent in {tuple(extents)}")
    return (int(extents[0]), int(extents[1])), (bool(periods[0]), bool(periods[1]))


def halo_exchange(x, halo_extents: Sequence[int], halo_periods: Sequence[bool], backend: str = "auto"):
    """Fill the halo regions of a padded sharded array from the neighbouring ranks.

    For each sharded axis with extent ``h`` and padded local size ``S``, rows
    ``[S-2h, S-h)`` land in the next rank's ``[0, h)`` and rows ``[h, 2h)`` in the
    previous rank's ``[S-h, S)``; corners come from the diagonal neighbours.
    At the edge of a non-periodic axis the halo is filled with zeros.  Axes
    whose mesh size is one are not exchanged.
    """
    extents, periods = _check(halo_extents, halo_periods)
    st, plain = as_sharded(x)
    b = resolve_backend(backend, st.local, family="halo")
    y = _HaloExchange.apply(st.local.contiguous(), st.mesh, extents, periods, b,
                            bool(config.reference_compat_halo_grad))
    return y if plain else ShardedTensor(y, st.mesh, st.spec)


def halo_exchange_(x, halo_extents: Sequence[int], halo_periods: Sequence[bool], backend: str = "auto"):
    """In-place variant of :func:`halo_exchange`: overwrites the halo regions of ``x`` and returns it.
    Not differentiable (use the functional op under autograd).  On the native backend this skips the
    copy of the padded block, so only the face and corner slabs move."""
    extents, periods = _check(halo_extents, halo_periods)
    st, plain = as_sharded(x)
    if st.local.requires_grad and torch.is_grad_enabled():
        raise RuntimeError("halo_exchange_ is not differentiable; use halo_exchange")
    b = resolve_backend(backend, st.local, family="halo")
    if b == "b200":
        from . import b200_backend

        b200_backend.halo_exchange(st.local, extents, periods, st.mesh, inplace=True)
    else:
        from . import torch_backend

        st.local.copy_(torch_backend.halo_exchange(st.local, extents, periods, st.mesh))
    return x


def halo_accumulate(x, halo_extents: Sequence[int], halo_periods: Sequence[bool], backend: str = "auto"):
    """Add the content of every halo region into the interior edge of the rank
    that owns those cells, and zero the halos (adjoint of :func:`halo_exchange`)."""
    extents, periods = _check(halo_extents, halo_periods)
    st, plain = as_sharded(x)
    b = resolve_backend(backend, st.local, family="halo")
    y = _HaloAccumulate.apply(st.local.contiguous(), st.mesh, extents, periods, b)
    return y if plain else ShardedTensor(y, st.mesh, st.spec)


def pad_halo(x, halo_extents: Sequence[int], value: float = 0.0):
    """Pad the two sharded axes of every local block by ``(h0, h1)`` cells on both sides."""
    h0, h1 = int(halo_extents[0]), int(halo_extents[1])
    st, plain = as_sharded(x)
    y = F.pad(st.local, (0, 0, h1, h1, h0, h0), value=value)
    return y if plain else ShardedTensor(y, st.mesh, st.spec)


def _unpad_local(y: torch.Tensor, h0: int, h1: int) -> torch.Tensor:
    nb = y.dim() - 3
    if h0:
        y = y.narrow(nb, h0, y.shape[nb] - 2 * h0)
    if h1:
        y = y.narrow(nb + 1, h1, y.shape[nb + 1] - 2 * h1)
    return y.contiguous()


def unpad_halo(x, halo_extents: Sequence[int]):
    """Inverse of :func:`pad_halo`: crop ``(h0, h1)`` cells from both sides."""
    st, plain = as_sharded(x)
    y = _unpad_local(st.local, int(halo_extents[0]), int(halo_extents[1]))
    return y if plain else ShardedTensor(y, st.mesh, st.spec)


def halo_reduce(x, halo_extents: Sequence[int], halo_periods: Sequence[bool] = (True, True), backend: str = "auto"):
    """``unpad_halo(halo_accumulate(x))``: fold the pad regions of a painted
    mesh into the owning ranks and return the un-padded field.  On an axis
    whose mesh size is one the fold is done locally (periodic wrap-around)."""
    h0, h1 = int(halo_extents[0]), int(halo_extents[1])
    st, plain = as_sharded(x)
    y = halo_accumulate(st, (h0, h1), halo_periods, backend).local
    nb = y.dim() - 3
    for k, (h, per) in enumerate(((h0, halo_periods[0]), (h1, halo_periods[1]))):
        if h and st.mesh.pdims[k] == 1:
            ax = nb + k
            s = y.shape[ax]
            y = y.clone()
            if per:
                y.narrow(ax, s - 2 * h, h).add_(y.narrow(ax, 0, h))
                y.narrow(ax, h, h).add_(y.narrow(ax, s - h, h))
    y = _unpad_local(y, h0, h1)
    return y if plain else ShardedTensor(y, st.mesh, st.spec)
