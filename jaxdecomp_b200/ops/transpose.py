"""The six pencil transposes as stand-alone differentiable ops.

Semantics follow ``src/jaxdecomp/transpose.py:7-242`` and the per-shard rules
of ``src/jaxdecomp/_src/jax/transpose.py:76-108``: each transpose is one tiled
all-to-all over a single mesh axis plus (contiguous mode) a local rotation, and
its gradient is the inverse transpose.  Unlike the reference's native backend,
``XtoZ``/``ZtoX`` are available on every backend.  Works for real and complex
element types of 4, 8 and 16 bytes.
"""
from __future__ import annotations

import torch

from ..parallel.sharding import ShardedTensor, as_sharded
from ..utils.config import config
from . import plan as _plan
from .dispatch import resolve_backend


def _run(x, mesh, kind, contiguous, backend, out=None):
    steps = _plan.transpose_steps(kind, contiguous)
    if backend == "b200":
        from . import b200_backend

        return b200_backend.run_steps(x, steps, mesh, False, 1.0, out=out)
    from . import torch_backend

    y = torch_backend.run_steps(x, steps, mesh, False)
    return y if out is None else out.copy_(y)


class _Transpose(torch.autograd.Function):
    @staticmethod
    def forward(x, mesh, kind, contiguous, backend):
        return _run(x, mesh, kind, contiguous, backend)

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.args = tuple(inputs[1:])

    @staticmethod
    def backward(ctx, g):
        mesh, kind, contiguous, backend = ctx.args
        return _Transpose.apply(g.contiguous(), mesh, _plan.INVERSE_KIND[kind], contiguous, backend), None, None, None, None

    @staticmethod
    def jvp(ctx, t, *_):
        mesh, kind, contiguous, backend = ctx.args
        return _Transpose.apply(t.contiguous(), mesh, kind, contiguous, backend)

    @staticmethod
    def vmap(info, in_dims, x, *args):
        from .fft import _vmap_leading

        return _vmap_leading(_Transpose.apply, in_dims, x, args)


def transpose(x, kind: str, backend: str = "auto", out=None):
    """One of the six transposes, ``kind`` in ``x_y, y_z, z_y, y_x, x_z, z_x``.

    ``out`` (a tensor or :class:`ShardedTensor` of the result's local shape and dtype; every rank passes
    one or none) receives the result, as ``out=`` does in ``torch``: no gradient flows through such a
    call.  On the native backend a peer-visible ``out`` (``jd.empty_peer_visible`` / ``jd.empty_sharded``,
    the same view on every rank) lets the exchange store straight into the other ranks' result blocks:
    one barrier before and one after the pass replace the staging slot and the copy out of it.
    """
    st, plain = as_sharded(x)
    mesh = st.mesh
    contiguous = bool(config.transpose_axis_contiguous)
    steps = _plan.transpose_steps(kind, contiguous)
    nb = st.local.dim() - 3
    spec = st.spatial_spec
    names = mesh.decomp_axis_names
    if not plain:
        _plan.check_input_spec(steps, spec, mesh.pdims, names)
    _, out_spec = _plan.propagate(steps, tuple(st.local.shape[nb:]), spec, mesh.pdims, names)
    b = resolve_backend(backend, st.local)
    if out is not None:
        dest = out.local if isinstance(out, ShardedTensor) else out
        if torch.is_grad_enabled() and (st.local.requires_grad or dest.requires_grad):
            raise RuntimeError("transpose(..., out=...) does not support automatic differentiation")
        y = _run(st.local.contiguous(), mesh, kind, contiguous, b, out=dest)
    else:
        y = _Transpose.apply(st.local.contiguous(), mesh, kind, contiguous, b)
    if plain:
        return y
    return ShardedTensor(y, mesh, tuple(st.spec[:nb]) + tuple(out_spec))


def transpose_shard(x: torch.Tensor, kind: str, mesh, backend: str = "auto") -> torch.Tensor:
    """Per-shard transpose on a raw local block, for code that manages its own
    sharding (the counterpart of ``transpose_shard`` used inside a user
    ``shard_map`` in the reference, ``_src/jax/transpose.py:349-366``)."""
    contiguous = bool(config.transpose_axis_contiguous)
    b = resolve_backend(backend, x)
    return _Transpose.apply(x.contiguous(), mesh, kind, contiguous, b)


def transposeXtoY(x, backend: str = "auto", out=None):
    """X-pencil -> Y-pencil: global ``(N0,N1,N2)`` -> ``(N2,N0,N1)`` (contiguous mode)."""
    return transpose(x, "x_y", backend, out)


def transposeYtoZ(x, backend: str = "auto", out=None):
    """Y-pencil -> Z-pencil."""
    return transpose(x, "y_z", backend, out)


def transposeZtoY(x, backend: str = "auto", out=None):
    """Z-pencil -> Y-pencil."""
    return transpose(x, "z_y", backend, out)


def transposeYtoX(x, backend: str = "auto", out=None):
    """Y-pencil -> X-pencil."""
    return transpose(x, "y_x", backend, out)


def transposeXtoZ(x, backend: str = "auto", out=None):
    """X-pencil -> Z-pencil in one exchange over the first mesh axis."""
    return transpose(x, "x_z", backend, out)


def transposeZtoX(x, backend: str = "auto", out=None):
    """Z-pencil -> X-pencil in one exchange over the first mesh axis."""
    return transpose(x, "z_x", backend, out)
