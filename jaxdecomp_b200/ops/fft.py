"""Distributed 3-D FFT: ``pfft3d``, ``pifft3d`` and the wave-number helpers.

Public behaviour follows ``src/jaxdecomp/fft.py:56-211`` and
``src/jaxdecomp/_src/jax/fftfreq.py:28-96`` of the reference:

* complex-to-complex only; real input is promoted to complex;
* in contiguous mode (default) the forward transform of an X-pencil array of
  global shape ``(N0, N1, N2)`` is returned rotated, ``(N1, N2, N0)``, and the
  inverse restores ``(N0, N1, N2)``;
* ``norm`` in {'backward', 'ortho', 'forward'} scales by 1, 1/sqrt(N), 1/N.

The autograd rule uses PyTorch's convention for complex functions (the
cotangent is multiplied by the conjugate transpose), which coincides with the
reference's plain-transpose rule (``_src/jax/fft.py:527-546``) for real inputs
with real losses.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from ..parallel.sharding import ShardedTensor, as_sharded, shard_offsets, validate_spec_matches_mesh
from ..utils.config import config
from . import plan as _plan
from .dispatch import resolve_backend


def _fft_norm(shape, inverse: bool, norm: Optional[str]) -> float:
    """Scale applied on top of the un-normalised transform."""
    n = 1
    for s in shape:
        n *= int(s)
    if norm is None or norm == "backward":
        return 1.0 / n if inverse else 1.0
    if norm == "ortho":
        return 1.0 / math.sqrt(n)
    if norm == "forward":
        return 1.0 if inverse else 1.0 / n
    raise ValueError(f'Invalid norm value {norm}; should be "backward", "ortho" or "forward".')


def _str_to_fft_type(s: str) -> str:
    s = str(s).lower()
    if s in ("fft", "ifft", "rfft", "irfft"):
        return s
    raise ValueError(f"Unrecognized string for FFT type: {s}")


def _run(x: torch.Tensor, mesh, steps, inverse: bool, scale: float, backend: str, contiguous: bool = True) -> torch.Tensor:
    if backend == "b200":
        from . import b200_backend

        return b200_backend.run_steps(x, steps, mesh, inverse, scale)
    from . import torch_backend

    if mesh.pdims[0] * mesh.pdims[1] == 1:
        y = torch_backend.fft_single_device(x, inverse, contiguous)
    else:
        y = torch_backend.run_steps(x, steps, mesh, inverse)
    if scale != 1.0:
        y = y * scale
    return y


def _vmap_leading(fn_apply, in_dims, x, args):
    """Batching rule shared by the ops of this package: move the mapped dimension to the front, fold
    all leading dimensions into the one batch dimension the kernels take, run the op once and unfold
    (the reference's rule moves the batch axis to 0 and recurses, ``_src/jax/fft.py:549-573``)."""
    bd = in_dims[0]
    if bd is None:
        return fn_apply(x, *args), None
    x = x.movedim(bd, 0)
    lead = tuple(x.shape[:-3])
    y = fn_apply(x.reshape((-1,) + tuple(x.shape[-3:])).contiguous(), *args)
    return y.reshape(lead + tuple(y.shape[-3:])), 0


class _DistFFT(torch.autograd.Function):
    """y = scale * (un-normalised forward or inverse pipeline)(x).  Written in the form that
    ``torch.func`` transforms need (``setup_context`` apart from ``forward``, a ``vmap`` rule), so that
    ``vmap``, ``jacfwd`` and ``jacrev`` work through it like ``grad`` does."""

    @staticmethod
    def forward(x, mesh, inverse, contiguous, scale, backend, pencil_type):
        steps = _plan.fft_steps(pencil_type, inverse, contiguous, native=(backend == "b200"))
        return _run(x, mesh, steps, inverse, scale, backend, contiguous)

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.args = tuple(inputs[1:])

    @staticmethod
    def backward(ctx, g):
        mesh, inverse, contiguous, scale, backend, pencil_type = ctx.args
        # conjugate transpose of scale * R * F is scale * F^H * R^T: the opposite
        # pipeline (inverse routing, conjugate kernels) without its 1/N.
        gx = _DistFFT.apply(g.contiguous(), mesh, not inverse, contiguous, scale, backend, pencil_type)
        return gx, None, None, None, None, None, None

    @staticmethod
    def jvp(ctx, t, *_):
        mesh, inverse, contiguous, scale, backend, pencil_type = ctx.args
        return _DistFFT.apply(t.contiguous(), mesh, inverse, contiguous, scale, backend, pencil_type)

    @staticmethod
    def vmap(info, in_dims, x, *args):
        return _vmap_leading(_DistFFT.apply, in_dims, x, args)


def _do_pfft(x, inverse: bool, norm, backend: str):
    st, plain = as_sharded(x)
    mesh = st.mesh
    local = st.local
    nb = local.dim() - 3
    if not local.is_complex():
        local = local.to(torch.complex128 if local.dtype == torch.float64 else torch.complex64)
    contiguous = bool(config.transpose_axis_contiguous)
    pt = mesh.pencil_type
    names = mesh.decomp_axis_names
    spec = st.spatial_spec
    steps = _plan.fft_steps(pt, inverse, contiguous)
    if plain:
        # a plain local block is taken to be in the layout the op expects: an X-pencil for the forward
        # transform, the forward transform's output layout for the inverse
        a0, a1 = names
        spec = (a0 if mesh.pdims[0] > 1 else None, a1 if mesh.pdims[1] > 1 else None, None)
        if inverse:
            fwd = _plan.fft_steps(pt, False, contiguous)
            _, spec = _plan.propagate(fwd, (mesh.pdims[0] * mesh.pdims[1],) * 3, spec, mesh.pdims, names)
    elif not inverse:
        validate_spec_matches_mesh(spec, mesh)
    else:
        _plan.check_input_spec(steps, spec, mesh.pdims, names)
    lshape = tuple(local.shape[nb:])
    out_lshape, out_spec = _plan.propagate(steps, lshape, spec, mesh.pdims, names)
    gshape = st.global_shape[nb:]
    scale = _fft_norm(gshape, inverse, norm)
    b = resolve_backend(backend, local)
    y = _DistFFT.apply(local.contiguous(), mesh, inverse, contiguous, scale, b, pt)
    if plain:
        return y
    full_spec = tuple(st.spec[:nb]) + tuple(out_spec)
    return ShardedTensor(y, mesh, full_spec)


def pfft3d(a, norm: Optional[str] = "backward", backend: str = "auto"):
    """Forward distributed c2c FFT of an X-pencil array.

    ``a`` is a :class:`ShardedTensor` (or the local block as a plain tensor
    under an active mesh).  Returns the transform in the layout documented in
    the module docstring, sharded as given by :func:`get_output_specs`.
    """
    return _do_pfft(a, False, norm, backend)


def pifft3d(a, norm: Optional[str] = "backward", backend: str = "auto"):
    """Inverse of :func:`pfft3d`; restores the X-pencil layout and sharding."""
    return _do_pfft(a, True, norm, backend)


def prfft3d(a, norm="backward", backend="auto"):
    """Real-to-complex distributed FFT.  Not implemented (neither is it in the
    reference, ``src/jaxdecomp/fft.py:127-128``); use :func:`pfft3d`, which
    promotes real input to complex."""
    raise NotImplementedError("real-to-complex distributed FFTs are not implemented; use pfft3d")


def pirfft3d(a, norm="backward", backend="auto"):
    raise NotImplementedError("complex-to-real distributed FFTs are not implemented; use pifft3d")


def _freq_vectors(k, d: float, real_axis1: bool, local: bool):
    if isinstance(k, ShardedTensor):
        gshape = k.global_shape[-3:]
        dtype_src = k.local
    else:
        gshape = tuple(k.shape[-3:])
        dtype_src = k
    if dtype_src.is_complex():
        dtype = torch.float32 if dtype_src.dtype == torch.complex64 else torch.float64
    else:
        dtype = dtype_src.dtype
    dev = dtype_src.device
    two_pi = 2.0 * math.pi
    k0 = torch.fft.fftfreq(gshape[0], d=d, dtype=dtype, device=dev) * two_pi
    if real_axis1:
        k1 = torch.fft.rfftfreq(gshape[1], d=d, dtype=dtype, device=dev) * two_pi
    else:
        k1 = torch.fft.fftfreq(gshape[1], d=d, dtype=dtype, device=dev) * two_pi
    k2 = torch.fft.fftfreq(gshape[2], d=d, dtype=dtype, device=dev) * two_pi
    if local and isinstance(k, ShardedTensor) and not real_axis1:
        offs = shard_offsets(k.global_shape, k.spec, k.mesh)[-3:]
        ls = tuple(k.local.shape[-3:])
        k0 = k0[offs[0]: offs[0] + ls[0]]
        k1 = k1[offs[1]: offs[1] + ls[1]]
        k2 = k2[offs[2]: offs[2] + ls[2]]
    return k2.reshape(1, 1, -1), k0.reshape(-1, 1, 1), k1.reshape(1, -1, 1)


def fftfreq3d(k_array, d: float = 1.0, local: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Angular wave numbers for the output of :func:`pfft3d`.

    Returns three vectors shaped ``[1,1,-1]``, ``[-1,1,1]`` and ``[1,-1,1]``
    built from ``2*pi*fftfreq`` of dimensions 2, 0 and 1 of ``k_array``.  In the
    rotated output layout ``(N1, N2, N0)`` these are the wave numbers of the
    original axes 0, 1 and 2 in that order.  For a :class:`ShardedTensor` the
    vectors are sliced to this rank's block (so they broadcast against
    ``k_array.local``) unless ``local=False``.  float32 for complex64 input,
    float64 for complex128.
    """
    src = k_array.local if isinstance(k_array, ShardedTensor) else k_array
    if not src.is_complex():
        raise AssertionError("fftfreq3d expects the (complex) output of pfft3d")
    return _freq_vectors(k_array, d, False, local)


def rfftfreq3d(k_array, d: float = 1.0, local: bool = False):
    """Like :func:`fftfreq3d` but with ``rfftfreq`` on dimension 1 (the layout a
    real-to-complex transform would produce); kept for API parity."""
    return _freq_vectors(k_array, d, True, local)
