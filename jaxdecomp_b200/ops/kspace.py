"""Pointwise Fourier-space operators on the rotated output of ``pfft3d``.

These are the k-space steps of the reference's LPT example
(``examples/lpt_nbody_demo.py:75-133``): colouring a white-noise field with
``sqrt(P(k))`` and forming the displacement potentials ``i k_d / k^2``.  The
operand is a :class:`ShardedTensor` in the layout ``pfft3d`` returns in
contiguous mode: global dims ``(N1, N2, N0)`` hold the original axes
``(1, 2, 0)``.  CUDA complex64 blocks use the native kernels (wave numbers are
generated from global indices inside the kernel); anything else uses PyTorch.
All operators are linear and differentiable.
"""
from __future__ import annotations

import math
from typing import Sequence, Tuple

import torch

from ..parallel.sharding import ShardedTensor, shard_offsets


class _Geo:
    """Light-weight geometry of a rotated k-space block (no reference to the data)."""

    def __init__(self, k: ShardedTensor):
        self.global_shape = k.global_shape
        self.spec = k.spec
        self.mesh = k.mesh
        self.local = torch.empty(k.local.shape, dtype=k.local.dtype, device="meta")
        self.device = k.local.device


def _geometry(k):
    g = k.global_shape[-3:]
    n0, n1, n2 = g[2], g[0], g[1]  # original axes from the rotated layout (N1, N2, N0)
    offs = shard_offsets(k.global_shape, k.spec, k.mesh)[-3:]
    return (n0, n1, n2), offs, tuple(k.local.shape[-3:])


def wave_numbers(k, box: Sequence[float]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Physical wave numbers of the original axes 0, 1, 2, sliced to this rank's
    block and shaped to broadcast against ``k.local``."""
    (n0, n1, n2), offs, ls = _geometry(k)
    dev = k.device if isinstance(k, _Geo) else k.local.device
    dt = torch.float32 if k.local.dtype == torch.complex64 else torch.float64

    def freq(n, L, o, m):
        return (torch.fft.fftfreq(n, d=1.0 / n, dtype=dt, device=dev) * (2 * math.pi / L))[o:o + m]

    k1 = freq(n1, box[1], offs[0], ls[0]).view(-1, 1, 1)
    k2 = freq(n2, box[2], offs[1], ls[1]).view(1, -1, 1)
    k0 = freq(n0, box[0], offs[2], ls[2]).view(1, 1, -1)
    return k0, k1, k2


def _native_ok(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.complex64 and t.dim() == 3


def _launch(mode, k: ShardedTensor, box, prm, x, outs, table=None):
    from .. import native

    nat = native.require()
    (n0, n1, n2), offs, ls = _geometry(k)
    ptr = [o.data_ptr() if o is not None else 0 for o in outs] + [0, 0]
    nat.kspace(mode, list(ls), [int(o) for o in offs], [n0, n1, n2], [float(b) for b in box], [float(p) for p in prm],
               0 if table is None else int(table.numel()), 0 if table is None else table.data_ptr(),
               x.data_ptr(), ptr[0], ptr[1], ptr[2], torch.cuda.current_stream().cuda_stream)


class _Scale(torch.autograd.Function):
    """y = m(k) x with a real multiplier m (modes 0, 1, 3): self-adjoint."""

    @staticmethod
    def forward(ctx, x, kst, box, mode, prm, table):
        ctx.meta = (kst, box, mode, prm, table)
        x = x.contiguous()
        if _native_ok(x):
            out = torch.empty_like(x)
            _launch(mode, kst, box, prm, x, [out], table)
            return out
        k0, k1, k2 = wave_numbers(kst, box)
        kk = k0 ** 2 + k1 ** 2 + k2 ** 2
        if mode == 3:
            m = torch.where(kk > 0, -1.0 / kk.clamp_min(1e-30), torch.zeros_like(kk))
        else:
            kabs = kk.sqrt()
            if mode == 0:
                amp, idx, kcut, norm = prm
                p = amp * kabs.clamp_min(1e-30) ** idx * torch.exp(-(kabs / kcut) ** 2)
            else:
                lk0, dlk, _, norm = prm
                u = ((kabs.clamp_min(1e-30).log() - lk0) / dlk).clamp(0, table.numel() - 1)
                i = u.floor().clamp(0, table.numel() - 2).long()
                t = u - i
                p = table[i] * (1 - t) + table[i + 1] * t
            p = torch.where(kk > 0, p, torch.zeros_like(p))
            m = (p * norm).clamp_min(0).sqrt()
        return x * m

    @staticmethod
    def backward(ctx, g):
        kst, box, mode, prm, table = ctx.meta
        return _Scale.apply(g, kst, box, mode, prm, table), None, None, None, None, None


class _Gradient(torch.autograd.Function):
    """(y0, y1, y2) = (i k_d / k^2) x."""

    @staticmethod
    def forward(ctx, x, kst, box):
        ctx.meta = (kst, box)
        x = x.contiguous()
        if _native_ok(x):
            outs = [torch.empty_like(x) for _ in range(3)]
            _launch(2, kst, box, (0, 0, 0, 0), x, outs)
            return tuple(outs)
        ks = wave_numbers(kst, box)
        kk = ks[0] ** 2 + ks[1] ** 2 + ks[2] ** 2
        inv = torch.where(kk > 0, 1.0 / kk.clamp_min(1e-30), torch.zeros_like(kk))
        return tuple(x * (1j * kd * inv) for kd in ks)

    @staticmethod
    def backward(ctx, g0, g1, g2):
        kst, box = ctx.meta
        return _GradientAdjoint.apply(g0, g1, g2, kst, box), None, None


class _GradientAdjoint(torch.autograd.Function):
    """x = sum_d conj(i k_d / k^2) y_d."""

    @staticmethod
    def forward(ctx, g0, g1, g2, kst, box):
        ctx.meta = (kst, box)
        g0, g1, g2 = g0.contiguous(), g1.contiguous(), g2.contiguous()
        if _native_ok(g0):
            out = torch.empty_like(g0)
            from .. import native

            nat = native.require()
            (n0, n1, n2), offs, ls = _geometry(kst)
            nat.kspace(4, list(ls), [int(o) for o in offs], [n0, n1, n2], [float(b) for b in box], [0.0, 0.0, 0.0, 0.0], 0,
                       0, g0.data_ptr(), out.data_ptr(), g1.data_ptr(), g2.data_ptr(),
                       torch.cuda.current_stream().cuda_stream)
            return out
        ks = wave_numbers(kst, box)
        kk = ks[0] ** 2 + ks[1] ** 2 + ks[2] ** 2
        inv = torch.where(kk > 0, 1.0 / kk.clamp_min(1e-30), torch.zeros_like(kk))
        return sum(g * (-1j * kd * inv) for g, kd in zip((g0, g1, g2), ks))

    @staticmethod
    def backward(ctx, gg):
        kst, box = ctx.meta
        return (*_Gradient.apply(gg, kst, box), None, None)


def _check(k: ShardedTensor):
    if not isinstance(k, ShardedTensor) or not k.local.is_complex():
        raise TypeError("expected the complex ShardedTensor returned by pfft3d")


def apply_power_law(k: ShardedTensor, box: Sequence[float], amplitude: float = 1.0, index: float = -2.0,
                    k_cut: float = 1.0, norm: float = 1.0) -> ShardedTensor:
    """Multiply by ``sqrt(norm * amplitude * |k|^index * exp(-(|k|/k_cut)^2))`` (zero at k = 0)."""
    _check(k)
    y = _Scale.apply(k.local, _Geo(k), tuple(box), 0, (amplitude, index, k_cut, norm), None)
    return ShardedTensor(y, k.mesh, k.spec, k.global_shape)


def apply_power_table(k: ShardedTensor, box: Sequence[float], log_k0: float, dlog_k: float, table: torch.Tensor,
                      norm: float = 1.0) -> ShardedTensor:
    """Multiply by ``sqrt(norm * P(|k|))`` with ``P`` tabulated at ``exp(log_k0 + i*dlog_k)``."""
    _check(k)
    table = table.to(device=k.local.device, dtype=torch.float32).contiguous()
    y = _Scale.apply(k.local, _Geo(k), tuple(box), 1, (log_k0, dlog_k, 0.0, norm), table)
    return ShardedTensor(y, k.mesh, k.spec, k.global_shape)


def inverse_laplacian(k: ShardedTensor, box: Sequence[float]) -> ShardedTensor:
    """Multiply by ``-1/|k|^2`` (zero at k = 0)."""
    _check(k)
    y = _Scale.apply(k.local, _Geo(k), tuple(box), 3, (0.0, 0.0, 0.0, 0.0), None)
    return ShardedTensor(y, k.mesh, k.spec, k.global_shape)


def displacement_potentials(k: ShardedTensor, box: Sequence[float]):
    """Return the three fields ``i k_d / k^2 * delta_k`` (d = original axes 0, 1, 2)."""
    _check(k)
    ys = _Gradient.apply(k.local, _Geo(k), tuple(box))
    return tuple(ShardedTensor(y, k.mesh, k.spec, k.global_shape) for y in ys)


class _InverseDisplacements(torch.autograd.Function):
    """psi_b = scale * IFFT(i k_b / k^2 * delta_k), b = 0, 1, 2, as one batched inverse transform whose first
    pass applies the multiplier while it reads ``delta_k`` (native backend), so the three potentials are
    never written to memory."""

    @staticmethod
    def forward(x, kst, box, mesh, contiguous, scale, pencil_type):
        from . import b200_backend
        from . import plan as _plan

        steps = _plan.fft_steps(pencil_type, True, contiguous, native=True)
        (n0, n1, n2), offs, _ = _geometry(kst)
        return b200_backend.run_steps(x, steps, mesh, True, scale, fused_mul=((n0, n1, n2), offs, box))

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.meta = tuple(inputs[1:])

    @staticmethod
    def backward(ctx, g):
        from .fft import _DistFFT

        kst, box, mesh, contiguous, scale, pencil_type = ctx.meta
        # adjoint: the opposite pipeline on the three cotangents (one batched plan), then sum_b conj(i k_b / k^2)
        gk = _DistFFT.apply(g.contiguous(), mesh, False, contiguous, scale, "b200", pencil_type)
        return _GradientAdjoint.apply(gk[0], gk[1], gk[2], kst, box), None, None, None, None, None, None


def inverse_displacements(k: ShardedTensor, box: Sequence[float], backend: str = "auto") -> ShardedTensor:
    """The three displacement fields in real space, ``pifft3d(i k_d / k^2 * k)`` for the original axes
    d = 0, 1, 2, stacked along a new leading dimension (complex; the imaginary parts vanish for the
    transform of a real field).  Counterpart of the potentials-then-three-inverse-FFTs sequence of the
    reference's example (``examples/lpt_nbody_demo.py:120-135``).  On the native backend this is one batched
    plan with the multiplier fused into its first pass; elsewhere the potentials are formed first and
    transformed as one batch."""
    from ..utils.config import config
    from .dispatch import resolve_backend
    from .fft import _fft_norm, pifft3d

    _check(k)
    b = resolve_backend(backend, k.local)
    mesh = k.mesh
    gshape = k.global_shape[-3:]
    if b == "b200" and k.local.dim() == 3 and bool(config.transpose_axis_contiguous):
        from . import b200_backend
        from . import plan as _plan

        rt = b200_backend.get_runtime(mesh)
        steps = _plan.fft_steps(mesh.pencil_type, True, True, native=True)
        if rt.fused_mul_supported(steps, tuple(k.local.shape), k.local.dtype):
            _plan.check_input_spec(steps, k.spatial_spec, mesh.pdims, mesh.decomp_axis_names)
            _, out_spec = _plan.propagate(steps, tuple(k.local.shape), k.spatial_spec, mesh.pdims, mesh.decomp_axis_names)
            scale = _fft_norm(gshape, True, "backward")
            y = _InverseDisplacements.apply(k.local.contiguous(), _Geo(k), tuple(float(v) for v in box), mesh, True,
                                            scale, mesh.pencil_type)
            return ShardedTensor(y, mesh, (None,) + tuple(out_spec))
    pots = displacement_potentials(k, box)
    stacked = ShardedTensor(torch.stack([p.local for p in pots]), mesh, (None,) + tuple(k.spec))
    return pifft3d(stacked, backend=backend)
