"""First-order Lagrangian perturbation theory (Zel'dovich) particle-mesh step.

The application the reference ships as its flagship example
(``examples/lpt_nbody_demo.py:94-229``): a white-noise field is coloured with a
power spectrum in Fourier space, the displacement field ``psi = i k / k^2 *
delta_k`` is brought back to real space with three inverse distributed FFTs,
particles starting on the lattice are displaced and painted onto a padded
local mesh with cloud-in-cell weights, and the mass that fell into the pads is
folded into the neighbouring ranks.  Every step is differentiable, so
``sum(density**2).backward()`` yields the gradient with respect to the noise.

Differences from the example: the fold uses :func:`halo_reduce` (the exact
adjoint of the halo exchange) instead of a half-width exchange followed by
hand-written adds, and the power spectrum is either the analytic
``A k^n exp(-(k/k_cut)^2)`` or a table, instead of a cosmology package.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..ops import kspace
from ..ops.cic import cic_paint
from ..ops.fft import pfft3d, pifft3d
from ..ops.halo import halo_reduce
from ..parallel.mesh import Mesh
from ..parallel.sharding import ShardedTensor


@dataclass
class LPTConfig:
    nc: int = 64                      # grid points (and particles) per side
    box_size: float = 64.0            # physical box length
    halo: int = 8                     # pad width (cells) of the painting mesh on the two sharded axes
    growth: float = 1.0               # linear growth factor applied to the displacement
    amplitude: float = 1.0            # P(k) = amplitude * k^index * exp(-(k/k_cut)^2)
    index: float = -2.0
    k_cut: Optional[float] = None     # defaults to the Nyquist wave number
    backend: str = "auto"


class LPTModel(torch.nn.Module):
    """``forward(noise)`` maps a real white-noise field (X-pencil ShardedTensor of
    global shape ``(nc, nc, nc)``) to the painted density field (same layout)."""

    def __init__(self, mesh: Mesh, config: LPTConfig, power_table: Optional[Tuple[float, float, torch.Tensor]] = None):
        super().__init__()
        self.mesh = mesh
        self.cfg = config
        self.power_table = power_table
        nc = config.nc
        p0, p1 = mesh.pdims
        if nc % p0 or nc % p1:
            raise ValueError(f"nc={nc} is not divisible by the process grid {mesh.pdims}")

    @property
    def box(self):
        return (self.cfg.box_size,) * 3

    def displacement(self, noise: ShardedTensor):
        """Return (delta_k, psi) with psi the three displacement fields in cell units, real, X-pencil,
        stacked along a leading dimension."""
        cfg = self.cfg
        nc = cfg.nc
        delta_k = pfft3d(noise, backend=cfg.backend)
        k_nyq = math.pi * nc / cfg.box_size
        norm = (nc / cfg.box_size) ** 3
        if self.power_table is not None:
            lk0, dlk, tab = self.power_table
            delta_k = kspace.apply_power_table(delta_k, self.box, lk0, dlk, tab, norm)
        else:
            delta_k = kspace.apply_power_law(delta_k, self.box, cfg.amplitude, cfg.index,
                                             cfg.k_cut if cfg.k_cut is not None else k_nyq, norm)
        # one batched inverse transform for the three components (multiplier fused into its first pass on
        # the native backend); the result stays planar, [3, l0, l1, l2], which is what the painter reads
        cells = nc / cfg.box_size * cfg.growth
        psi = kspace.inverse_displacements(delta_k, self.box, backend=cfg.backend).local.real * cells
        return delta_k, psi

    def paint(self, psi) -> ShardedTensor:
        """Displace lattice particles by ``psi`` (``[3, l0, l1, l2]`` or three blocks) and paint them;
        returns the density (X-pencil)."""
        cfg = self.cfg
        hs = cfg.halo
        p0, p1 = self.mesh.pdims
        h0 = hs if p0 > 1 else 0
        h1 = hs if p1 > 1 else 0
        if not isinstance(psi, torch.Tensor):
            psi = torch.stack(list(psi))
        l0, l1, l2 = psi.shape[1:]
        padded = cic_paint(psi.contiguous(), (l0 + 2 * h0, l1 + 2 * h1, l2), wrap=(p0 == 1, p1 == 1, True),
                           lattice=(l0, l1, l2), origin=(float(h0), float(h1), 0.0), planar=True)
        st = ShardedTensor(padded, self.mesh)
        return halo_reduce(st, (h0, h1), (True, True), backend=cfg.backend)

    def forward(self, noise: ShardedTensor, return_initial_conditions: bool = False):
        delta_k, psi = self.displacement(noise)
        density = self.paint(psi)
        if return_initial_conditions:
            ic = pifft3d(delta_k, backend=self.cfg.backend)
            return ShardedTensor(ic.local.real, self.mesh, noise.spec, noise.global_shape), density
        return density


def lpt_loss(model: LPTModel, noise: ShardedTensor) -> torch.Tensor:
    """``sum(density**2)`` over the global grid (every rank returns the same value)."""
    density = model(noise)
    return ShardedTensor(density.local ** 2, density.mesh, density.spec, density.global_shape).global_sum()
