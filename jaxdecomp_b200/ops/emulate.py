"""Single-process CPU emulation of the native backend on a whole mesh.

All ranks of a ``pdims`` mesh are emulated in one process: each holds its
local block in host memory, and every compiled pass is executed for all ranks
(one after the other) by the CPU implementation of the tile pass in the native
module, which shares its index arithmetic and butterflies with the CUDA
kernel.  Destination pointers of the emulated peers point into the other
ranks' host buffers, so peer addressing, chunk routing and the fused
permutations are exercised exactly as on NVLink -- without a GPU.  Used by the
unit tests; not a product path.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import passes as _passes
from .plan import Step


def _elem_bytes(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def split_blocks(x: torch.Tensor, pdims: Sequence[int], spec_axes=(0, 1)) -> List[torch.Tensor]:
    """Cut a global array into the row-major list of local blocks of an
    X-pencil layout (array axis ``spec_axes[k]`` sharded by mesh axis ``k``)."""
    p0, p1 = pdims
    nb = x.dim() - 3
    out = []
    for i in range(p0):
        for j in range(p1):
            blk = x
            for k, (p, c) in enumerate(((p0, i), (p1, j))):
                ax = nb + spec_axes[k]
                n = blk.shape[ax] // p
                blk = blk.narrow(ax, c * n, n)
            out.append(blk.contiguous())
    return out


def emulate_steps(blocks: List[torch.Tensor], steps: Sequence[Step], pdims: Sequence[int], inverse: bool = False,
                  scale: float = 1.0, pipeline_chunks: int = 0, fused_mul=None, copy_twin: bool = False,
                  stats: Optional[dict] = None) -> List[torch.Tensor]:
    """Run a step list on the blocks of all ranks (row-major rank order) and
    return the per-rank results.

    With ``pipeline_chunks >= 2`` every exchange pass that the native backend
    would pipeline with the local pass after it (:func:`passes.pipeline_cut`)
    is executed the way the pipelined executor does: chunk by chunk, the
    consumer's chunk k right after chunk k of all producers and *before* their
    chunk k+1 exists -- so a consumer chunk that read outside its producers'
    chunk would see zeros and the result would differ.

    ``fused_mul = (n_orig, offsets_per_rank, box)`` runs the first pass with the fused k-space multiplier
    (three batch entries read from the one input block, entry b multiplied by ``i k_b / k^2``).

    ``copy_twin`` runs every copy pass that the GPU would hand to the rotating copy kernels
    (``csrc/copy_fast.cu``) through their host restatement instead of the general pass; ``stats``, when
    given, receives ``{"twin_passes": n}``."""
    from .. import native as _native

    nat = _native.require()
    p0, p1 = int(pdims[0]), int(pdims[1])
    world = p0 * p1
    assert len(blocks) == world
    dtype = blocks[0].dtype
    eb = _elem_bytes(dtype)
    nbatch = 1
    if blocks[0].dim() == 4:
        nbatch = blocks[0].shape[0]
    if fused_mul is not None:
        assert blocks[0].dim() == 3
        nbatch = 3
    compiled = []
    for r in range(world):
        coords = (r // p1, r % p1)
        ps, final_shape = _passes.compile_passes(steps, blocks[r].shape[-3:], pdims, coords)
        compiled.append(ps)
    npass = len(compiled[0])
    last_fft = max((i for i, p in enumerate(compiled[0]) if p.fft), default=-1)
    cur = [b.contiguous() for b in blocks]

    def alloc(i):
        full = ((nbatch,) if (blocks[0].dim() == 4 or fused_mul is not None) else ()) + tuple(compiled[0][i].out_shape)
        return [torch.zeros(full, dtype=dtype) for _ in range(world)]

    def desc(i, r, src, dst_bufs):
        sp = compiled[r][i]
        coords = (r // p1, r % p1)
        d = _passes.fill_desc(nat, sp, eb, inverse, scale if i == last_fft else 1.0, nbatch,
                              remote=sp.npeers > 1, device_tables=False)
        d.use_bulk = 0
        if fused_mul is not None and i == 0:
            n_orig, offs, box = fused_mul
            rot = (1, 2, 0)
            d.set_mul(1, [int(v) for v in n_orig], [int(offs[r][a]) for a in sp.axes], [rot[a] for a in sp.axes],
                      [2.0 * 3.141592653589793 / float(b) for b in box])
            d.is_b = 0
        d.in_ptr = src[r].data_ptr()
        for p in range(sp.npeers):
            if sp.mesh_axis is None:
                dst = r
            elif sp.mesh_axis == 0:
                dst = p * p1 + coords[1]
            else:
                dst = coords[0] * p1 + p
            d.set_out(p, dst_bufs[dst].data_ptr())
        return d

    i = 0
    twin_passes = 0
    while i < npass:
        cut = None
        if pipeline_chunks >= 2 and i + 1 < npass:
            cut = _passes.pipeline_cut(compiled[0][i], compiled[0][i + 1], pipeline_chunks)
        if cut is None:
            nxt = alloc(i)
            for r in range(world):
                d = desc(i, r, cur, nxt)
                if copy_twin and nat.copy_fast_eligible(d):
                    nat.run_copy_fast_host(d)
                    twin_passes += 1
                else:
                    nat.run_pass_host(d)
            cur = nxt
            i += 1
            continue
        prole, crole, K = cut
        mid, nxt = alloc(i), alloc(i + 1)
        pd = [desc(i, r, cur, mid) for r in range(world)]
        cd = [desc(i + 1, r, mid, nxt) for r in range(world)]
        ext = compiled[0][i].ext[prole - 1]
        step = ext // K
        for k in range(K):
            for r in range(world):
                nat.run_pass_host(pd[r].restricted(prole, k * step, step))
            for r in range(world):
                nat.run_pass_host(cd[r].restricted(crole, k * step, step))
        cur = nxt
        i += 2
    if stats is not None:
        stats["twin_passes"] = twin_passes
    return cur
