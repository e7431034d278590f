"""Host-level collectives used by the baseline backend, the tests and the
benchmarks: tiled all-to-all over a mesh axis, a differentiable all-reduce and
a gather of a sharded array onto every rank.

``all_to_all_tiled`` reproduces ``lax.all_to_all(x, axis_name, split_axis,
concat_axis, tiled=True)`` as used throughout the reference's JAX backend
(``src/jaxdecomp/_src/jax/transpose.py:76-108``): over a sub-group of size P,
rank r cuts its block into P equal chunks along ``split_axis``, sends chunk j
to rank j and concatenates what it receives along ``concat_axis`` in source
order.  Only ``all_to_all_single`` is used because the gloo backend has no
list-form all-to-all.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def all_to_all_tiled(x: torch.Tensor, group, group_size: int, split_axis: int, concat_axis: int) -> torch.Tensor:
    """``split_axis``/``concat_axis`` count from the end when negative; callers
    pass spatial axes offset by the number of leading batch dimensions."""
    if group_size == 1:
        return x
    nd = x.dim()
    split_axis %= nd
    concat_axis %= nd
    n = x.shape[split_axis]
    if n % group_size:
        raise ValueError(f"axis {split_axis} of extent {n} cannot be split over {group_size} ranks")
    send = x.unflatten(split_axis, (group_size, n // group_size)).movedim(split_axis, 0).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[j] is the chunk that rank j sent; lay the source index just before concat_axis
    out = recv.movedim(0, concat_axis)
    return out.flatten(concat_axis, concat_axis + 1)


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        # every rank holds the same total, and every rank's loss uses it: the
        # cotangents are summed over ranks before flowing back.
        g = g.clone()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g / dist.get_world_size(ctx.group), None


def all_reduce_sum(x: torch.Tensor, group=None) -> torch.Tensor:
    """Sum over ranks, differentiable.  The backward assumes the usual SPMD
    convention that all ranks compute the same scalar loss from the result,
    so that d(loss)/d(local term) equals the upstream gradient."""
    if not (dist.is_available() and dist.is_initialized()):
        return x
    return _AllReduceSum.apply(x, group)


def gather_global(st) -> torch.Tensor:
    """Return the full global array of a ShardedTensor on every rank."""
    mesh = st.mesh
    if mesh.world_size == 1:
        return st.local
    group = mesh.submesh_group()
    ranks = mesh.submesh_ranks()
    local = st.local.contiguous()
    bufs = [torch.empty_like(local) for _ in ranks]
    dist.all_gather(bufs, local, group=group)
    from ..parallel.sharding import shard_offsets

    out = torch.empty(st.global_shape, dtype=local.dtype, device=local.device)
    for r, b in zip(ranks, bufs):
        offs = shard_offsets(st.global_shape, st.spec, mesh, rank=r)
        idx = tuple(slice(o, o + n) for o, n in zip(offs, b.shape))
        out[idx] = b
    return out
