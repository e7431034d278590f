"""CUDA-graph capture of sequences of distributed ops.

For small grids the cost of a distributed FFT is dominated by kernel launches
and host dispatch (the reference hides this inside one XLA executable).  The
native executor is capturable: it allocates nothing on the host side of a
launch, its cross-rank barriers take their epoch from device memory and
advance it themselves, and results are written into tensors from the graph's
private pool.  ``capture`` records ``fn(*args)`` once and returns a callable
that copies new inputs into the static buffers, replays the graph and returns
the static outputs.

Every rank must capture and replay the same sequence (SPMD).  Run the function
eagerly a few times first -- ``capture`` does -- so that plans exist and the
peer-visible arena has its final size: arena growth is a host-side collective
and cannot happen inside a capture.
"""
from __future__ import annotations

from typing import Callable

import torch

from ..parallel.sharding import ShardedTensor


def _local(a):
    return a.local if isinstance(a, ShardedTensor) else a


class GraphedCallable:
    def __init__(self, fn: Callable, *example_args, warmup: int = 3):
        self.fn = fn
        self.static_in = []
        for a in example_args:
            if isinstance(a, ShardedTensor):
                self.static_in.append(ShardedTensor(a.local.detach().clone(), a.mesh, a.spec, a.global_shape))
            elif isinstance(a, torch.Tensor):
                self.static_in.append(a.detach().clone())
            else:
                self.static_in.append(a)
        self.graph = torch.cuda.CUDAGraph()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(max(1, warmup)):
                fn(*self.static_in)
            torch.cuda.synchronize()
            with torch.cuda.graph(self.graph, stream=stream):
                self.static_out = fn(*self.static_in)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()

    def __call__(self, *args):
        for dst, src in zip(self.static_in, args):
            if isinstance(dst, (ShardedTensor, torch.Tensor)):
                _local(dst).copy_(_local(src))
        self.graph.replay()
        return self.static_out


def capture(fn: Callable, *example_args, warmup: int = 3) -> GraphedCallable:
    """Capture ``fn(*example_args)`` (no autograd) into a CUDA graph; see the module docstring."""
    with torch.no_grad():
        return GraphedCallable(fn, *example_args, warmup=warmup)
