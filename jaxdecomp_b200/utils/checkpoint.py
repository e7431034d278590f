"""Per-rank save / load of sharded fields.

The reference has no checkpoint facility; its LPT example dumps one ``.npy``
per process (``examples/lpt_nbody_demo.py:256-257``).  Here every rank writes
``<name>_<rank>.npy`` plus (rank 0 only) a JSON side-car that records global
shape, process grid, spec, dtype and each rank's offsets, so that a field can
be re-assembled elementwise by any consumer -- including one that loads the
reference's own per-rank dumps, which use the same block layout.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import numpy as np
import torch

from ..parallel.mesh import Mesh
from ..parallel.sharding import ShardedTensor, shard_offsets


def save_sharded(t: ShardedTensor, directory: str, name: str = "field") -> str:
    os.makedirs(directory, exist_ok=True)
    mesh = t.mesh
    arr = t.local.detach().cpu().numpy()
    path = os.path.join(directory, f"{name}_{mesh.rank}.npy")
    np.save(path, arr)
    if mesh.rank == 0:
        meta = {
            "name": name,
            "global_shape": list(t.global_shape),
            "mesh_shape": list(mesh.shape),
            "axis_names": [n for n in mesh.axis_names],
            "pdims": list(mesh.pdims),
            "spec": [s for s in t.spec],
            "dtype": str(t.local.dtype).replace("torch.", ""),
            "world_size": mesh.world_size,
            "offsets": {str(r): list(shard_offsets(t.global_shape, t.spec, mesh, rank=r)) for r in range(mesh.world_size)},
            "local_shape": list(t.local.shape),
        }
        with open(os.path.join(directory, f"{name}.json"), "w") as f:
            json.dump(meta, f, indent=1)
    mesh.barrier()
    return path


def load_sharded(directory: str, mesh: Mesh, name: str = "field", device=None) -> ShardedTensor:
    with open(os.path.join(directory, f"{name}.json")) as f:
        meta = json.load(f)
    if list(mesh.shape) != meta["mesh_shape"]:
        raise ValueError(f"checkpoint was written on mesh {meta['mesh_shape']}, current mesh is {list(mesh.shape)}")
    arr = np.load(os.path.join(directory, f"{name}_{mesh.rank}.npy"))
    local = torch.from_numpy(arr)
    if device is not None:
        local = local.to(device)
    return ShardedTensor(local, mesh, tuple(meta["spec"]), tuple(meta["global_shape"]))


def assemble(directory: str, name: str = "field") -> np.ndarray:
    """Re-assemble the global array from the per-rank files on one process."""
    with open(os.path.join(directory, f"{name}.json")) as f:
        meta = json.load(f)
    out: Optional[np.ndarray] = None
    for r in range(meta["world_size"]):
        blk = np.load(os.path.join(directory, f"{name}_{r}.npy"))
        if out is None:
            out = np.zeros(meta["global_shape"], dtype=blk.dtype)
        offs = meta["offsets"][str(r)]
        idx = tuple(slice(o, o + n) for o, n in zip(offs, blk.shape))
        out[idx] = blk
    return out
