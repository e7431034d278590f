"""Library life cycle, pencil geometry queries and process-grid autotuning.

Parity targets in the reference's native module: ``init``/``finalize``
(``src/csrc/jaxdecomp.cc:35-47``), ``get_pencil_info`` (``jaxdecomp.cc:53-69``),
``get_autotuned_config`` (``jaxdecomp.cc:74-128``) and ``make_config`` =
``GridConfig`` (``jaxdecomp.cc:617-622``).  The reference's README also shows a
``jaxdecomp.autotune(shape=...)`` call that does not exist in its code; here
:func:`autotune` is that convenience entry point.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..parallel.mesh import Mesh, current_mesh
from ..parallel.sharding import PencilInfo, ShardedTensor, pencil_info
from .config import (
    HALO_COMM_P2P,
    TRANSPOSE_COMM_P2P,
    HaloCommBackend,
    TransposeCommBackend,
    config,
)


@dataclass
class GridConfig:
    """Global grid, process grid and transports of a decomposition."""

    gdims: Tuple[int, int, int] = (0, 0, 0)
    pdims: Tuple[int, int] = (1, 1)
    transpose_comm_backend: TransposeCommBackend = TRANSPOSE_COMM_P2P
    halo_comm_backend: HaloCommBackend = HALO_COMM_P2P


def make_config(gdims=(0, 0, 0), pdims=(1, 1), transpose_comm_backend=TRANSPOSE_COMM_P2P,
                halo_comm_backend=HALO_COMM_P2P) -> GridConfig:
    return GridConfig(tuple(gdims), tuple(pdims), TransposeCommBackend(transpose_comm_backend),
                      HaloCommBackend(halo_comm_backend))


_initialised = False
_monitor = None  # parallel.protocol.HealthMonitor started by init(heartbeat=...)


def init(workspace_bytes: Optional[int] = None, heartbeat: Optional[float] = None, heartbeat_max_age: Optional[float] = None) -> None:
    """Load the native core eagerly on machines with a GPU.  Optional: every op
    initialises what it needs on first use.

    ``heartbeat`` (seconds) starts a host-side liveness monitor: every rank publishes a time stamp
    through the process group's store at that period, and :func:`check_peers` raises
    :class:`~jaxdecomp_b200.parallel.protocol.PeerDeadError` for ranks whose last stamp is older than
    ``heartbeat_max_age`` (default: ten periods).  Call :func:`check_peers` between steps, before
    launching kernels that would wait on a peer that is gone; the device-side waits stay bounded
    either way.

    ``workspace_bytes`` pre-sizes the peer-visible workspace: every arena created afterwards holds
    at least that many bytes per exchange buffer (there are two), so that no later, larger problem
    makes it grow -- growth is a stop-the-world collective.  A good value is the size of the largest
    local block that will be transformed (``get_fft_workspace_size`` reports it for a grid)."""
    global _initialised
    if torch.cuda.is_available():
        from .. import native

        native.require()
    if workspace_bytes is not None:
        from ..ops import b200_backend

        b200_backend.set_default_workspace(int(workspace_bytes))
    global _monitor
    if heartbeat is not None and _monitor is None and dist.is_available() and dist.is_initialized() \
            and dist.get_world_size() > 1:
        from ..parallel.protocol import HealthMonitor

        period = float(heartbeat)
        _monitor = HealthMonitor(period=period, max_age=float(heartbeat_max_age or 10 * period))
    _initialised = True


def check_peers() -> None:
    """Raise :class:`~jaxdecomp_b200.parallel.protocol.PeerDeadError` when a rank has stopped publishing its
    heartbeat (see :func:`init`); a no-op without a monitor.  Host-side only: nothing is launched."""
    if _monitor is not None:
        _monitor.check()


def reserve_workspace(mesh, slot_bytes: int) -> None:
    """Create (or grow) the peer-visible workspace of ``mesh`` now, with ``slot_bytes`` per exchange
    buffer.  Collective over the ranks of the mesh's decomposition group; CUDA only."""
    from ..ops import b200_backend

    b200_backend.get_runtime(mesh).ensure_arena(int(slot_bytes))


def finalize() -> None:
    """Free peer-visible memory, FFT tables and cached plans.  Collective when
    more than one rank is in use; safe to call repeatedly.  A later op simply
    re-creates what it needs (this is also the recovery path after a reported
    peer time-out)."""
    global _initialised, _monitor
    if _monitor is not None:
        _monitor.stop()
        _monitor = None
    try:
        from ..ops import b200_backend

        b200_backend.finalize(collective=True)
    except Exception:  # noqa: BLE001
        pass
    try:
        from .. import native

        if native.is_built():
            nat = native.load(build_if_needed=False)
            nat.clear_fft_tables()
            nat.trace_flush()
    except Exception:  # noqa: BLE001
        pass
    _initialised = False


def get_pencil_info(grid_config: GridConfig, axis: int, coords: Optional[Sequence[int]] = None,
                    halo_extents: Sequence[int] = (0, 0, 0)) -> PencilInfo:
    """Geometry (shape, lo, hi, order, halo extents, size) of this rank's pencil
    for ``axis`` in {0: X, 1: Y, 2: Z}.  ``coords`` defaults to this rank's
    coordinates on the active mesh."""
    if coords is None:
        mesh = current_mesh()
        if mesh is not None and tuple(mesh.pdims) == tuple(grid_config.pdims):
            coords = mesh.coords[-2:]
        else:
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
            p1 = int(grid_config.pdims[1])
            coords = ((rank // p1) % int(grid_config.pdims[0]), rank % p1)
    return pencil_info(grid_config.gdims, grid_config.pdims, axis, coords, halo_extents)


def _factorizations(n: int) -> List[Tuple[int, int]]:
    return [(a, n // a) for a in range(1, n + 1) if n % a == 0]


def _time_candidate(shape, pdims, dtype, device, iters: int, backend: str, halo=None) -> float:
    from ..ops.fft import pfft3d, pifft3d
    from ..ops.halo import halo_exchange

    mesh = Mesh(pdims, ("z", "y"))
    p0, p1 = pdims
    lshape = (shape[0] // p0, shape[1] // p1, shape[2])
    x = ShardedTensor(torch.randn(lshape, dtype=dtype, device=device), mesh)

    def step():
        if halo is None:
            return pifft3d(pfft3d(x, backend=backend), backend=backend)
        return halo_exchange(ShardedTensor(x.local.real.contiguous(), mesh), halo[0], halo[1], backend=backend)

    step()
    if device.type == "cuda":
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(iters):
            step()
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / iters
    else:
        import time

        t0 = time.perf_counter()
        for _ in range(iters):
            step()
        ms = (time.perf_counter() - t0) * 1e3 / iters
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def autotune(shape: Sequence[int], dtype: torch.dtype = torch.complex64, device=None, iters: int = 3,
             backend: str = "auto", candidates: Optional[Sequence[Tuple[int, int]]] = None,
             halo: Optional[Tuple[Sequence[int], Sequence[bool]]] = None, return_timings: bool = False):
    """Time every admissible process grid ``(P0, P1)`` with ``P0*P1 == world``
    on a round trip ``pifft3d(pfft3d(x))`` (or on a halo exchange when ``halo``
    is given) and return the fastest, measured as the maximum over ranks.
    Collective: all ranks must call it with the same arguments."""
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    device = torch.device(device)
    n0, n1, n2 = (int(s) for s in shape)
    cands = list(candidates) if candidates is not None else _factorizations(world)
    timings = {}
    for p0, p1 in cands:
        ok = n0 % p0 == 0 and n1 % p1 == 0 and n2 % p1 == 0 and n1 % p0 == 0 and n2 % p0 == 0
        if not ok:
            continue
        timings[(p0, p1)] = _time_candidate((n0, n1, n2), (p0, p1), dtype, device, iters, backend, halo)
    if not timings:
        raise ValueError(f"no process grid of {world} ranks divides the global shape {tuple(shape)}")
    best = min(timings, key=timings.get)
    return (best, timings) if return_timings else best


def get_autotuned_config(grid_config: GridConfig, double_precision: bool = False, disable_nccl_backends: bool = False,
                         disable_nvshmem_backends: bool = True, tune_with_transpose: bool = True,
                         halo_extents: Sequence[int] = (0, 0, 0),
                         halo_periods: Sequence[bool] = (True, True, True)) -> GridConfig:
    """Return a copy of ``grid_config`` with ``pdims`` and both transports
    chosen by measurement: the transposes of an FFT round trip when
    ``tune_with_transpose`` else a halo exchange with the given extents.  The
    signature follows the reference's seven positional arguments.  Candidates
    on a GPU: the peer-store kernels with the pipelined transport, the same
    without pipelining, and (unless ``disable_nccl_backends``) the NCCL
    baseline; every candidate is timed on every admissible process grid and the
    fastest pair wins.  On a CPU only the library collectives exist."""
    dtype = torch.complex128 if double_precision else torch.complex64
    halo = None
    if not tune_with_transpose:
        halo = ((int(halo_extents[0]), int(halo_extents[1])), (bool(halo_periods[0]), bool(halo_periods[1])))
    from .config import HALO_COMM_NCCL, TRANSPOSE_COMM_NCCL, TRANSPOSE_COMM_P2P_PL

    # candidates: (op backend, transpose transport); the peer-store kernels with and without pipelining
    # (only the transposes of an FFT have a pipelined form), then the library collectives
    native_ok = torch.cuda.is_available()
    cands = []
    if native_ok:
        cands.append(("auto", TRANSPOSE_COMM_P2P_PL if tune_with_transpose else TRANSPOSE_COMM_P2P))
        if tune_with_transpose:
            cands.append(("auto", TRANSPOSE_COMM_P2P))
    if not disable_nccl_backends or not cands:
        cands.append(("torch" if native_ok else "auto", TRANSPOSE_COMM_NCCL))
    saved = config.transpose_comm_backend
    best = None
    try:
        for b, transport in cands:
            if b == "auto" and native_ok:
                config.update("transpose_comm_backend", transport)
            pd, timings = autotune(grid_config.gdims, dtype=dtype, backend=b, halo=halo, return_timings=True)
            if best is None or timings[pd] < best[2]:
                best = (pd, transport, timings[pd])
    finally:
        config.update("transpose_comm_backend", saved)
    native = best[1] != TRANSPOSE_COMM_NCCL
    return GridConfig(tuple(grid_config.gdims), tuple(best[0]), best[1], HALO_COMM_P2P if native else HALO_COMM_NCCL)


def _workspace_bytes(gdims, pdims, elem_bytes: int, slots: int) -> int:
    n0, n1, n2 = (int(g) for g in gdims)
    p0, p1 = (int(p) for p in pdims)
    local = (n0 // p0) * (n1 // p1) * n2
    return slots * local * int(elem_bytes)


def get_fft_workspace_size(grid_config: GridConfig, double_precision: bool = False) -> int:
    """Bytes of peer-visible arena a distributed FFT of this grid needs on each rank (two pencil
    buffers; one on a single rank).  Counterpart of the reference's workspace query
    (``src/csrc/jaxdecomp.cc:400-427``); the arena is sized automatically, this is informational."""
    single = tuple(grid_config.pdims) == (1, 1)
    return _workspace_bytes(grid_config.gdims, grid_config.pdims, 16 if double_precision else 8, 1 if single else 2)


def get_transpose_workspace_size(grid_config: GridConfig, elem_bytes: int = 8) -> int:
    """Bytes of arena used by a stand-alone transpose (one pencil buffer)."""
    return _workspace_bytes(grid_config.gdims, grid_config.pdims, elem_bytes, 1)


def get_halo_workspace_size(grid_config: GridConfig, halo_extents: Sequence[int], elem_bytes: int = 4) -> int:
    """Bytes of arena staging used by a halo exchange of the padded X-pencil block."""
    n0, n1, n2 = (int(g) for g in grid_config.gdims)
    p0, p1 = (int(p) for p in grid_config.pdims)
    h0 = int(halo_extents[0]) if p0 > 1 else 0
    h1 = int(halo_extents[1]) if p1 > 1 else 0
    s0, s1 = n0 // p0 + 2 * h0, n1 // p1 + 2 * h1
    return (2 * h0 * s1 + 2 * h1 * s0 - 4 * h0 * h1) * n2 * int(elem_bytes)
