"""Native backend: executes step lists and halo exchanges with the sm_100a
kernels of ``_jdb200``.

One :class:`MeshRuntime` exists per 2-D decomposition mesh.  It owns the native
``Runtime`` (peer-visible arena, plan cache, executor), grows the arena
collectively when a larger problem arrives, and converts device-side status
records into Python exceptions.  Call path of ``pfft3d`` on this backend:

    ops.fft._DistFFT -> run_steps -> (cached) compile_passes/fill_desc ->
    Runtime.execute  -> per pass: [barrier kernel] tile_pass_kernel (peer stores)

The reference reaches its native executor through an XLA FFI call per op
(``src/csrc/jaxdecomp.cc:137-179``), with plans created at lowering time; here
plans are created on first use and looked up by a string key afterwards.
"""
from __future__ import annotations

import atexit
import os
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import native as _native
from ..parallel.mesh import Mesh
from ..utils.config import config
from ..utils.errors import KernelStatusError, PeerAbortedError, PeerTimeoutError, StaleEpochError
from . import passes as _passes
from .plan import Step
from .torch_backend import halo_regions

_runtimes: Dict[tuple, "MeshRuntime"] = {}
# bytes every new arena provides per slot at least (see utils.api.init / reserve_workspace)
_default_slot_bytes = 0
# switches that change how a plan is tiled: part of the plan key
_TUNING_ENV = ("JD_B200_TILE_T", "JD_B200_BULK", "JD_B200_INTRAPAD", "JD_B200_ROWPAD", "JD_B200_FAST",
               "JD_B200_PIPE_MIN_BYTES", "JD_B200_COPY_T", "JD_B200_COPY_CC", "JD_B200_COPY_PAD", "JD_B200_COPY_FAST")


def auto_pipeline_ctas(npeers: int) -> int:
    """Thread-block limit of a pipelined exchange chunk when the configuration leaves it open
    (``pipeline_ctas = -1``).  With two peers half of the pass's traffic stays local and 96 of the 148 SMs
    were the best setting measured; with four and eight peers the exchange is the longer of the two
    overlapped passes and 112 blocks were faster (1024^3 complex64 round trips on 2, 4 and 8 B200s)."""
    return 96 if npeers <= 2 else 112


# exchange passes smaller than this (bytes per rank) are not pipelined: below it the extra launches and
# per-chunk barriers cost more than the overlap gains
_PIPE_MIN_BYTES = 256 << 20


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _aligned(x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous()
    if x.data_ptr() % 16:
        x = x.clone()
    return x


class MeshRuntime:
    def __init__(self, mesh: Mesh):
        self.nat = _native.require()
        self.mesh = mesh
        self.ranks = mesh.submesh_ranks()
        self.world = len(self.ranks)
        self.me = self.ranks.index(mesh.rank)
        self.group = mesh.submesh_group() if self.world > 1 else None
        self.rt = self.nat.Runtime(self.world, self.me)
        self.rt.set_timeout_ms(int(config.wait_timeout_ms))
        self.nat.trace_set_rank(mesh.rank)
        self._shapes: Dict[int, tuple] = {}
        self._pycache: Dict[tuple, tuple] = {}
        self.plan_hits = 0
        self.arena_generation = 0  # how many times the arena was (re)created

    # ---- arena --------------------------------------------------------------------------------
    def ensure_arena(self, slot_bytes: int) -> None:
        """Collective: every rank of the mesh must call this with the same size.

        Growing the arena stops the world (device synchronise, close all peer mappings, host barrier,
        allocate, exchange handles, reopen), so it should happen once: size the workspace up front with
        ``init(workspace_bytes=...)`` or ``reserve_workspace`` when the largest problem is known."""
        if self.rt.has_arena() and self.rt.slot_bytes() >= slot_bytes:
            return
        slot_bytes = max(int(slot_bytes), int(_default_slot_bytes))
        self.arena_generation += 1
        torch.cuda.synchronize()
        if self.world > 1:
            if self.rt.has_arena():
                self.rt.close_peers()
            dist.barrier(group=self.group)
        self.rt.create_arena(int(slot_bytes))
        if self.world > 1:
            blobs: List[bytes] = [b""] * self.world
            dist.all_gather_object(blobs, self.rt.export_handles(), group=self.group)
            self.rt.open_peers(blobs)
            dist.barrier(group=self.group)

    def release(self, collective: bool = True) -> None:
        if not self.rt.has_arena():
            return
        torch.cuda.synchronize()
        met = False
        if self.world > 1 and collective and dist.is_initialized():
            self.rt.close_peers()
            dist.barrier(group=self.group)
            met = True
        # Without the host barrier a peer may still have this rank's blocks mapped and be writing to
        # them: only the imports are closed then, and the exported blocks stay until the process ends.
        self.rt.destroy_arena(met or self.world == 1)

    # ---- status ---------------------------------------------------------------------------------
    def check_status(self, sync: bool = False) -> None:
        if sync:
            torch.cuda.synchronize()
        code, peer, expected, seen, where = self.rt.read_status()
        if code == 0:
            return
        self.rt.clear_status()
        name = self.nat.status_name(code)
        msg = (f"native kernel reported {name} (peer={peer}, expected={expected}, seen={seen}, where={where}) "
               f"on rank {self.mesh.rank}")
        if name == "TIMEOUT_PEER_SIGNAL":
            raise PeerTimeoutError(msg, peer=peer, expected=expected, seen=seen)
        if name == "STALE_EPOCH":
            raise StaleEpochError(msg)
        if name == "PEER_ABORTED":
            raise PeerAbortedError(msg, peer=peer)
        raise KernelStatusError(msg)

    # ---- plans -----------------------------------------------------------------------------------
    def _peer_arena_rank(self, mesh_axis: int, p: int) -> int:
        coords = list(self.mesh.coords)
        coords[self.mesh.ndim - 2 + mesh_axis] = p
        return self.ranks.index(self.mesh.rank_of(coords))

    def build_plan(self, key: str, steps: Sequence[Step], lshape, dtype, inverse: bool, scale: float, nbatch: int,
                   fused_mul=None, peer_out: bool = False):
        """Compile ``steps`` into a native plan.  ``peer_out``: the result tensor is a peer-visible block
        that every rank allocated alike; when the last pass is an exchange it then stores straight into
        the other ranks' result blocks instead of into a workspace slot that is copied out afterwards."""
        nat = self.nat
        eb = torch.empty((), dtype=dtype).element_size()
        coords = self.mesh.coords[-2:]
        specs, final_shape = _passes.compile_passes(steps, lshape, self.mesh.pdims, coords)
        if not specs:
            raise ValueError("empty step list")
        last_fft = max((i for i, s in enumerate(specs) if s.fft), default=-1)
        n = len(specs)
        # From which pass on can everything run in place inside the result tensor?
        tail_plain_from = n
        while tail_plain_from > 0 and specs[tail_plain_from - 1].plain:
            tail_plain_from -= 1
        bytes_per = specs[0].numel * eb * nbatch
        plan_steps = []
        slot_bytes = 0
        cur_kind = nat.BUF_USER_IN
        next_slot = nat.BUF_SLOT_A
        for i, sp in enumerate(specs):
            remote = sp.npeers > 1
            d = _passes.fill_desc(nat, sp, eb, inverse, scale if i == last_fft else 1.0, nbatch, remote, True)
            if fused_mul is not None and i == 0:
                # the first pass reads one block for all three batch entries and multiplies entry b by
                # i k_b / k^2 on the fly; dims of the rotated layout hold the original axes (1, 2, 0)
                n_orig, offs, box = fused_mul
                rot = (1, 2, 0)
                d.set_mul(1, [int(v) for v in n_orig], [int(offs[a]) for a in sp.axes], [rot[a] for a in sp.axes],
                          [2.0 * 3.141592653589793 / float(b) for b in box])
                d.is_b = 0
                d.use_bulk = 0
            st = nat.PlanStep()
            st.in_kind = cur_kind
            last = i == n - 1
            if not remote and (last or i + 1 >= tail_plain_from):
                out_kind = nat.BUF_USER_OUT
            elif remote and last and peer_out:
                out_kind = nat.BUF_PEER_OUT
            else:
                out_kind = next_slot
                next_slot = nat.BUF_SLOT_B if next_slot == nat.BUF_SLOT_A else nat.BUF_SLOT_A
                slot_bytes = max(slot_bytes, bytes_per)
            st.out_kind = out_kind
            if remote:
                st.set_group_ranks([self._peer_arena_rank(sp.mesh_axis, p) for p in range(sp.npeers)])
            else:
                st.set_group_ranks([self.me])
            st.desc = d
            plan_steps.append(st)
            cur_kind = out_kind
        # pipelined transports: overlap every exchange pass with the local pass that consumes it
        min_bytes = int(os.environ.get("JD_B200_PIPE_MIN_BYTES", _PIPE_MIN_BYTES))
        if config.pipelined and config.pipeline_chunks >= 2 and bytes_per >= min_bytes:
            for i in range(n - 1):
                cut = _passes.pipeline_cut(specs[i], specs[i + 1], int(config.pipeline_chunks))
                if cut is None or plan_steps[i].out_kind == nat.BUF_USER_OUT:
                    continue
                plan_steps[i].pipe_role, plan_steps[i + 1].pipe_role, plan_steps[i].pipe_chunks = cut
                limit = int(config.pipeline_ctas)
                plan_steps[i].pipe_grid_limit = limit if limit >= 0 else auto_pipeline_ctas(specs[i].npeers)
        if cur_kind not in (nat.BUF_USER_OUT, nat.BUF_PEER_OUT):
            st = nat.PlanStep()
            st.in_kind = cur_kind
            st.out_kind = nat.BUF_USER_OUT
            st.copy_only = 1
            st.copy_bytes = bytes_per
            plan_steps.append(st)
        pid = self.rt.add_plan(key, plan_steps, slot_bytes)
        return pid, final_shape

    def fused_mul_supported(self, steps: Sequence[Step], lshape, dtype) -> bool:
        """True when the first pass of ``steps`` can carry the fused k-space multiplier: a power-of-two
        transform of complex data (the kernels that read element by element)."""
        eb = torch.empty((), dtype=dtype).element_size()
        if eb not in (8, 16):
            return False
        specs, _ = _passes.compile_passes(steps, lshape, self.mesh.pdims, self.mesh.coords[-2:])
        if not specs or not specs[0].fft:
            return False
        c = specs[0].ext[0]
        return c >= 8 and (c & (c - 1)) == 0

    def run_steps(self, x: torch.Tensor, steps: Sequence[Step], inverse: bool, scale: float,
                  fused_mul=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Execute a step list on a local block.  ``out``: a contiguous tensor of the result's shape and
        dtype to write into (collective: every rank passes one or none).  When it is a peer-visible block
        (``ops/peer.py``) and the last pass is an exchange, the exchange stores straight into the other
        ranks' ``out`` blocks and the copy out of the workspace disappears.
  ``fused_mul = (n_orig, offsets, box)`` makes the result a
        batch of three: entry b is the pipeline applied to ``x * i k_b / k^2`` (``x`` in the rotated layout of
        ``pfft3d``, ``offsets`` the global indices of its first element), with the multiplier applied inside
        the first pass instead of by a kernel of its own."""
        x = _aligned(x)
        nb = x.dim() - 3
        if nb not in (0, 1):
            raise ValueError("expected a 3-D block or a 4-D block with one leading batch dimension")
        if fused_mul is not None and nb:
            raise ValueError("the fused multiplier takes a single 3-D block")
        nbatch = x.shape[0] if nb else (3 if fused_mul is not None else 1)
        if fused_mul is not None:
            nb = 1
            lshape = tuple(x.shape)
        else:
            lshape = tuple(x.shape[nb:])
        env = tuple(os.environ.get(k, "") for k in _TUNING_ENV)
        fkey = None if fused_mul is None else (tuple(fused_mul[0]), tuple(int(o) for o in fused_mul[1]),
                                               tuple(float(b) for b in fused_mul[2]))
        peer_hit = None
        if out is not None and self.world > 1 and os.environ.get("JD_B200_PEER_OUT", "1") != "0":
            from . import peer as _peer

            peer_hit = _peer.lookup(self.mesh, out)
        pykey = (tuple(steps), lshape, x.dtype, bool(inverse), float(scale), nbatch, env, config.snapshot(), fkey,
                 peer_hit is not None)
        hit = self._pycache.get(pykey)
        if hit is None:
            if not _passes._group_steps(steps, self.mesh.pdims):
                # every step is an exchange over a single rank: the identity
                return x.clone() if out is None else out.copy_(x.reshape(out.shape))
            key = "|".join(map(str, pykey + (self.mesh.pdims, self.mesh.coords[-2:])))
            pid = self.rt.find_plan(key)
            if pid < 0:
                pid, final_shape = self.build_plan(key, steps, lshape, x.dtype, inverse, scale, nbatch, fused_mul,
                                                   peer_out=peer_hit is not None)
                self._shapes[pid] = final_shape
            hit = self._pycache[pykey] = (pid, self._shapes[pid], self.rt.plan_slot_bytes(pid))
        else:
            self.plan_hits += 1
        pid, final_shape, need = hit
        if need > 0 or self.world > 1:
            self.ensure_arena(max(need, 1))
        oshape = ((nbatch,) if nb else ()) + tuple(final_shape)
        if out is None:
            out = torch.empty(oshape, dtype=x.dtype, device=x.device)
        elif (tuple(out.shape) != oshape or out.dtype != x.dtype or not out.is_contiguous() or out.data_ptr() % 16
              or out.device != x.device):
            raise ValueError(f"out must be a contiguous, 16-byte aligned {x.dtype} tensor of shape {oshape} on {x.device}")
        elif out.data_ptr() == x.data_ptr():
            raise ValueError("out must not be the operand")
        self.check_status()
        if peer_hit is not None:
            alloc, offset = peer_hit
            self.rt.execute_peer_out(pid, x.data_ptr(), [p + offset for p in alloc.ptrs], _stream())
        else:
            self.rt.execute(pid, x.data_ptr(), out.data_ptr(), _stream())
        return out

    # ---- halos -------------------------------------------------------------------------------------
    def _halo_common(self, x: torch.Tensor, extents, periods):
        nb = x.dim() - 3
        B = x.shape[0] if nb else 1
        S0, S1, S2 = x.shape[nb:]
        h0, h1 = int(extents[0]), int(extents[1])
        p0, p1 = self.mesh.pdims
        if p0 == 1:
            h0 = 0
        if p1 == 1:
            h1 = 0
        if (h0 and S0 < 2 * h0) or (h1 and S1 < 2 * h1):
            raise ValueError(f"padded block {tuple(x.shape)} is smaller than twice the halo extents {(h0, h1)}")
        regions = list(halo_regions(S0, S1, h0, h1))
        offs, acc = [], 0
        for (_, _, send, _recv) in regions:
            offs.append(acc)
            acc += B * (send[0][1] - send[0][0]) * (send[1][1] - send[1][0]) * S2
        return nb, B, (S0, S1, S2), regions, offs, acc

    def _arena_rank(self, rank):
        return -1 if rank is None else self.ranks.index(rank)

    def halo_exchange(self, x: torch.Tensor, extents, periods, inplace: bool = False) -> torch.Tensor:
        if inplace:
            if not x.is_contiguous() or x.data_ptr() % 16:
                raise ValueError("in-place halo exchange needs a contiguous, 16-byte aligned block")
        else:
            x = _aligned(x)
        nb, B, (S0, S1, S2), regions, offs, total = self._halo_common(x, extents, periods)
        if inplace:
            out = x
            if not regions:
                return out
            from . import peer as _peer

            hit = _peer.lookup(self.mesh, x) if os.environ.get("JD_B200_HALO_DIRECT", "1") != "0" else None
            if hit is not None:
                return self._halo_direct(x, hit, (S0, S1, S2), B, regions, periods)
        else:
            out = torch.empty_like(x)
            if not regions:
                out.copy_(x)
                return out
        eb = x.element_size()
        per = (bool(periods[0]), bool(periods[1]))
        pack, unpack = [], []
        for (d0, d1, send, recv), off in zip(regions, offs):
            dst = self.mesh.neighbor(d0, d1, per)
            src = self.mesh.neighbor(-d0, -d1, per)
            pack.append((send[0][0], send[0][1], send[1][0], send[1][1], self._arena_rank(dst), off))
            unpack.append((recv[0][0], recv[0][1], recv[1][0], recv[1][1], self.me if src is not None else -1, off))
        self.ensure_arena(total * eb)
        self.check_status()
        is_f64 = int(x.dtype in (torch.float64, torch.complex128))
        self.rt.halo(pack, unpack, [], S0, S1, S2, B, eb, is_f64, 0, x.data_ptr(), out.data_ptr(), _stream())
        return out

    def _halo_direct(self, x, hit, shape, B, regions, periods):
        """In-place exchange on a peer-visible block: every slab is stored at its final place in the
        neighbour's block (which has the same shape and sits at the same offset of the neighbour's
        allocation), between two barriers."""
        alloc, offset = hit
        S0, S1, S2 = shape
        per = (bool(periods[0]), bool(periods[1]))
        push, zero = [], []
        for (d0, d1, send, recv) in regions:
            dst = self.mesh.neighbor(d0, d1, per)
            src = self.mesh.neighbor(-d0, -d1, per)
            if dst is not None:
                push.append((send[0][0], send[0][1], send[1][0], send[1][1], self._arena_rank(dst), recv[0][0], recv[1][0]))
            if src is None:
                zero.append((recv[0][0], recv[0][1], recv[1][0], recv[1][1], -1, 0))
        self.ensure_arena(1)  # the flags of the barriers live in the arena
        self.check_status()
        blocks = [p + offset for p in alloc.ptrs]
        self.rt.halo_direct(push, zero, S0, S1, S2, B, x.element_size(), blocks, _stream())
        return x

    def halo_accumulate(self, g: torch.Tensor, extents, periods) -> torch.Tensor:
        g = _aligned(g)
        nb, B, (S0, S1, S2), regions, offs, total = self._halo_common(g, extents, periods)
        out = torch.empty_like(g)
        if not regions:
            out.copy_(g)
            return out
        eb = g.element_size()
        per = (bool(periods[0]), bool(periods[1]))
        pack, unpack, zero = [], [], []
        for (d0, d1, send, recv), off in zip(regions, offs):
            back_to = self.mesh.neighbor(-d0, -d1, per)
            comes_from = self.mesh.neighbor(d0, d1, per)
            pack.append((recv[0][0], recv[0][1], recv[1][0], recv[1][1], self._arena_rank(back_to), off))
            zero.append((recv[0][0], recv[0][1], recv[1][0], recv[1][1], -1, off))
            unpack.append((send[0][0], send[0][1], send[1][0], send[1][1],
                           self.me if comes_from is not None else -1, off))
        self.ensure_arena(total * eb)
        self.check_status()
        is_f64 = int(g.dtype in (torch.float64, torch.complex128))
        self.rt.halo(pack, unpack, zero, S0, S1, S2, B, eb, is_f64, 1, g.data_ptr(), out.data_ptr(), _stream())
        return out


def set_default_workspace(slot_bytes: int) -> None:
    global _default_slot_bytes
    _default_slot_bytes = max(0, int(slot_bytes))


def get_runtime(mesh: Mesh) -> MeshRuntime:
    key = (tuple(mesh.submesh_ranks()), mesh.pdims, torch.cuda.current_device())
    rt = _runtimes.get(key)
    if rt is None:
        rt = _runtimes[key] = MeshRuntime(mesh)
    return rt


def run_steps(x: torch.Tensor, steps: Sequence[Step], mesh: Mesh, inverse: bool, scale: float,
              fused_mul=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return get_runtime(mesh).run_steps(x, steps, inverse, scale, fused_mul, out)


def halo_exchange(x, extents, periods, mesh: Mesh, inplace: bool = False) -> torch.Tensor:
    return get_runtime(mesh).halo_exchange(x, extents, periods, inplace=inplace)


def halo_accumulate(g, extents, periods, mesh: Mesh) -> torch.Tensor:
    return get_runtime(mesh).halo_accumulate(g, extents, periods)


def check_status(mesh: Mesh, sync: bool = True) -> None:
    """Raise if any kernel of this mesh's runtime recorded a failure."""
    get_runtime(mesh).check_status(sync=sync)


def launches(mesh: Mesh) -> int:
    """Number of kernels/copies this backend has launched on the mesh so far."""
    return int(get_runtime(mesh).rt.launches())


def finalize(collective: bool = True) -> None:
    """Free every arena and peer-visible block and forget all plans (collective when ranks > 1)."""
    try:
        from . import peer as _peer

        _peer.free_peer_visible(None, collective=collective)
    except Exception:  # noqa: BLE001 - best effort at shutdown
        pass
    for rt in list(_runtimes.values()):
        try:
            rt.release(collective=collective)
        except Exception:  # noqa: BLE001 - best effort at shutdown
            pass
    _runtimes.clear()


@atexit.register
def _at_exit():
    # at interpreter exit the process group may be gone: free without a host barrier
    try:
        from . import peer as _peer

        _peer.free_peer_visible(None, collective=False)
    except Exception:  # noqa: BLE001
        pass
    for rt in list(_runtimes.values()):
        try:
            rt.release(collective=False)
        except Exception:  # noqa: BLE001
            pass
    _runtimes.clear()
