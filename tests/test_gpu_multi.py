"""Native kernels on 2+ GPUs (one process per GPU, NCCL for bootstrap):
every op is compared elementwise with the baseline backend on the same ranks."""
import pytest
import torch

import jaxdecomp_b200 as jd
from jaxdecomp_b200.utils.testing import run_ranks

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _pdims_list(world):
    out = [(1, world), (world, 1)]
    if world >= 4:
        out += [(2, world // 2), (world // 2, 2)]
    return out


def _rel(a, b):
    d = b.abs().max().clamp_min(1e-30)
    return ((a - b).abs().max() / d).item()


def _fft_case(x, mesh, tol, tag):
    """Forward against the baseline backend on the same ranks, inverse back to the input, and the
    pipelined transport bit-identical to the plain one."""
    k_ref = jd.pfft3d(x, backend="torch")
    jd.config.update("transpose_comm_backend", jd.TRANSPOSE_COMM_P2P)
    k0 = jd.pfft3d(x, backend="b200")
    b0 = jd.pifft3d(k0, backend="b200")
    jd.config.update("transpose_comm_backend", jd.TRANSPOSE_COMM_P2P_PL)
    k = jd.pfft3d(x, backend="b200")
    b = jd.pifft3d(k, backend="b200")
    assert tuple(k.spec) == tuple(k_ref.spec) and k.local.shape == k_ref.local.shape, tag
    assert _rel(k.local, k_ref.local) < tol, tag
    assert _rel(b.local, x.local) < 10 * tol, tag
    assert torch.equal(k.local, k0.local) and torch.equal(b.local, b0.local), tag


def _transposes_case(x, mesh, pencil):
    y = jd.transposeXtoY(x, backend="b200")
    assert torch.equal(y.local, jd.transposeXtoY(x, backend="torch").local)
    z = jd.transposeYtoZ(y, backend="b200")
    assert torch.equal(z.local, jd.transposeYtoZ(y, backend="torch").local)
    y2 = jd.transposeZtoY(z, backend="b200")
    assert torch.equal(y2.local, y.local)
    assert torch.equal(jd.transposeYtoX(y2, backend="b200").local, x.local)
    if pencil:
        zz = jd.transposeXtoZ(x, backend="b200")
        assert torch.equal(zz.local, jd.transposeXtoZ(x, backend="torch").local)
        assert torch.equal(jd.transposeZtoX(zz, backend="b200").local, x.local)


def _peer_out_transposes(x, mesh, pencil):
    """``out=`` on a peer-visible block: the exchange stores straight into the other ranks' results (a
    barrier, the pass, a barrier: no staging slot, no copy out of it); an ordinary ``out`` is filled too."""
    from jaxdecomp_b200.ops import b200_backend

    rt = b200_backend.get_runtime(mesh)
    kinds = ["XtoY", "YtoZ", "ZtoY", "YtoX"] + (["XtoZ", "ZtoX"] if pencil else [])
    cur = {"X": x}
    for kind in kinds:
        src_p, dst_p = kind[0], kind[-1]
        fn = getattr(jd, "transpose" + kind)
        src = cur[src_p]
        want = fn(src, backend="torch")
        pv = jd.empty_sharded(mesh, tuple(want.local.shape), want.local.dtype, spec=want.spec)
        pv.local.fill_(-1)
        before = rt.rt.launches()
        got = fn(src, backend="b200", out=pv)
        n = rt.rt.launches() - before
        assert got.local.data_ptr() == pv.local.data_ptr() and tuple(got.spec) == tuple(want.spec), kind
        assert torch.equal(pv.local, want.local), kind
        exchanged = mesh.pdims[0 if kind in ("YtoZ", "ZtoY", "XtoZ", "ZtoX") else 1] > 1
        assert n <= (3 if exchanged else 1), (kind, n)
        plain_out = torch.full_like(want.local, -1)
        fn(src, backend="b200", out=plain_out)
        assert torch.equal(plain_out, want.local), kind
        cur[dst_p] = want
        jd.free_peer_visible(mesh)


def _ops_worker(rank, world):
    from jaxdecomp_b200.ops import b200_backend

    dev = torch.device("cuda", rank)
    for pdims in _pdims_list(world):
        mesh = jd.make_mesh(pdims, ("z", "y"))
        p0, p1 = pdims
        rt = b200_backend.get_runtime(mesh)
        # one arena for everything this mesh will run (the largest block below is 256x512x1024 complex64)
        jd.reserve_workspace(mesh, 256 * 512 * 1024 * 8 // world)
        grew = rt.arena_generation
        for contiguous in (True, False):
            jd.config.update("transpose_axis_contiguous", contiguous)
            cases = [(torch.complex64, (64, 32, 128), 3e-6), (torch.complex128, (24, 40, 56), 1e-12)]
            if contiguous:
                # the sizes of the headline run: 1024-point rows, the large tiles of the exchange pass
                cases = [(torch.complex64, (256, 512, 1024), 3e-6), (torch.complex128, (128, 256, 512), 1e-12),
                         (torch.complex64, (96, 192, 160), 3e-6)] + cases
            for dtype, shape, tol in cases:
                g = torch.Generator(device=dev).manual_seed(1234)
                real = torch.float32 if dtype == torch.complex64 else torch.float64
                xg = torch.complex(torch.randn(shape, generator=g, device=dev, dtype=real),
                                   torch.randn(shape, generator=g, device=dev, dtype=real))
                x = jd.shard(xg, mesh)
                del xg
                _fft_case(x, mesh, tol, (pdims, contiguous, dtype, shape))
                if contiguous and shape[2] == 1024:
                    _transposes_case(x, mesh, p0 > 1 and p1 > 1)
                    _peer_out_transposes(x, mesh, p0 > 1 and p1 > 1)
                del x
            # transposes, exact
            for dtype in (torch.float32, torch.complex128):
                xg = torch.randn((16, 32, 64), generator=torch.Generator().manual_seed(7), dtype=torch.float64).to(dtype)
                _transposes_case(jd.shard(xg.to(dev), mesh), mesh, p0 > 1 and p1 > 1)
                if dtype == torch.float32:
                    _peer_out_transposes(jd.shard(xg.to(dev), mesh), mesh, p0 > 1 and p1 > 1)
        jd.config.update("transpose_axis_contiguous", True)
        assert rt.rt.pipelined_sections() > 0
        assert rt.arena_generation == grew, "the reserved workspace should have covered every case"
        # halos: copy and accumulate, periodic and not
        for periods in ((True, True), (False, True)):
            for dtype in (torch.float32, torch.float64):
                blk = torch.randn((12, 14, 10), generator=torch.Generator().manual_seed(50 + rank), dtype=dtype).to(dev)
                st = jd.ShardedTensor(blk, mesh)
                a = jd.halo_exchange(st, (2, 3), periods, backend="b200")
                b = jd.halo_exchange(st, (2, 3), periods, backend="torch")
                assert torch.equal(a.local, b.local), (pdims, periods)
                c = jd.halo_exchange_(jd.ShardedTensor(blk.clone(), mesh), (2, 3), periods, backend="b200")
                assert torch.equal(c.local, b.local), (pdims, periods)
                # peer-visible block: slabs are stored straight into the neighbours' padded blocks
                pv = jd.empty_sharded(mesh, (2, 12, 14, 10), dtype, spec=(None, "z", "y", None))
                want = []
                for i in range(2):
                    pv.local[i].copy_(blk * (i + 1))
                    want.append(jd.halo_exchange(jd.ShardedTensor(blk * (i + 1), mesh), (2, 3), periods, backend="torch").local)
                rtm = b200_backend.get_runtime(mesh)
                before = rtm.rt.launches()
                jd.halo_exchange_(pv, (2, 3), periods, backend="b200")
                assert torch.equal(pv.local, torch.stack(want)), (pdims, periods)
                # two barriers and one push (plus one zero fill at a non-periodic edge): no staging, no unpack
                assert rtm.rt.launches() - before <= 4
                view = jd.ShardedTensor(pv.local[1], mesh)                # a slice of the block works too
                view.local.copy_(blk)
                jd.halo_exchange_(view, (2, 3), periods, backend="b200")
                assert torch.equal(view.local, c.local), (pdims, periods)
                jd.free_peer_visible(mesh)
                a = jd.halo_accumulate(st, (2, 3), periods, backend="b200")
                b = jd.halo_accumulate(st, (2, 3), periods, backend="torch")
                torch.testing.assert_close(a.local, b.local, rtol=1e-6, atol=1e-6)
        # gradient through the native path
        xl = torch.randn((64 // p0, 32 // p1, 16), device=dev, requires_grad=True)
        k = jd.pfft3d(jd.ShardedTensor(xl, mesh), backend="b200")
        (k.local.abs() ** 2 * (rank + 1)).sum().backward()
        xr = xl.detach().clone().requires_grad_(True)
        kr = jd.pfft3d(jd.ShardedTensor(xr, mesh), backend="torch")
        (kr.local.abs() ** 2 * (rank + 1)).sum().backward()
        assert _rel(xl.grad, xr.grad) < 1e-5
        b200_backend.check_status(mesh, sync=True)
        jd.finalize()


_ENV = {"NCCL_NVLS_ENABLE": "0", "JD_B200_PIPE_MIN_BYTES": "0"}


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_native_ops_match_baseline_on_all_gpus():
    world = 1
    while world * 2 <= min(_ngpu(), 8):
        world *= 2
    run_ranks(_ops_worker, world, backend="nccl", env=_ENV, timeout=900)


def _lpt_worker(rank, world):
    from jaxdecomp_b200.models.lpt import LPTConfig, LPTModel, lpt_loss

    dev = torch.device("cuda", rank)
    for pdims in _pdims_list(world)[:2] + _pdims_list(world)[2:3]:
        mesh = jd.make_mesh(pdims, ("z", "y"))
        noise_g = torch.randn((32, 32, 32), generator=torch.Generator().manual_seed(0))
        res = {}
        for backend in ("b200", "torch"):
            cfg = LPTConfig(nc=32, box_size=32.0, halo=4, amplitude=0.05, backend=backend)
            noise = jd.shard(noise_g.to(dev), mesh)
            noise.local.requires_grad_(True)
            model = LPTModel(mesh, cfg)
            loss = lpt_loss(model, noise)
            loss.backward()
            res[backend] = (float(loss), noise.local.grad.clone(), model(noise).local.detach())
        assert abs(res["b200"][0] - res["torch"][0]) < 1e-4 * abs(res["torch"][0])
        assert _rel(res["b200"][2], res["torch"][2]) < 1e-3
        assert _rel(res["b200"][1], res["torch"][1]) < 5e-3
        jd.finalize()


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_lpt_step_native_vs_baseline_multi_gpu():
    world = 1
    while world * 2 <= min(_ngpu(), 8):
        world *= 2
    run_ranks(_lpt_worker, world, backend="nccl", env={"NCCL_NVLS_ENABLE": "0"}, timeout=600)


def _graph_worker(rank, world):
    from jaxdecomp_b200.utils.graphs import capture

    dev = torch.device("cuda", rank)
    mesh = jd.make_mesh((1, world), ("z", "y"))
    x = jd.ShardedTensor(torch.randn((32, 64 // world, 128), device=dev, dtype=torch.complex64), mesh)
    g = capture(lambda v: jd.pifft3d(jd.pfft3d(v, backend="b200"), backend="b200"), x)
    for seed in (1, 2, 3):
        y = jd.ShardedTensor(torch.randn(x.local.shape, device=dev, dtype=torch.complex64,
                                         generator=torch.Generator(device=dev).manual_seed(seed + rank)), mesh)
        out = g(y)
        torch.cuda.synchronize()
        assert _rel(out.local, y.local) < 3e-5
    from jaxdecomp_b200.ops import b200_backend

    b200_backend.check_status(mesh, sync=True)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_cuda_graph_replay_across_ranks():
    run_ranks(_graph_worker, 2, backend="nccl", env={"NCCL_NVLS_ENABLE": "0"}, timeout=300)


def _autotune_worker(rank, world):
    best, timings = jd.autotune((64, 64, 64), dtype=torch.complex64, iters=2, return_timings=True)
    assert best in timings and all(t > 0 for t in timings.values())
    cfg = jd.get_autotuned_config(jd.make_config((64, 64, 64), (1, world)), False, True, True, False, (2, 2, 0),
                                  (True, True, True))
    assert cfg.pdims in timings
    # complex halos on the native path
    mesh = jd.make_mesh((1, world), ("z", "y"))
    blk = torch.randn((8, 12, 6), device=torch.device("cuda", rank), dtype=torch.complex128)
    st = jd.ShardedTensor(blk, mesh)
    assert torch.equal(jd.halo_exchange(st, (0, 2), (True, True), backend="b200").local,
                       jd.halo_exchange(st, (0, 2), (True, True), backend="torch").local)
    torch.testing.assert_close(jd.halo_accumulate(st, (0, 2), (True, False), backend="b200").local,
                               jd.halo_accumulate(st, (0, 2), (True, False), backend="torch").local)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_autotune_and_complex_halos_on_gpus():
    run_ranks(_autotune_worker, 2, backend="nccl", env={"NCCL_NVLS_ENABLE": "0"}, timeout=300)


def _barrier_worker(rank, world):
    from jaxdecomp_b200.ops import b200_backend

    mesh = jd.make_mesh((1, world), ("z", "y"))
    rt = b200_backend.get_runtime(mesh)
    rt.ensure_arena(1 << 20)
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(50):
        rt.rt.barrier(stream)
    torch.cuda.synchronize()
    rt.check_status()
    assert rt.rt.barriers_issued() == 50


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_signal_barrier_many_rounds():
    run_ranks(_barrier_worker, 2, backend="nccl", env={"NCCL_NVLS_ENABLE": "0"}, timeout=300)


def _abort_worker(rank, world):
    """A barrier that one rank joins late (host-side delay, 100 ms budget): the waiting rank records a
    time-out and marks the whole group as aborted, the late rank learns of it in its own barrier, later
    passes return at entry instead of computing on incomplete data, and finalize() + a fresh arena
    bring the mesh back."""
    import time

    from jaxdecomp_b200.ops import b200_backend
    from jaxdecomp_b200.utils.errors import PeerAbortedError, PeerTimeoutError

    dev = torch.device("cuda", rank)
    mesh = jd.make_mesh((1, world), ("z", "y"))
    rt = b200_backend.get_runtime(mesh)
    rt.ensure_arena(1 << 22)
    x = jd.ShardedTensor(torch.randn((32, 64 // world, 128), device=dev, dtype=torch.complex64), mesh)
    good = jd.pfft3d(x, backend="b200").local.clone()
    torch.cuda.synchronize()
    rt.rt.set_timeout_ms(100)
    stream = torch.cuda.current_stream().cuda_stream
    torch.distributed.barrier()
    if rank == 1:
        time.sleep(1.0)  # joins the barrier long after the other rank's budget has run out
    rt.rt.barrier(stream)
    torch.cuda.synchronize()
    torch.distributed.barrier()
    assert rt.rt.peek_flag(rt.nat.FLAG_ABORT_WORD) == 1  # set by rank 0 on every rank
    with pytest.raises(PeerTimeoutError if rank == 0 else PeerAbortedError):
        rt.check_status()
    # kernels launched now return at entry; nothing waits, nothing faults, the context stays usable
    before = rt.rt.launches()
    jd.pfft3d(x, backend="b200")
    torch.cuda.synchronize()
    assert rt.rt.launches() > before
    try:
        rt.check_status()
    except (PeerTimeoutError, PeerAbortedError):
        pass
    jd.finalize()  # collective: frees the aborted arena
    again = jd.pfft3d(x, backend="b200").local
    assert torch.equal(again, good)
    b200_backend.check_status(mesh, sync=True)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least two GPUs")
def test_late_rank_aborts_the_group_and_finalize_recovers():
    run_ranks(_abort_worker, 2, backend="nccl", env={"NCCL_NVLS_ENABLE": "0"}, timeout=300)


def _nested_worker(rank, world):
    """Native backend on a 3-D mesh: the leading mesh axis splits a batch into independent groups of
    2x2 GPUs, each op also carries a local batch dimension; everything against the baseline backend."""
    from jaxdecomp_b200.ops import b200_backend

    dev = torch.device("cuda", rank)
    mesh = jd.Mesh((world // 4, 2, 2), ("c", "z", "y"))
    grp = mesh.coords[0]
    g = torch.Generator(device=dev).manual_seed(100 + grp)
    xg = torch.complex(torch.randn((3, 64, 128, 256), generator=g, device=dev),
                       torch.randn((3, 64, 128, 256), generator=g, device=dev))
    x = jd.shard(xg, mesh, (None, "z", "y", None))
    k = jd.pfft3d(x, backend="b200")
    kr = jd.pfft3d(x, backend="torch")
    assert tuple(k.spec) == tuple(kr.spec) and _rel(k.local, kr.local) < 3e-6
    assert _rel(jd.pifft3d(k, backend="b200").local, x.local) < 3e-5
    y = jd.transposeXtoY(x, backend="b200")
    assert torch.equal(y.local, jd.transposeXtoY(x, backend="torch").local)
    z = jd.transposeYtoZ(y, backend="b200")
    assert torch.equal(z.local, jd.transposeYtoZ(y, backend="torch").local)
    assert torch.equal(jd.transposeYtoX(jd.transposeZtoY(z, backend="b200"), backend="b200").local, x.local)
    blk = jd.ShardedTensor(x.local.real.contiguous(), mesh, x.spec)
    assert torch.equal(jd.halo_exchange(blk, (2, 2), (True, False), backend="b200").local,
                       jd.halo_exchange(blk, (2, 2), (True, False), backend="torch").local)
    torch.testing.assert_close(jd.halo_accumulate(blk, (2, 2), (True, True), backend="b200").local,
                               jd.halo_accumulate(blk, (2, 2), (True, True), backend="torch").local)
    with mesh:
        kv = torch.func.vmap(lambda v: jd.pfft3d(v, backend="b200"))(x.local)
    assert torch.equal(kv, k.local)
    b200_backend.check_status(mesh, sync=True)


@pytest.mark.skipif(_ngpu() < 4, reason="needs at least four GPUs")
def test_native_backend_on_nested_mesh():
    world = 8 if _ngpu() >= 8 else 4
    run_ranks(_nested_worker, world, backend="nccl", env=_ENV, timeout=600)
