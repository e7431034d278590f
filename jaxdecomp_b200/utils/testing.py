"""Helpers to run a function on several ranks of one machine.

The reference simulates eight devices inside one process with XLA's forced
host devices (``tests/conftest.py:27-33``).  PyTorch has no such mode, so the
equivalent here is eight real processes on the ``gloo`` backend (CPU), or one
process per GPU on ``nccl``.
"""
from __future__ import annotations

import os
import socket
import traceback
from typing import Callable

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, backend: str, fn: Callable, args: tuple, env: dict):
    os.environ.update({k: str(v) for k, v in env.items()})
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    os.environ["LOCAL_RANK"] = str(rank)
    torch.set_num_threads(1)
    kwargs = {}
    if backend == "nccl":
        torch.cuda.set_device(rank)
        kwargs["device_id"] = torch.device("cuda", rank)
    import datetime

    dist.init_process_group(backend=backend, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=float(os.environ.get("JD_TEST_PG_TIMEOUT", "120"))), **kwargs)
    try:
        try:
            fn(rank, world, *args)
        except BaseException:
            # report at once and leave without collective tear-down: the other ranks may be
            # blocked in a collective that this rank will never join
            traceback.print_exc()
            import sys

            sys.stderr.flush()
            if backend == "nccl":
                os._exit(1)
            raise
        if backend == "nccl":
            torch.cuda.synchronize()
            try:
                import jaxdecomp_b200

                jaxdecomp_b200.finalize()
            except Exception:  # noqa: BLE001
                traceback.print_exc()
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def run_ranks(fn: Callable, world: int, *args, backend: str = "gloo", env: dict = None, timeout: float = 600.0) -> None:
    """Run ``fn(rank, world, *args)`` on ``world`` processes; raise if any fails.  The rendezvous port
    is picked by binding to port 0 and releasing it, so another process can take it in between: a run
    that fails because the address is in use is repeated once on a fresh port."""
    try:
        _run_ranks_once(fn, world, args, backend, env, timeout)
    except Exception as e:  # noqa: BLE001
        if "EADDRINUSE" not in str(e) and "address already in use" not in str(e).lower():
            raise
        _run_ranks_once(fn, world, args, backend, env, timeout)


def _run_ranks_once(fn: Callable, world: int, args: tuple, backend: str, env: dict, timeout: float) -> None:
    port = free_port()
    ctx = mp.start_processes(_worker, args=(world, port, backend, fn, args, env or {}), nprocs=world, join=False,
                             start_method="spawn")
    import time

    deadline = time.time() + timeout
    try:
        while not ctx.join(timeout=1.0):
            if time.time() > deadline:
                for p in ctx.processes:
                    if p.is_alive():
                        p.terminate()
                raise TimeoutError(f"run_ranks: ranks still running after {timeout} s")
    except Exception:
        for p in ctx.processes:
            if p.is_alive():
                p.terminate()
        raise
