"""Python face of the native trace log and step profiler.

``JD_PERFO_STEP=TIMER|CUDA|NVTX`` (read when the native module is first used)
or :func:`set_mode` turns on per-step records around every pass, copy and
barrier that the native executor launches; :func:`report` returns them and
:func:`to_csv` / :func:`to_markdown` format them, like the reference's
``Perfostep`` (``src/csrc/include/perfostep.hpp:302-352``).  ``JD_TRACE=1`` and
friends control the per-rank trace log (``src/csrc/include/logger.hpp:53-99``).
"""
from __future__ import annotations

import contextlib
from typing import List, Tuple

import torch

from .. import native

MODES = {"OFF": 0, "TIMER": 1, "CUDA": 2, "NVTX": 3}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else 0


def set_mode(mode: str) -> None:
    native.require().profiler_set_mode(MODES[mode.upper()])


def get_mode() -> str:
    m = native.require().profiler_mode()
    return {v: k for k, v in MODES.items()}[m]


@contextlib.contextmanager
def step(name: str):
    """Time (or NVTX-annotate) a region of user code under the active mode."""
    nat = native.require()
    nat.profiler_start(name, _stream())
    try:
        yield
    finally:
        nat.profiler_stop(_stream())


def report() -> List[Tuple[str, int, float]]:
    """List of ``(step name, count, total milliseconds)``."""
    return list(native.require().profiler_report())


def to_csv() -> str:
    return native.require().profiler_csv()


def to_markdown() -> str:
    return native.require().profiler_markdown()


def reset() -> None:
    native.require().profiler_reset()


def trace(logger: str, message: str, verbose: bool = False) -> None:
    """Write a record to the native trace log (no-op unless ``JD_TRACE`` enables it)."""
    native.require().trace_write(logger, 1 if verbose else 0, message)


def trace_flush() -> None:
    native.require().trace_flush()
