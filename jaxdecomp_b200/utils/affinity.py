"""CPU placement of a rank next to its GPU.

A rank that feeds its GPU from pinned host memory gets the full PCIe rate only
when that memory lives on the NUMA node the GPU hangs off.  Linux places pages
on the node of the thread that first touches them, so it is enough to restrict
the process to the CPUs NVML reports as local to the device *before* the
buffers are allocated.  Only this process's own scheduling mask is changed;
nothing is written to the GPU or the driver.

The reference leaves placement to the job launcher (``slurms/template.slurm``
uses ``--cpu-bind`` / ``--hint=nomultithread``).
"""
from __future__ import annotations

import os
from typing import Optional, Set

__all__ = ["device_local_cpus", "bind_to_device_cpus"]


def _nvml_handle(device_index: int):
    import pynvml
    import torch

    pynvml.nvmlInit()
    props = torch.cuda.get_device_properties(device_index)
    uuid = getattr(props, "uuid", None)
    if uuid is not None:
        for cand in (f"GPU-{uuid}", str(uuid)):
            try:
                return pynvml, pynvml.nvmlDeviceGetHandleByUUID(cand.encode())
            except Exception:  # noqa: BLE001 - try the next spelling
                continue
    return pynvml, pynvml.nvmlDeviceGetHandleByIndex(device_index)


def device_local_cpus(device_index: int) -> Optional[Set[int]]:
    """CPUs that NVML lists as local to CUDA device ``device_index`` (None when unknown)."""
    try:
        nv, h = _nvml_handle(device_index)
        ncpu = os.cpu_count() or 1
        words = (ncpu + 63) // 64
        mask = nv.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {i for i in range(words * 64) if (int(mask[i // 64]) >> (i % 64)) & 1}
        return cpus or None
    except Exception:  # noqa: BLE001 - no NVML, no permission, or not a CUDA device
        return None


def bind_to_device_cpus(device_index: int) -> Optional[Set[int]]:
    """Restrict this process to the CPUs local to its GPU (intersected with the CPUs it is already allowed
    to use).  Returns the new mask, or None when nothing was changed.  ``JD_B200_BIND_CPUS=0`` disables it."""
    if os.environ.get("JD_B200_BIND_CPUS", "1") == "0" or not hasattr(os, "sched_setaffinity"):
        return None
    local = device_local_cpus(device_index)
    if not local:
        return None
    try:
        allowed = os.sched_getaffinity(0)
        target = local & allowed
        if not target or target == allowed:
            return None
        os.sched_setaffinity(0, target)
        return target
    except OSError:
        return None
