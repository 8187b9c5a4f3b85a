"""Placing pinned host memory on the NUMA node of the GPU that will copy from / to it.

The reference keeps master weights, moments and the shared gradient / staging buffers in pinned
host memory (transformer_layer.py:192-196, offload_transformer.py:85-93) wherever the process
happens to run.  On a two-socket host with eight GPUs, half of the GPUs then reach their buffers
across the socket interconnect; allocating them from a CPU next to the GPU keeps every PCIe
copy on the local root complex.
"""
from __future__ import annotations

import contextlib
import os
from pathlib import Path
from typing import Optional

import torch


def _parse_cpulist(text: str) -> set:
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


_CPUS_OF_GPU: dict = {}


def gpu_numa_cpus(device, sysfs: str = "/sys") -> Optional[set]:
    """CPUs of the NUMA node the GPU's PCIe slot hangs off, read from sysfs; None when the
    machine does not say (single node, virtualised PCI topology, no NVML).  Looked up once per
    device."""
    key = (str(device), sysfs)
    if key not in _CPUS_OF_GPU:
        _CPUS_OF_GPU[key] = _gpu_numa_cpus(device, sysfs)
    return _CPUS_OF_GPU[key]


def _gpu_numa_cpus(device, sysfs: str) -> Optional[set]:
    try:
        import pynvml
        pynvml.nvmlInit()
        dev = torch.device(device)
        uuid = str(torch.cuda.get_device_properties(dev).uuid)
        bus = None
        for i in range(pynvml.nvmlDeviceGetCount()):
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            u = pynvml.nvmlDeviceGetUUID(h)
            if uuid in (u.decode() if isinstance(u, bytes) else u):
                b = pynvml.nvmlDeviceGetPciInfo(h).busId
                bus = (b.decode() if isinstance(b, bytes) else b).lower()
                break
        if bus is None:
            return None
        if len(bus.split(":")[0]) == 8:          # NVML prints an 8-digit PCI domain, sysfs a 4-digit one
            bus = bus[4:]
        return numa_cpus_of_pci(bus, sysfs)
    except Exception:
        return None


def numa_cpus_of_pci(bus_id: str, sysfs: str = "/sys") -> Optional[set]:
    try:
        node = int((Path(sysfs) / "bus/pci/devices" / bus_id / "numa_node").read_text())
        if node < 0:
            return None
        cpus = _parse_cpulist((Path(sysfs) / f"devices/system/node/node{node}/cpulist").read_text())
        return cpus or None
    except (OSError, ValueError):
        return None


@contextlib.contextmanager
def numa_local(device):
    """Run the body on the CPUs next to `device`, so that host memory allocated (and pinned)
    inside lands on the GPU's own NUMA node and its PCIe copies do not cross the socket
    interconnect.  The thread's CPU mask is restored afterwards; without topology information
    the body simply runs where it is."""
    cpus = gpu_numa_cpus(device)
    old = None
    if cpus:
        try:
            old = os.sched_getaffinity(0)
            allowed = cpus & old
            if allowed:
                os.sched_setaffinity(0, allowed)
            else:
                old = None
        except OSError:
            old = None
    try:
        yield bool(old)
    finally:
        if old is not None:
            os.sched_setaffinity(0, old)


def pinned_empty(numel: int, dtype, device) -> torch.Tensor:
    """Pinned host tensor placed on the NUMA node of `device` where the topology is known."""
    with numa_local(device):
        t = torch.empty(int(numel), dtype=dtype).pin_memory()
    return t


