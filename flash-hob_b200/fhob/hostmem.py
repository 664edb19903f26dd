"""Host-side placement for the host-buffer path.

``flash_bwdbwd`` with host tensors moves every input over PCIe once and every
result back, so its speed is the speed of those copies.  On a two-socket host
a pinned buffer that lives on the other socket's memory crosses the socket
interconnect on its way to the GPU and can run at half the rate.  Pinned pages
are placed on the NUMA node of the thread that allocates them, so binding the
process to the CPUs next to the GPU *before* allocating is all it takes.
"""
from __future__ import annotations

import os
from contextlib import contextmanager
from pathlib import Path
from typing import Optional, Set

import torch


def _parse_cpulist(text: str) -> Set[int]:
    cpus: Set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def device_local_cpus(device, sysfs: str = "/sys/bus/pci/devices") -> Optional[dict]:
    """CPUs and NUMA node the kernel reports as local to a CUDA device's PCIe slot, or None."""
    try:
        props = torch.cuda.get_device_properties(device)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        base = Path(sysfs) / bdf
        cpus = _parse_cpulist((base / "local_cpulist").read_text())
        node = int((base / "numa_node").read_text().strip())
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None
    return dict(pci=bdf, numa_node=node, cpus=cpus)


@contextmanager
def near_device(device):
    """Binds the calling process to the CPUs local to `device` for the duration of the block
    (allocate and fill pinned buffers inside it).  Yields a short record of what was done; does
    nothing when the topology cannot be read or none of the local CPUs is allowed to the process."""
    info = device_local_cpus(device)
    before = os.sched_getaffinity(0)
    record = dict(bound=False)
    if info is not None:
        record.update(pci=info["pci"], numa_node=info["numa_node"])
        target = info["cpus"] & before
        if target and target != before:
            try:
                os.sched_setaffinity(0, target)
                record.update(bound=True, cpus=len(target))
            except OSError:
                pass
        elif target:
            record.update(cpus=len(target), note="already on the device's CPUs")
    try:
        yield record
    finally:
        if record["bound"]:
            os.sched_setaffinity(0, before)
