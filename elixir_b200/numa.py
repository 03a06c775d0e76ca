"""Host memory close to a GPU.

Pinned host buffers are placed on the NUMA node of the CPU that allocates them (first touch); a buffer on the other
socket makes every PCIe transfer cross the inter-socket link as well.  ``near_gpu(device)`` narrows the calling
thread's CPU affinity to the CPUs of the GPU's own NUMA node for the duration of a ``with`` block — allocate the pinned
buffers inside it — and restores it afterwards.  Where the node is unknown, or none of its CPUs may be used by this
process, the block runs unchanged.  Linux sysfs only; nothing is read from or written to the GPU.
"""
import contextlib
import os

import torch


def _parse_cpulist(text: str):
    cpus = set()
    for part in text.strip().split(','):
        if not part:
            continue
        lo, _, hi = part.partition('-')
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_cpus(device) -> set:
    """CPUs of the NUMA node the GPU hangs on that this process may run on; empty if that cannot be told."""
    try:
        props = torch.cuda.get_device_properties(device)
        bus = f'{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0'
        with open(f'/sys/bus/pci/devices/{bus}/numa_node') as f:
            node = int(f.read().strip())
        if node < 0:
            return set()
        with open(f'/sys/devices/system/node/node{node}/cpulist') as f:
            local = _parse_cpulist(f.read())
        return local & os.sched_getaffinity(0)
    except (OSError, ValueError, AttributeError, RuntimeError, AssertionError):
        return set()


@contextlib.contextmanager
def near_gpu(device):
    """Run the block on the CPUs of ``device``'s NUMA node (see the module text).  Yields the CPU set used, or an empty
    set when the affinity was left as it was."""
    cpus = gpu_numa_cpus(device)
    before = os.sched_getaffinity(0)
    if not cpus or cpus == before:
        yield set() if not cpus else cpus
        return
    os.sched_setaffinity(0, cpus)
    try:
        yield cpus
    finally:
        os.sched_setaffinity(0, before)
