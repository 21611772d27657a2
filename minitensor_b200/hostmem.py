"""Host-side placement for the batches a training loop feeds to its GPU.

On a multi-socket host a pinned buffer lives on the NUMA node of the thread that first touches it.  A rank whose
buffers sit on the far socket pulls every batch across the socket interconnect, and with eight ranks copying at once
that link, not PCIe, bounds the copy rate.  ``bind_host_to_gpu`` restricts the calling process to the CPUs NVML
reports as local to the GPU, so that buffers allocated and filled afterwards are local too.  It changes nothing on
the device and no setting that outlasts the process.
"""
from __future__ import annotations

import os
from typing import Optional


def _nvml_handle(pynvml, device_index: int):
    import torch
    props = torch.cuda.get_device_properties(device_index)
    uuid = getattr(props, "uuid", None)
    if uuid is not None:
        try:
            return pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
        except Exception:
            pass
    bus = getattr(props, "pci_bus_id", None)
    if bus is not None:
        bus_id = f"{getattr(props, 'pci_domain_id', 0):08x}:{bus:02x}:{getattr(props, 'pci_device_id', 0):02x}.0"
        try:
            return pynvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
        except Exception:
            pass
    if "CUDA_VISIBLE_DEVICES" not in os.environ:
        return pynvml.nvmlDeviceGetHandleByIndex(device_index)   # same enumeration order only without a device mask
    raise RuntimeError("cannot match the CUDA device to an NVML device")


def bind_host_to_gpu(device_index: int) -> Optional[dict]:
    """Restrict this process to the CPUs local to CUDA device ``device_index``.

    Returns ``{"cpus": n, "first": lowest cpu, "last": highest cpu}`` or ``None`` when the host gives no answer
    (no NVML, a single node, an affinity mask that excludes the local CPUs); failure never raises.
    """
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            handle = _nvml_handle(pynvml, device_index)
            ncpu = os.cpu_count() or 1
            words = pynvml.nvmlDeviceGetCpuAffinity(handle, (ncpu + 63) // 64)
        finally:
            pynvml.nvmlShutdown()
        local = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        cpus = sorted(local & allowed)
        if not cpus or len(cpus) == len(allowed):
            return None
        os.sched_setaffinity(0, cpus)
        return {"cpus": len(cpus), "first": cpus[0], "last": cpus[-1]}
    except Exception:
        return None
