"""Keep a rank's host threads on the CPUs next to its GPU.

A training step of an eager PyTorch model is a few hundred kernel launches, and with one process
per GPU on a two-socket host the scheduler is free to run a rank on the socket its GPU is not
attached to (and to move it between steps): every launch then crosses the socket interconnect,
and the slowest rank's launching thread paces every collective.  `bind_to_gpu_cpus` asks NVML
for the CPUs that are local to the GPU and restricts all threads of the process to the ones the
process was already allowed to use.  It only ever narrows the existing mask, does nothing when
fewer than `min_cpus` CPUs (or fewer than four per GPU that reports the same set) would be left,
and changes nothing on the GPU (NVML is only read).

The reference leaves placement to the launcher (it has no counterpart); NCCL does the same for
its own threads.  Switch off with BAGUA_B200_CPU_AFFINITY=0.
"""
from __future__ import annotations

import os
from typing import Iterable, Optional, Set


def _mask_words_to_cpus(words: Iterable[int], bits: int = 64) -> Set[int]:
    cpus: Set[int] = set()
    for w_index, word in enumerate(words):
        word = int(word)
        bit = 0
        while word:
            if word & 1:
                cpus.add(w_index * bits + bit)
            word >>= 1
            bit += 1
    return cpus


def _nvml_handle(nvml, device_index: int, uuid: Optional[str], pci_bus_id: Optional[str]):
    """The NVML handle of the CUDA device: by UUID, else by PCI bus id, else by index (NVML's
    index equals CUDA's only when CUDA_VISIBLE_DEVICES does not reorder the devices)."""
    if uuid:
        name = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        for arg in (name, name.encode()):  # NVML bindings differ in whether they take str or bytes
            try:
                return nvml.nvmlDeviceGetHandleByUUID(arg)
            except Exception:
                pass
    if pci_bus_id:
        for arg in (pci_bus_id, pci_bus_id.encode()):
            try:
                return nvml.nvmlDeviceGetHandleByPciBusId(arg)
            except Exception:
                pass
    if os.environ.get("CUDA_VISIBLE_DEVICES"):
        return None
    return nvml.nvmlDeviceGetHandleByIndex(device_index)


def gpu_local_cpus(device_index: int, nvml=None, uuid: Optional[str] = None,
                   pci_bus_id: Optional[str] = None):
    """(CPUs that NVML reports as local to the GPU, number of GPUs of the machine that report the
    same set), or (None, 0) when that cannot be found out."""
    own = nvml is None
    try:
        if own:
            import pynvml as nvml  # type: ignore
        nvml.nvmlInit()
    except Exception:
        return None, 0
    try:
        handle = _nvml_handle(nvml, device_index, uuid, pci_bus_id)
        if handle is None:
            return None, 0
        n_words = ((os.cpu_count() or 64) + 63) // 64
        cpus = _mask_words_to_cpus(nvml.nvmlDeviceGetCpuAffinity(handle, n_words))
        if not cpus:
            return None, 0
        sharing = 0
        try:
            for i in range(int(nvml.nvmlDeviceGetCount())):
                other = nvml.nvmlDeviceGetHandleByIndex(i)
                if _mask_words_to_cpus(nvml.nvmlDeviceGetCpuAffinity(other, n_words)) == cpus:
                    sharing += 1
        except Exception:
            sharing = 0
        return cpus, max(sharing, 1)
    except Exception:
        return None, 0
    finally:
        try:
            nvml.nvmlShutdown()
        except Exception:
            pass


def _all_thread_ids() -> list:
    try:
        return [int(t) for t in os.listdir("/proc/self/task")]
    except OSError:
        return [0]


def bind_to_gpu_cpus(device_index: int, min_cpus: int = 8, nvml=None, uuid: Optional[str] = None,
                     pci_bus_id: Optional[str] = None, per_rank_cpus: int = 4) -> dict:
    """Restrict every thread of this process to the CPUs local to GPU `device_index`.

    Returns what was done: {"applied": bool, "cpus": count in force afterwards, "reason": why not}.
    Threads created later inherit the mask of the thread that creates them."""
    if os.environ.get("BAGUA_B200_CPU_AFFINITY", "1") == "0":
        return {"applied": False, "cpus": 0, "reason": "switched off"}
    if not hasattr(os, "sched_setaffinity"):
        return {"applied": False, "cpus": 0, "reason": "no sched_setaffinity on this platform"}
    allowed = set(os.sched_getaffinity(0))
    local, sharing = gpu_local_cpus(device_index, nvml=nvml, uuid=uuid, pci_bus_id=pci_bus_id)
    if not local:
        return {"applied": False, "cpus": len(allowed), "reason": "NVML reports no CPU set for the GPU"}
    target = allowed & local
    # every GPU that reports the same set may have a rank of its own on it: leave each at least
    # `per_rank_cpus`, or a mask that looked local would crowd the ranks onto a few cores
    need = max(min_cpus, per_rank_cpus * sharing)
    if len(target) < need:
        return {"applied": False, "cpus": len(allowed),
                "reason": f"only {len(target)} of the GPU's CPUs are available to this process "
                          f"({sharing} GPU(s) share them, {need} wanted)"}
    if target == allowed:
        return {"applied": False, "cpus": len(allowed), "reason": "already there"}
    done = 0
    for tid in _all_thread_ids():
        try:
            os.sched_setaffinity(tid, target)
            done += 1
        except OSError:
            pass  # a thread that has just exited, or one the kernel does not let us move
    if done == 0:
        return {"applied": False, "cpus": len(allowed), "reason": "sched_setaffinity refused"}
    return {"applied": True, "cpus": len(target), "reason": ""}


def bind_for_cuda_device(device) -> dict:
    """`bind_to_gpu_cpus` for a torch CUDA device (identifies it to NVML by UUID or PCI address)."""
    import torch

    uuid = pci = None
    try:
        props = torch.cuda.get_device_properties(device)
        uuid = str(getattr(props, "uuid", "") or "") or None
        if hasattr(props, "pci_bus_id"):
            pci = "%08x:%02x:%02x.0" % (int(getattr(props, "pci_domain_id", 0)), int(props.pci_bus_id),
                                        int(getattr(props, "pci_device_id", 0)))
    except Exception:
        pass
    index = device.index if getattr(device, "index", None) is not None else torch.cuda.current_device()
    return bind_to_gpu_cpus(int(index), uuid=uuid, pci_bus_id=pci)
