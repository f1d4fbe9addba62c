"""Process-group plumbing: one process per GPU, `torch.distributed` for bootstrap, and the
engine's communicators on a dedicated high-priority CUDA stream.

This is the part of the external trainer (`bagua.torch_api.communication`) that the
reference expects to exist around it: it creates `BaguaCommBackendPy(schedule_channel_cap,
device_id)`, generates the NCCL unique id on rank 0, distributes it out of band and builds
one `BaguaSingleCommunicatorPy` per (group, stream)
(reference: bagua-core-py/src/lib.rs:21-38,190-193,308-313).
"""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import BaguaCommBackendPy, BaguaSingleCommunicatorPy

_lock = threading.Lock()
_state: Optional["BaguaProcessGroup"] = None


def get_rank() -> int:
    return int(os.environ.get("RANK", "0"))


def get_world_size() -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


def get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def get_local_size() -> int:
    return int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))


@dataclass
class BaguaProcessGroup:
    """Communicators of one set of ranks.

    `global_comm` spans all ranks.  `intra_comm` spans the ranks of this node and
    `inter_comm` the node leaders (local rank 0); they are what `hierarchical=True`
    algorithms use.
    """

    rank: int
    world_size: int
    device: torch.device
    backend: BaguaCommBackendPy
    comm_stream: Optional[torch.cuda.Stream]
    global_comm: BaguaSingleCommunicatorPy
    intra_comm: Optional[BaguaSingleCommunicatorPy] = None
    inter_comm: Optional[BaguaSingleCommunicatorPy] = None
    _keep: list = field(default_factory=list)
    _hier_done: bool = False
    cpu_affinity: dict = field(default_factory=dict)  # what utils.affinity.bind_to_gpu_cpus did for this rank

    @property
    def stream_ptr(self) -> int:
        return self.comm_stream.cuda_stream if self.comm_stream is not None else 0

    @property
    def is_cuda(self) -> bool:
        return self.device.type == "cuda"

    def ensure_hierarchical(self):
        """Create the intra-node / inter-node communicators on first use.  Collective over
        all ranks (every rank reaches it when it builds a `hierarchical=True` op); kept lazy
        so that the common flat case pays for one communicator only."""
        if self._hier_done:
            return
        self._hier_done = True
        world = self.world_size
        local_size = max(1, min(get_local_size(), world))
        if world < 2 or world % local_size != 0:
            return
        n_nodes = world // local_size
        for node in range(n_nodes):
            ranks = list(range(node * local_size, (node + 1) * local_size))
            c = _new_comm(ranks, self.rank, self.device, self.stream_ptr, self._keep)
            if c is not None:
                self.intra_comm = c
        leaders = [n * local_size for n in range(n_nodes)]
        self.inter_comm = _new_comm(leaders, self.rank, self.device, self.stream_ptr, self._keep)

    def wait_comm_stream(self):
        """Make the current (compute) stream wait for everything queued on the comm stream."""
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)


def _bcast_str(s: Optional[str], src: int, group=None) -> str:
    obj = [s]
    dist.broadcast_object_list(obj, src=src, group=group)
    return obj[0]


def _new_comm(ranks: List[int], my_rank: int, device: torch.device, stream_ptr: int, keep: list):
    """Collective over ALL ranks of the default group (new_group is); returns this rank's
    communicator for `ranks`, or None if it is not a member."""
    member = my_rank in ranks
    if device.type == "cuda":
        group = dist.new_group(ranks)
        keep.append(group)
        uid = None
        if member:
            if my_rank == ranks[0]:
                uid = BaguaSingleCommunicatorPy.generate_nccl_unique_id_str()
            uid = _bcast_str(uid, src=ranks[0], group=group)
            return BaguaSingleCommunicatorPy(ranks.index(my_rank), len(ranks), device.index, stream_ptr, uid)
        return None
    group = dist.new_group(ranks, backend="gloo")
    keep.append(group)
    if not member:
        return None
    return BaguaSingleCommunicatorPy(ranks.index(my_rank), len(ranks), -1, 0, "c10d:" + group.group_name)


def init_process_group(device: Optional[torch.device] = None, schedule_channel_cap: int = 100) -> BaguaProcessGroup:
    """Initialise torch.distributed (if needed) and the engine's communicators.

    Reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT like `torchrun` sets
    them.  On CUDA the default torch backend is NCCL, on CPU gloo.
    """
    global _state
    with _lock:
        if _state is not None:
            return _state
        rank, world = get_rank(), get_world_size()
        if device is None:
            device = torch.device("cuda", get_local_rank()) if torch.cuda.is_available() else torch.device("cpu")
        affinity = {"applied": False, "cpus": 0, "reason": "host backend"}
        if device.type == "cuda":
            torch.cuda.set_device(device)
            # before any of this package's threads exist: they inherit the mask
            from ..utils.affinity import bind_for_cuda_device

            affinity = bind_for_cuda_device(device)
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            if device.type == "cuda":
                dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
            else:
                dist.init_process_group("gloo", rank=rank, world_size=world)
        keep: list = []
        if device.type == "cuda":
            # highest priority by default, so that communication kernels are scheduled ahead of the
            # backward kernels queued before them (BAGUA_B200_COMM_PRIORITY=low|normal|high)
            lo, hi = torch.cuda.Stream.priority_range() if hasattr(torch.cuda.Stream, "priority_range") else (0, -1)
            prio = {"low": lo, "normal": 0, "high": hi}.get(os.environ.get("BAGUA_B200_COMM_PRIORITY", "high"), hi)
            comm_stream = torch.cuda.Stream(device=device, priority=prio)
            stream_ptr = comm_stream.cuda_stream
            dev_id = device.index
        else:
            comm_stream, stream_ptr, dev_id = None, 0, -1
        backend = BaguaCommBackendPy(schedule_channel_cap, dev_id)
        all_ranks = list(range(world))
        global_comm = _new_comm(all_ranks, rank, device, stream_ptr, keep)
        _state = BaguaProcessGroup(rank, world, device, backend, comm_stream, global_comm, None, None, keep)
        _state.cpu_affinity = affinity
        return _state


def get_process_group() -> BaguaProcessGroup:
    if _state is None:
        return init_process_group()
    return _state


def destroy_process_group():
    global _state
    with _lock:
        if _state is None:
            return
        try:
            _state.backend.wait_pending_comm_ops()
        except Exception:
            pass
        _state.backend.close()
        _state = None
