"""Functional collectives on torch tensors, the way a trainer calls them
(`allreduce(send, recv, op)`, `broadcast(t, src)`, `alltoall_v(...)`, ...).

Each function wraps the tensors as `BaguaTensorPy`, orders the engine's communication stream
after the caller's current CUDA stream, issues the communicator call there
(reference surface: bagua-core-py/src/lib.rs:60-188), and orders the caller's stream after it, so
the result can be used like the output of any other asynchronous CUDA op — no host
synchronisation.  On the CPU backend the calls are synchronous.  `comm` defaults to the global
communicator of `init_process_group()`.
"""
from __future__ import annotations

from contextlib import contextmanager
from enum import IntEnum
from typing import Optional, Sequence

import torch

from .. import BaguaSingleCommunicatorPy, BaguaTensorPy
from .communication import get_process_group


class ReduceOp(IntEnum):
    """Reduction codes of the communicator API (the `op: u8` argument)."""

    SUM = 0
    PRODUCT = 1
    MIN = 2
    MAX = 3
    LOR = 4
    LAND = 5
    LXOR = 6
    BOR = 7
    BAND = 8
    BXOR = 9
    AVG = 10


def _comm(comm: Optional[BaguaSingleCommunicatorPy]) -> BaguaSingleCommunicatorPy:
    return comm if comm is not None else get_process_group().global_comm


@contextmanager
def _on_comm_stream(*tensors: torch.Tensor):
    """Order the communication stream after the current stream, and the current stream after it."""
    pg = get_process_group()
    stream = pg.comm_stream
    cuda = [t for t in tensors if t is not None and t.is_cuda]
    if stream is None or not cuda:
        yield
        return
    current = torch.cuda.current_stream(cuda[0].device)
    stream.wait_stream(current)
    for t in cuda:
        t.record_stream(stream)
    yield
    current.wait_stream(stream)


def _wrap(t: torch.Tensor, name: str) -> BaguaTensorPy:
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return BaguaTensorPy(t, name)


def allreduce(send_tensor: torch.Tensor, recv_tensor: torch.Tensor, op: int = ReduceOp.SUM, comm=None):
    with _on_comm_stream(send_tensor, recv_tensor):
        _comm(comm).allreduce(_wrap(send_tensor, "send"), _wrap(recv_tensor, "recv"), int(op))


def allreduce_inplace(tensor: torch.Tensor, op: int = ReduceOp.SUM, comm=None):
    with _on_comm_stream(tensor):
        _comm(comm).allreduce_inplace(_wrap(tensor, "tensor"), int(op))


def broadcast(tensor: torch.Tensor, src: int = 0, comm=None):
    with _on_comm_stream(tensor):
        _comm(comm).broadcast(_wrap(tensor, "tensor"), src)


def reduce(send_tensor: torch.Tensor, recv_tensor: torch.Tensor, dst: int, op: int = ReduceOp.SUM, comm=None):
    with _on_comm_stream(send_tensor, recv_tensor):
        _comm(comm).reduce(_wrap(send_tensor, "send"), _wrap(recv_tensor, "recv"), dst, int(op))


def reduce_inplace(tensor: torch.Tensor, dst: int, op: int = ReduceOp.SUM, comm=None):
    with _on_comm_stream(tensor):
        _comm(comm).reduce_inplace(_wrap(tensor, "tensor"), dst, int(op))


def send(tensor: torch.Tensor, dst: int, comm=None):
    with _on_comm_stream(tensor):
        _comm(comm).send(_wrap(tensor, "tensor"), dst)


def recv(tensor: torch.Tensor, src: int, comm=None):
    with _on_comm_stream(tensor):
        _comm(comm).recv(_wrap(tensor, "tensor"), src)


def allgather(send_tensor: torch.Tensor, recv_tensor: torch.Tensor, comm=None):
    """recv_tensor holds world_size * send_tensor.numel() elements, rank r's part at chunk r."""
    with _on_comm_stream(send_tensor, recv_tensor):
        _comm(comm).allgather(_wrap(send_tensor, "send"), _wrap(recv_tensor, "recv"))


def allgather_inplace(tensor: torch.Tensor, comm=None):
    """Chunk `rank` of the tensor is this rank's contribution."""
    with _on_comm_stream(tensor):
        _comm(comm).allgather_inplace(_wrap(tensor, "tensor"))


def gather(send_tensor: torch.Tensor, recv_tensor: torch.Tensor, dst: int, comm=None):
    with _on_comm_stream(send_tensor, recv_tensor):
        _comm(comm).gather(_wrap(send_tensor, "send"), _wrap(recv_tensor, "recv"), dst)


def gather_inplace(tensor: torch.Tensor, count: int, dst: int, comm=None):
    with _on_comm_stream(tensor):
        _comm(comm).gather_inplace(_wrap(tensor, "tensor"), count, dst)


def scatter(send_tensor: torch.Tensor, recv_tensor: torch.Tensor, src: int, comm=None):
    with _on_comm_stream(send_tensor, recv_tensor):
        _comm(comm).scatter(_wrap(send_tensor, "send"), _wrap(recv_tensor, "recv"), src)


def scatter_inplace(tensor: torch.Tensor, count: int, src: int, comm=None):
    with _on_comm_stream(tensor):
        _comm(comm).scatter_inplace(_wrap(tensor, "tensor"), count, src)


def reduce_scatter(send_tensor: torch.Tensor, recv_tensor: torch.Tensor, op: int = ReduceOp.SUM, comm=None):
    """send_tensor holds world_size * recv_tensor.numel() elements; rank r receives the sum of chunk r."""
    with _on_comm_stream(send_tensor, recv_tensor):
        _comm(comm).reduce_scatter(_wrap(send_tensor, "send"), _wrap(recv_tensor, "recv"), int(op))


def reduce_scatter_inplace(tensor: torch.Tensor, op: int = ReduceOp.SUM, comm=None):
    """The reduced chunk `rank` replaces chunk `rank` of the tensor."""
    with _on_comm_stream(tensor):
        _comm(comm).reduce_scatter_inplace(_wrap(tensor, "tensor"), int(op))


def alltoall(send_tensor: torch.Tensor, recv_tensor: torch.Tensor, comm=None):
    with _on_comm_stream(send_tensor, recv_tensor):
        _comm(comm).alltoall(_wrap(send_tensor, "send"), _wrap(recv_tensor, "recv"))


def alltoall_inplace(tensor: torch.Tensor, comm=None):
    with _on_comm_stream(tensor):
        _comm(comm).alltoall_inplace(_wrap(tensor, "tensor"))


def alltoall_v(send_tensor: torch.Tensor, send_counts: Sequence[int], send_displs: Sequence[int],
               recv_tensor: torch.Tensor, recv_counts: Sequence[int], recv_displs: Sequence[int], comm=None):
    """Element counts and displacements per peer rank, as in MPI_Alltoallv."""
    with _on_comm_stream(send_tensor, recv_tensor):
        _comm(comm).alltoall_v(_wrap(send_tensor, "send"), list(send_counts), list(send_displs),
                               _wrap(recv_tensor, "recv"), list(recv_counts), list(recv_displs))


def barrier(comm=None):
    """Returns once every rank of the communicator has reached the call."""
    pg = get_process_group()
    if pg.comm_stream is not None:
        pg.comm_stream.wait_stream(torch.cuda.current_stream(pg.device))
    _comm(comm).barrier()
