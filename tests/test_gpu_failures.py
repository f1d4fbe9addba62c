"""Failure detection on real GPUs, without faulting one: a rank that stays alive but never joins a
fused op.  The other rank's kernel waits for its signal with a short budget, gives up, records
what it waited for in the host-mapped status record and returns; the engine turns that into a
`RuntimeError` from `wait_pending_comm_ops`, marks the communicator aborted and refuses to start
further kernels on it, and the CUDA context stays usable.  A second case shows that `abort()`
reaches a kernel that is waiting for a peer long before its budget is spent.  The silent rank
keeps its memory mapped until both are done, so no kernel ever touches freed memory.

Runs as two child processes with NVLS off in NCCL and the fused kernels on plain peer stores."""
import time

import pytest
import torch

from mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _mk(rank, world, wait_ms):
    import torch.distributed as dist

    import bagua_core as bc

    stream = torch.cuda.Stream()
    uid = [bc.BaguaSingleCommunicatorPy.generate_nccl_unique_id_str() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    comm = bc.BaguaSingleCommunicatorPy(rank, world, rank, stream.cuda_stream, uid[0])
    assert comm.fused_available()
    comm.set_device_wait_ms(wait_ms)
    return bc, comm, stream


def _silent_peer(rank, world):
    import torch.distributed as dist

    bc, comm, stream = _mk(rank, world, 1000.0)
    dev = torch.device("cuda", rank)
    x = torch.full((1 << 16,), float(rank + 1), device=dev)
    bt = bc.BaguaTensorPy(x, "x")
    backend = bc.BaguaCommBackendPy(10, rank)
    bucket = bc.BaguaBucketPy("b", [bt])
    bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True)
    backend.register_ordered_buckets([bucket])

    # step 1: everybody joins, through the engine (scheduler, worker thread, fused kernel)
    torch.cuda.synchronize()
    backend.mark_communication_ready(bt, 0)
    assert backend.wait_pending_comm_ops() == 1
    stream.synchronize()
    assert torch.allclose(x, torch.full_like(x, 1.5))
    dist.barrier()

    out = {"first": "silent", "later": "", "elapsed": 0.0}
    if rank == 0:
        # step 2: the peer never launches its half
        t0 = time.time()
        backend.mark_communication_ready(bt, 0)
        backend.wait_pending_comm_ops()  # the kernel is queued and waiting: nothing to report yet
        stream.synchronize()  # returns: the kernel gave up after its budget
        out["elapsed"] = time.time() - t0
        try:
            backend.wait_pending_comm_ops()
            out["first"] = "no error"
        except RuntimeError as e:
            out["first"] = "error:" + str(e)
        assert comm.check_abort()
        # no further kernel is started on the aborted communicator: the next bucket fails at once
        backend.mark_communication_ready(bt, 0)
        try:
            backend.wait_pending_comm_ops()
            out["later"] = "no error"
        except RuntimeError as e:
            out["later"] = str(e)
        # the context is still usable
        y = torch.ones(1024, device=dev) * 3
        assert float(y.sum().item()) == 3072.0
    # the silent rank stays alive (its staging stays mapped) until rank 0 has finished
    dist.barrier()
    backend.close()
    return out


def test_a_rank_that_never_joins_fails_the_step_and_the_context_survives(monkeypatch):
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    res = run_ranks(_silent_peer, 2, backend="nccl", timeout=300)
    assert res[1]["first"] == "silent"
    first = res[0]["first"]
    assert first.startswith("error:") and "ran out" in first and "peer 1" in first, first
    assert "aborted" in res[0]["later"], res[0]["later"]
    assert res[0]["elapsed"] < 30.0


def _abort_while_waiting(rank, world):
    import torch.distributed as dist

    bc, comm, stream = _mk(rank, world, 60000.0)
    dev = torch.device("cuda", rank)
    x = torch.full((1 << 16,), float(rank + 1), device=dev)
    bt = bc.BaguaTensorPy(x, "x")
    torch.cuda.synchronize()
    assert comm.fused_allreduce(bt, bt, True)
    stream.synchronize()
    dist.barrier()
    elapsed = 0.0
    if rank == 0:
        assert comm.fused_allreduce(bt, bt, True)  # waits for a peer that stays silent, budget one minute
        time.sleep(0.3)
        assert not stream.query()
        t0 = time.time()
        comm.abort()
        stream.synchronize()
        elapsed = time.time() - t0
        assert comm.check_abort()
        y = torch.ones(1024, device=dev) * 3
        assert float(y.sum().item()) == 3072.0
    dist.barrier()
    return elapsed


def test_abort_reaches_a_kernel_that_waits_for_a_peer(monkeypatch):
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    res = run_ranks(_abort_while_waiting, 2, backend="nccl", timeout=300)
    assert res[0] < 10.0, res
