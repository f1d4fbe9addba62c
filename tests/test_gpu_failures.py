"""Failure detection on real GPUs, without faulting one: a rank that stays alive but never joins a
fused op.  The other rank's kernel waits for its signal with a one-second budget, gives up, records
what it waited for in the host-mapped status record and returns; the host turns that into a
`RuntimeError`, marks the communicator aborted, and the CUDA context stays usable.  The silent rank
keeps its memory mapped until both are done, so no kernel ever touches freed memory.

Runs as two child processes with NVLS off in NCCL and the fused kernels on plain peer stores.
Switched on with BAGUA_B200_TEST_GPU_FAILURES=1 (it has not had its first run on hardware yet)."""
import os
import time

import pytest
import torch

from mp_util import run_ranks

pytestmark = [
    pytest.mark.gpu,
    pytest.mark.multigpu,
    pytest.mark.skipif(os.environ.get("BAGUA_B200_TEST_GPU_FAILURES", "0") != "1",
                       reason="set BAGUA_B200_TEST_GPU_FAILURES=1 to run the multi-GPU failure-detection test"),
]


def _silent_peer(rank, world):
    import torch.distributed as dist

    import bagua_core as bc

    dev = torch.device("cuda", rank)
    stream = torch.cuda.Stream()
    uid = [bc.BaguaSingleCommunicatorPy.generate_nccl_unique_id_str() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    comm = bc.BaguaSingleCommunicatorPy(rank, world, rank, stream.cuda_stream, uid[0])
    assert comm.fused_available()
    comm.set_device_wait_ms(1000.0)
    x = torch.full((1 << 16,), float(rank + 1), device=dev)
    bt = bc.BaguaTensorPy(x, "x")

    # step 1: everybody joins
    torch.cuda.synchronize()
    assert comm.fused_allreduce(bt, bt, True)
    stream.synchronize()
    comm.check_device_status()
    assert torch.allclose(x, torch.full_like(x, 1.5))
    dist.barrier()

    outcome = "silent"
    if rank == 0:
        # step 2: the peer never launches its half
        t0 = time.time()
        assert comm.fused_allreduce(bt, bt, True)
        stream.synchronize()  # returns: the kernel gave up after its budget
        elapsed = time.time() - t0
        try:
            comm.check_device_status()
            outcome = "no error"
        except RuntimeError as e:
            outcome = "error:" + str(e)
        assert comm.check_abort()
        # the context is still usable
        y = torch.ones(1024, device=dev) * 3
        assert float(y.sum().item()) == 3072.0
        assert elapsed < 30.0
    # the silent rank stays alive (its staging stays mapped) until rank 0 has finished
    dist.barrier()
    return outcome


def test_a_rank_that_never_joins_is_reported_and_the_context_survives(monkeypatch):
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    res = run_ranks(_silent_peer, 2, backend="nccl", timeout=300)
    assert res[1] == "silent"
    assert res[0].startswith("error:") and "ran out" in res[0] and "peer 1" in res[0], res[0]
