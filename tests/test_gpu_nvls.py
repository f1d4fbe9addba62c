"""All-reduce through the NVSwitch's multicast / reduction units (`multimem.ld_reduce` +
`multimem.st` on buckets in multicast-mapped symmetric memory, BAGUA_B200_NVLS=1) against the
fp32 sum.  Needs several GPUs behind an NVSwitch; newer than the rest of the GPU suite and
off by default, so it runs when BAGUA_B200_TEST_NVLS=1."""
import os

import pytest
import torch

from mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _mk_comm(rank, world, stream):
    import torch.distributed as dist

    import bagua_core as bc

    uid = [bc.BaguaSingleCommunicatorPy.generate_nccl_unique_id_str() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    return bc.BaguaSingleCommunicatorPy(rank, world, rank, stream.cuda_stream, uid[0])


def _nvls_allreduce(rank, world):
    """All-reduce through the switch's reduction units on buckets in multicast-mapped memory.

    A rank must not leave while its memory is bound to the multicast object and its peers are still
    inside a collective, so nothing here raises half way: mismatches are collected, every rank runs
    the same sequence to the end, all ranks drop their multicast bindings together, and only then is
    the list of mismatches returned."""
    import bagua_core as bc
    import bagua_core_b200 as bb

    dev = torch.device("cuda", rank)
    stream = torch.cuda.Stream()
    comm = _mk_comm(rank, world, stream)
    assert comm.fused_available()
    comm.set_device_wait_ms(20000.0)
    probe = comm.alloc_symmetric(1 << 20, torch.float32)
    assert probe is not None
    if not comm.is_nvls_mapped(probe):
        return "no multicast"  # the platform refused; the heap fell back to CUDA IPC on every rank (they agree)
    problems = []
    checked = 0
    for dt, tol in ((torch.float32, 1e-5), (torch.float16, 2e-3), (torch.bfloat16, 1.6e-2)):
        for n in ((1 << 18) + 64, 6 << 20):
            buf = comm.alloc_symmetric(n, dt)
            if not comm.is_nvls_mapped(buf):
                problems.append(f"{dt} {n}: not multicast-mapped")
            x = torch.randn(n, generator=torch.Generator().manual_seed(31 * rank + n % 53)).to(dt).to(dev)
            allx = [torch.empty_like(x) for _ in range(world)]
            torch.distributed.all_gather(allx, x)
            ref = torch.stack([a.float() for a in allx]).sum(0)
            for average in (True, False):
                buf.copy_(x)
                torch.cuda.synchronize()
                torch.distributed.barrier()
                before = comm.fused_launches()
                bt = bc.BaguaTensorPy(buf, "b")
                ok = comm.fused_allreduce(bt, bt, average)
                stream.synchronize()
                try:
                    comm.check_device_status()
                except RuntimeError as e:
                    problems.append(f"{dt} {n}: {e}")
                if not ok or comm.fused_launches() != before + 1:
                    problems.append(f"{dt} {n}: no fused launch")
                want = ref / world if average else ref
                if not torch.allclose(buf.float(), want, rtol=tol, atol=tol * max(1.0, want.abs().max().item())):
                    problems.append(f"{dt} {n} average={average}: max error {(buf.float() - want).abs().max().item()}")
                mine = buf.clone()  # the gather below runs on ordinary memory
                outs = [torch.empty_like(mine) for _ in range(world)]
                torch.distributed.all_gather(outs, mine)
                if not all(torch.equal(outs[0], o) for o in outs):
                    problems.append(f"{dt} {n}: ranks disagree")
                checked += 1
    torch.cuda.synchronize()
    torch.distributed.barrier()
    bb._C.release_multicast_slabs()  # every rank unbinds while all of them are alive
    torch.distributed.barrier()
    return problems if problems else checked


@pytest.mark.skipif(os.environ.get("BAGUA_B200_TEST_NVLS", "0") != "1",
                    reason="set BAGUA_B200_TEST_NVLS=1 to run the NVSwitch multicast all-reduce")
def test_nvls_allreduce_matches_fp32_sum(monkeypatch):
    monkeypatch.setenv("BAGUA_B200_NVLS", "1")
    world = min(torch.cuda.device_count(), int(os.environ.get("BAGUA_TEST_WORLD", "8")))
    res = run_ranks(_nvls_allreduce, world, backend="nccl", timeout=600)
    if res[0] == "no multicast":
        assert all(r == "no multicast" for r in res)
        pytest.skip("NVSwitch multicast is not available on this machine")
    assert all(r == 12 for r in res), res
