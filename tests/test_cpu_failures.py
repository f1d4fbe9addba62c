"""Failure handling, exercised on CPU ranks only (gloo): a rank that leaves, mismatched
buckets, aborted communicators.  Failures are made on the host; nothing here touches a GPU."""
import datetime
import os
import time
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mp_util import free_port


def _entry(rank, world, port, fn, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
        q.put((rank, "ok", fn(rank, world)))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def _run(fn, world=2, timeout=90):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    deadline = time.time() + timeout
    while len(out) < world and time.time() < deadline:
        try:
            rank, status, val = q.get(timeout=0.5)
            out[rank] = (status, val)
        except Exception:
            # a rank whose process is gone without a report died (e.g. the transport aborted it)
            for r, p in enumerate(procs):
                if r not in out and not p.is_alive():
                    p.join()
                    try:
                        rank, status, val = q.get(timeout=0.5)
                        out[rank] = (status, val)
                    except Exception:
                        out[r] = ("died", p.exitcode)
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.kill()
    return out


def _comm(rank, world):
    import bagua_core as bc

    return bc.BaguaSingleCommunicatorPy(rank, world, -1, 0, "c10d:" + dist.group.WORLD.group_name)


def _peer_leaves(rank, world):
    """Rank 1 leaves between steps; rank 0's next bucket must fail with an exception, not hang."""
    import bagua_core as bc

    comm = _comm(rank, world)
    backend = bc.BaguaCommBackendPy(10, -1)
    x = torch.ones(1024)
    t = bc.BaguaTensorPy(x, "x")
    b = bc.BaguaBucketPy("b", [t])
    b.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True)
    backend.register_ordered_buckets([b])
    backend.mark_communication_ready(t, 0)
    assert backend.wait_pending_comm_ops() == 1  # step 1 succeeds on both ranks
    if rank == 1:
        backend.close()
        dist.destroy_process_group()
        return "left"
    time.sleep(1.0)
    t0 = time.time()
    backend.mark_communication_ready(t, 0)
    try:
        backend.wait_pending_comm_ops()
        result = "no error"
    except RuntimeError as e:
        result = "error: " + str(e)[:200]
    elapsed = time.time() - t0
    backend.close()
    return result, elapsed


def test_rank_leaving_turns_into_an_exception_on_the_survivor():
    out = _run(_peer_leaves)
    assert out[1] == ("ok", "left")
    status, (result, elapsed) = out[0]
    assert status == "ok"
    assert result.startswith("error: ") and "communication failed" in result
    assert elapsed < 30


def _mismatched_sizes(rank, world):
    import bagua_core as bc

    comm = _comm(rank, world)
    backend = bc.BaguaCommBackendPy(10, -1)
    x = torch.ones(1024 if rank == 0 else 2048)
    t = bc.BaguaTensorPy(x, "x")
    b = bc.BaguaBucketPy("b", [t])
    b.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True)
    backend.register_ordered_buckets([b])
    backend.mark_communication_ready(t, 0)
    try:
        backend.wait_pending_comm_ops()
        r = "no error"
    except RuntimeError as e:
        r = "error"
    backend.close()
    return r


def test_mismatched_bucket_sizes_fail_instead_of_corrupting():
    out = _run(_mismatched_sizes)
    # every rank either raises or is taken down by the transport's own consistency check
    # (gloo aborts the process that receives a message of the wrong size); none may hang
    # or return as if the collective had worked
    assert len(out) == 2, out
    assert all(v == ("ok", "error") or v[0] == "died" for v in out.values()), out
    assert any(v == ("ok", "error") for v in out.values()), out


def _abort(rank, world):
    import bagua_core as bc

    comm = _comm(rank, world)
    x = torch.ones(16)
    t = bc.BaguaTensorPy(x, "x")
    comm.allreduce_inplace(t, 0)
    assert not comm.check_abort()
    comm.abort()
    assert comm.check_abort()
    with pytest.raises(RuntimeError, match="aborted"):
        comm.allreduce_inplace(t, 0)
    # the asynchronous op polls the flag and returns quietly, leaving the weights alone
    backend = bc.BaguaCommBackendPy(10, -1)
    w = torch.full((64,), float(rank))
    bw = bc.BaguaTensorPy(w, "w")
    b = bc.BaguaBucketPy("async", [bw])
    b.append_decentralized_asynchronous_op(comm, None, peer_selection_mode="all", torch_stream=0)
    backend.register_ordered_buckets([b])
    backend.mark_communication_ready(bw, 0)
    assert backend.wait_pending_comm_ops() == 1
    backend.close()
    return x.tolist()[0], w.tolist()[0]


def test_abort_stops_collectives_and_the_async_op():
    out = _run(_abort)
    for rank in (0, 1):
        status, (x0, w0) = out[rank]
        assert status == "ok", out[rank]
        assert x0 == 2.0 and w0 == float(rank)


def _rank_raises(rank, world):
    """A rank that raises before its collective: the other one gets an error within the
    process-group timeout."""
    import bagua_core as bc

    comm = _comm(rank, world)
    if rank == 1:
        raise ValueError("injected failure on rank 1")
    x = torch.ones(8)
    t0 = time.time()
    try:
        comm.allreduce_inplace(bc.BaguaTensorPy(x, "x"), 0)
        return "no error", time.time() - t0
    except RuntimeError as e:
        return "error", time.time() - t0


def test_rank_raising_is_seen_by_its_peer():
    out = _run(_rank_raises)
    assert out[1][0] == "error" and "injected failure" in out[1][1]
    status, (result, elapsed) = out[0]
    assert status == "ok" and result == "error" and elapsed < 40
