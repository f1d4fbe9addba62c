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


def _killed_mid_step(rank, world):
    """Rank 1 is killed (SIGKILL, no clean-up of any kind) while rank 0 is already inside the bucket's
    collective of the second step."""
    import signal

    import bagua_core as bc

    comm = _comm(rank, world)
    backend = bc.BaguaCommBackendPy(10, -1)
    t = bc.BaguaTensorPy(torch.ones(4096), "x")
    b = bc.BaguaBucketPy("b", [t])
    b.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True)
    backend.register_ordered_buckets([b])
    backend.mark_communication_ready(t, 0)
    assert backend.wait_pending_comm_ops() == 1
    if rank == 1:
        time.sleep(1.0)  # rank 0 is waiting for this rank's contribution by now
        os.kill(os.getpid(), signal.SIGKILL)
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


def test_rank_killed_while_its_peer_is_inside_the_collective():
    out = _run(_killed_mid_step)
    assert out[1][0] == "died", out
    status, (result, elapsed) = out[0]
    assert status == "ok", out[0]
    assert result.startswith("error: "), result
    assert elapsed < 30


def _delayed_past_watchdog(rank, world):
    """Rank 1 joins the bucket's collective three seconds late; rank 0's watchdog is set to half a
    second, so rank 0 hears about the stuck bucket by name while its worker is still waiting, and the
    collective itself completes once rank 1 arrives."""
    import bagua_core as bc

    comm = _comm(rank, world)
    backend = bc.BaguaCommBackendPy(10, -1)
    if rank == 0:
        backend.set_watchdog_timeout(0.5)
    x = torch.full((256,), float(rank + 1))
    t = bc.BaguaTensorPy(x, "x")
    b = bc.BaguaBucketPy("late_bucket", [t])
    b.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True)
    backend.register_ordered_buckets([b])
    if rank == 1:
        time.sleep(3.0)
    backend.mark_communication_ready(t, 0)
    report = ""
    t0 = time.time()
    try:
        backend.wait_pending_comm_ops()
    except RuntimeError as e:
        report = str(e)
    reported_after = time.time() - t0
    # the late rank arrives and the worker finishes the collective: after a watchdog report the op is
    # still owed to the caller, so a second wait returns it
    waited_again = backend.wait_pending_comm_ops() if report else 0
    backend.close()
    return report[:300], reported_after, x[0].item(), waited_again


def test_rank_delayed_past_the_watchdog_is_reported_by_bucket_name():
    out = _run(_delayed_past_watchdog)
    assert out[0][0] == "ok" and out[1][0] == "ok", out
    report0, after0, value0, again0 = out[0][1]
    report1, after1, value1, again1 = out[1][1]
    assert "watchdog" in report0 and "late_bucket" in report0, report0
    assert after0 < 2.5  # long before the late rank arrived
    assert report1 == "" and again0 == 1 and again1 == 0
    assert value0 == 1.5 and value1 == 1.5  # the collective still completed on both ranks


def test_corrupted_chunk_header_does_not_make_decompression_leave_its_buffers():
    """A compressed chunk whose header was overwritten (NaN, infinities, min > max) decompresses to
    meaningless values, but the call returns, stays inside the output tensor (poison on both sides is
    intact) and inside its pool blocks (guard regions intact)."""
    import struct

    import bagua_core as bc
    import bagua_core_b200 as bb

    C = bb._C
    was = C.pool_guard()
    C.pool_release_cached(-1)
    C.pool_set_guard(True)
    try:
        src = torch.randn(1000)
        c = bc.BaguaTensorPy(src, "src").compress("MinMaxUInt8", 4, -1)
        import ctypes

        stride = c.num_elements() // 4  # per chunk: 32-byte header {min, max, padding}, then the bytes
        first = struct.unpack("<ff", bytes((ctypes.c_char * 8).from_address(c.data_ptr())))
        assert first == (src[:250].min().item(), src[:250].max().item())
        for lo, hi in [(float("nan"), 1.0), (float("inf"), float("-inf")), (5.0, -5.0), (0.0, 0.0), (-3e38, 3e38)]:
            for chunk in range(4):
                header = (ctypes.c_char * 8).from_address(c.data_ptr() + chunk * stride)
                header[:] = struct.pack("<ff", lo, hi)
            whole = torch.full((1000 + 64,), -777.0)
            out = whole[32:1032]
            bc.BaguaTensorPy(out, "out").decompress_from("MinMaxUInt8", 4, c)
            assert torch.all(whole[:32] == -777.0) and torch.all(whole[1032:] == -777.0)
            assert C.pool_check_guards(-1) == 0
        del c
    finally:
        C.pool_release_cached(-1)
        C.pool_set_guard(was)
