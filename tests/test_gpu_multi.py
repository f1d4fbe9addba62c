"""Multi-GPU tests (one process per GPU, NCCL bootstrap): the fused peer-memory kernels
against the library path that replays the reference's call sequence, and against plain
fp32 PyTorch math."""
import os

import pytest
import torch

from mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _world():
    return min(torch.cuda.device_count(), int(os.environ.get("BAGUA_TEST_WORLD", "8")))


def _mk_comm(rank, world, stream):
    import torch.distributed as dist

    import bagua_core as bc

    uid = [bc.BaguaSingleCommunicatorPy.generate_nccl_unique_id_str() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    return bc.BaguaSingleCommunicatorPy(rank, world, rank, stream.cuda_stream, uid[0])


def _gather_all(t):
    import torch.distributed as dist

    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t)
    return out


def _fused_allreduce(rank, world):
    # small one-shot limit so that the two-shot kernels are exercised at every world size
    os.environ["BAGUA_B200_ONESHOT_BYTES"] = "262144"
    import bagua_core as bc

    dev = torch.device("cuda", rank)
    stream = torch.cuda.Stream()
    comm = _mk_comm(rank, world, stream)
    assert comm.fused_available(), "peer arena must come up on an NVLink box"
    comm.set_device_wait_ms(20000.0)
    report = []
    sizes = [16, 4096, 65536 + 16, 1 << 20, (3 << 20) + 4096, 1 << 24]
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        for n in sizes:
            n = n // (8 if dt != torch.float32 else 4) * (8 if dt != torch.float32 else 4)
            g = torch.Generator().manual_seed(100 * rank + n % 97)
            x = torch.randn(n, generator=g).to(dt).to(dev)
            allx = _gather_all(x)
            ref_sum = torch.stack([a.float() for a in allx]).sum(0)
            # out of place, average
            out = torch.zeros_like(x)
            torch.cuda.synchronize()
            assert comm.fused_allreduce(bc.BaguaTensorPy(x, "s"), bc.BaguaTensorPy(out, "r"), True)
            stream.synchronize()
            comm.check_device_status()
            tol = {torch.float32: 1e-6, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dt]
            ref = ref_sum / world
            assert torch.allclose(out.float(), ref, rtol=tol, atol=tol * max(1.0, ref.abs().max().item())), (dt, n)
            # every rank holds the same bits
            outs = _gather_all(out)
            assert all(torch.equal(outs[0], o) for o in outs)
            # in place, sum
            y = x.clone()
            torch.cuda.synchronize()
            bt = bc.BaguaTensorPy(y, "y")
            assert comm.fused_allreduce(bt, bt, False)
            stream.synchronize()
            assert torch.allclose(y.float(), ref_sum, rtol=tol, atol=tol * max(1.0, ref_sum.abs().max().item()))
            report.append((str(dt), n))
    # symmetric memory: in-place two-shot with direct peer loads/stores, no staging
    for dt in (torch.float32, torch.bfloat16):
        n = (24 << 20) + 4096
        sym = comm.alloc_symmetric(n, dt)
        assert sym is not None and comm.is_symmetric(sym)
        g = torch.Generator().manual_seed(500 + rank)
        sym.copy_(torch.randn(n, generator=g).to(dt))
        allx = _gather_all(sym.clone())
        ref = torch.stack([a.float() for a in allx]).mean(0)
        torch.cuda.synchronize()
        bt = bc.BaguaTensorPy(sym, "sym")
        for rep in range(2):  # second pass averages identical values: result must not change
            assert comm.fused_allreduce(bt, bt, True)
            stream.synchronize()
            comm.check_device_status()
            tol = 1e-6 if dt == torch.float32 else 1.6e-2
            assert torch.allclose(sym.float(), ref, rtol=tol, atol=tol * max(1.0, ref.abs().max().item())), (dt, rep)
            outs = _gather_all(sym.clone())
            assert all(torch.equal(outs[0], o) for o in outs)
        # the same bucket through the bulk-copy (TMA) variant of the kernel: bit-identical result
        if world in (2, 4, 8):
            import bagua_core_b200 as bb

            first = sym.clone()
            sym.copy_(allx[rank])
            torch.cuda.synchronize()
            torch.distributed.barrier()
            before = dict(bb._C.get_tuning())
            bb._C.set_tuning("tma_min_bytes", 1 << 20)
            bb._C.set_tuning("tma_isolated", 1)
            try:
                assert comm.fused_allreduce(bt, bt, True)
                stream.synchronize()
                comm.check_device_status()
            finally:
                bb._C.set_tuning("tma_min_bytes", before["tma_min_bytes"])
                bb._C.set_tuning("tma_isolated", before["tma_isolated"])
            assert torch.equal(sym, first), dt
        # ... and with the bytes moved by the copy engines
        sym.copy_(allx[rank])
        torch.cuda.synchronize()
        torch.distributed.barrier()
        assert comm.fused_allreduce_ce(bt, bt, True)
        stream.synchronize()
        comm.check_device_status()
        if world in (2, 4, 8):
            assert torch.equal(sym, first), dt
        tol = 1e-6 if dt == torch.float32 else 1.6e-2
        assert torch.allclose(sym.float(), ref, rtol=tol, atol=tol * max(1.0, ref.abs().max().item())), dt
        # out of place into a second symmetric buffer, sum
        out2 = comm.alloc_symmetric(n, dt)
        sym.copy_(allx[rank])
        torch.cuda.synchronize()
        torch.distributed.barrier()
        assert comm.fused_allreduce_ce(bt, bc.BaguaTensorPy(out2, "o2"), False)
        stream.synchronize()
        comm.check_device_status()
        assert torch.equal(sym, allx[rank])
        assert torch.allclose(out2.float(), ref * world, rtol=tol, atol=tol * world * max(1.0, ref.abs().max().item())), dt
    # back-to-back ops of different sizes without host sync in between (staging reuse protocol)
    xs = [torch.full((s,), float(rank + 1), device=dev) for s in (1 << 12, 1 << 22, 1 << 14, 1 << 21, 64)]
    torch.cuda.synchronize()
    for _ in range(5):
        for x in xs:
            bt = bc.BaguaTensorPy(x, "x")
            assert comm.fused_allreduce(bt, bt, True)
    stream.synchronize()
    comm.check_device_status()
    expect = sum(range(1, world + 1)) / world
    for x in xs:
        assert torch.allclose(x, torch.full_like(x, expect)), x[:4]
    return len(report), comm.fused_launches()


def test_fused_allreduce_matches_fp32_sum():
    world = _world()
    res = run_ranks(_fused_allreduce, world, backend="nccl", timeout=600)
    assert all(r[0] == 18 for r in res)
    assert all(r[1] > 0 for r in res)


def _bucket_ops(rank, world):
    """Each op: fused path vs library path on identical inputs."""
    import bagua_core as bc
    import bagua_core_b200 as bb

    dev = torch.device("cuda", rank)
    stream = torch.cuda.Stream()
    comm = _mk_comm(rank, world, stream)
    assert comm.fused_available()
    comm.set_device_wait_ms(20000.0)
    backend = bc.BaguaCommBackendPy(10, rank)

    def run(bucket, tensors):
        backend.register_ordered_buckets([bucket])
        events = []
        for t in tensors:
            ev = torch.cuda.Event()
            ev.record()
            events.append(ev)
            backend.mark_communication_ready(t, ev.cuda_event)
        backend.wait_pending_comm_ops()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        comm.check_device_status()

    n = 16 * world * 4099  # odd multiple: exercises uneven block slices
    for dt in (torch.float32, torch.float16):
        g = torch.Generator().manual_seed(7 + rank)
        base = torch.randn(n, generator=g).to(dt).to(dev)
        allb = _gather_all(base)
        mean = torch.stack([a.float() for a in allb]).mean(0)
        tol = 1e-6 if dt == torch.float32 else 2e-3

        # O1
        outs = {}
        for fused in (True, False):
            comm.set_fused(fused)
            x = base.clone()
            bt = bc.BaguaTensorPy(x, "g")
            b = bc.BaguaBucketPy("o1", [bt])
            b.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True, scattergather=not fused)
            run(b, [bt])
            outs[fused] = x
            assert torch.allclose(x.float(), mean, rtol=tol, atol=tol * 4), ("o1", dt, fused)
        # O2 ByteGrad
        for fused in (True, False):
            comm.set_fused(fused)
            x = base.clone()
            bt = bc.BaguaTensorPy(x, "g")
            b = bc.BaguaBucketPy("o2", [bt])
            b.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True, scattergather=True,
                                                compression="MinMaxUInt8")
            run(b, [bt])
            outs[("bg", fused)] = x
            chunk = n // world
            for c in range(world):
                sl = slice(c * chunk, (c + 1) * chunk)
                rng = max((a[sl].float().max() - a[sl].float().min()).item() for a in allb)
                err = (x[sl].float() - mean[sl]).abs().max().item()
                assert err <= 2 * rng / 255 + tol * 8, ("o2", dt, fused, c, err, rng)
            same = _gather_all(x)
            assert all(torch.equal(same[0], s) for s in same), "ranks disagree after ByteGrad"
        # fused and library ByteGrad quantise the same grid: results agree up to rounding ties
        d = (outs[("bg", True)].float() - outs[("bg", False)].float()).abs()
        rng_all = (mean.max() - mean.min()).item()
        assert d.max().item() <= 2.1 * rng_all / 255 and (d > 1e-3 * rng_all).float().mean().item() < 0.02

        # O3 shift_one, 3 steps
        if world % 2 == 0:
            for fused in (True, False):
                comm.set_fused(fused)
                x = base.clone()
                peer = torch.zeros_like(x)
                bt = bc.BaguaTensorPy(x, "w")
                b = bc.BaguaBucketPy("o3", [bt])
                b.append_decentralized_synchronous_op(comm, None, hierarchical=False,
                                                      peer_selection_mode="shift_one",
                                                      peer_weight=bc.BaguaTensorPy(peer, "p"))
                cur = [a.float() for a in allb]
                for step in range(3):
                    run(b, [bt])
                    p = bb._C.shift_one_peer(rank, world, step)
                    exp = (cur[rank] + cur[p]) / 2
                    assert torch.allclose(peer.float(), exp, rtol=tol, atol=tol * 4), ("o3", dt, fused, step)
                    cur = [(cur[r] + cur[bb._C.shift_one_peer(r, world, step)]) / 2 for r in range(world)]
                    if dt != torch.float32:
                        cur = [c.to(dt).float() for c in cur]
                    x.copy_(peer)
        # O3 all
        comm.set_fused(True)
        x = base.clone()
        peer = torch.zeros_like(x)
        bt = bc.BaguaTensorPy(x, "w")
        b = bc.BaguaBucketPy("o3a", [bt])
        b.append_decentralized_synchronous_op(comm, None, hierarchical=False, peer_selection_mode="all",
                                              peer_weight=bc.BaguaTensorPy(peer, "p"))
        run(b, [bt])
        assert torch.allclose(peer.float(), mean, rtol=tol, atol=tol * 4)
        assert torch.equal(x, base)

        # O4 low-precision ring: fused vs library, two steps
        lp = {}
        for fused in (True, False):
            comm.set_fused(fused)
            x = base.clone()
            w = allb[rank].clone()
            left = allb[(rank - 1) % world].clone()
            right = allb[(rank + 1) % world].clone()
            bt = bc.BaguaTensorPy(x, "x")
            b = bc.BaguaBucketPy("o4", [bt])
            b.append_low_precision_decentralized_synchronous_op(
                comm, None, hierarchical=False, peer_selection_mode="ring", compression="MinMaxUInt8",
                weight=bc.BaguaTensorPy(w, "w"), left_peer_weight=bc.BaguaTensorPy(left, "l"),
                right_peer_weight=bc.BaguaTensorPy(right, "r"))
            for step in range(2):
                x.add_(0.01)
                run(b, [bt])
            assert torch.equal(x, w)
            ws = _gather_all(w)
            atol = 1e-5 if dt == torch.float32 else 2e-2
            assert torch.allclose(left.float(), ws[(rank - 1) % world].float(), atol=atol)
            assert torch.allclose(right.float(), ws[(rank + 1) % world].float(), atol=atol)
            lp[fused] = x.clone()
        dd = (lp[True].float() - lp[False].float()).abs().max().item()
        assert dd <= 0.05, dd

    # O5 async (fp32 only)
    comm.set_fused(True)
    x = torch.full((1 << 16,), float(rank), device=dev)
    bt = bc.BaguaTensorPy(x, "x")
    b = bc.BaguaBucketPy("o5", [bt])
    b.append_decentralized_asynchronous_op(comm, None, peer_selection_mode="all",
                                           torch_stream=torch.cuda.current_stream().cuda_stream)
    run(b, [bt])
    assert torch.allclose(x, torch.full_like(x, (world - 1) / 2))
    stats = bb._C.stats()
    backend.close()
    return stats["fused_launches"], stats["library_fallbacks"]


def test_bucket_ops_fused_vs_library():
    world = _world()
    res = run_ranks(_bucket_ops, world, backend="nccl", timeout=900)
    for fused, fallbacks in res:
        assert fused >= 10
        assert fallbacks == 0


def _train(rank, world, algo_name):
    import time

    import bagua_core_b200 as bb
    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import MLP

    dev = torch.device("cuda", rank)
    torch.manual_seed(3)
    model = MLP(64, 256, 10, depth=3).to(dev)
    pg = P.init_process_group(dev)
    steps = 6
    if algo_name == "qadam":
        opt = P.QAdamOptimizer(model.parameters(), lr=0.01, warmup_steps=2, eps=1e-2)
        algo = P.QAdamAlgorithm(opt)
    elif algo_name == "async":
        opt = P.FlatSGD(model.parameters(), lr=0.01, momentum=0.9)
        algo = P.AsyncModelAverageAlgorithm(sync_interval_ms=5)
        steps = 40
    else:
        opt = P.FlatSGD(model.parameters(), lr=0.05, momentum=0.9)
        algo = {"allreduce": P.GradientAllReduceAlgorithm, "bytegrad": P.ByteGradAlgorithm,
                "allreduce_hier": lambda: P.GradientAllReduceAlgorithm(hierarchical=True),
                "bytegrad_hier": lambda: P.ByteGradAlgorithm(hierarchical=True)}[algo_name]()
    bm = P.with_bagua(model, [opt], algo, bucket_bytes=64 * 1024)
    g = torch.Generator().manual_seed(11)
    xs = torch.randn(6, world * 16, 64, generator=g)
    ys = torch.randn(6, world * 16, 10, generator=g)
    losses = []
    for s in range(steps):
        x = xs[s % 6, rank * 16:(rank + 1) * 16].to(dev)
        y = ys[s % 6, rank * 16:(rank + 1) * 16].to(dev)
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(bm(x), y)
        loss.backward()
        opt.step()
        losses.append(float(loss.item()))
        if algo_name == "async":
            time.sleep(0.005)  # let a few averaging rounds land between steps
    extra = {}
    with torch.no_grad():  # the loss on the first batch again, to compare with losses[0]
        x0 = xs[0, rank * 16:(rank + 1) * 16].to(dev)
        y0 = ys[0, rank * 16:(rank + 1) * 16].to(dev)
        extra["final_loss_first_batch"] = float(torch.nn.functional.mse_loss(model(x0), y0).item())
    if algo_name == "async":
        algo.abort(bm)  # returns once no averaging round is in flight
        extra["rounds"] = algo.rounds
    if algo_name == "qadam":
        extra["compressed"] = bool(bm.bagua_state_dict()["algorithm"]["compressed"])
    if algo_name.endswith("_hier"):
        extra["single_node"] = pg.intra_comm is not None and pg.intra_comm.nranks() == world
    torch.cuda.synchronize()
    pg.global_comm.check_device_status()
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()]).cpu()
    fused = bb._C.stats()["fused_launches"]
    P.destroy_process_group()
    return flat, fused, losses, extra


def _reference_weights(world):
    from bagua_core_b200.models import MLP

    torch.manual_seed(3)
    model = MLP(64, 256, 10, depth=3)
    opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    g = torch.Generator().manual_seed(11)
    xs = torch.randn(6, world * 16, 64, generator=g)
    ys = torch.randn(6, world * 16, 10, generator=g)
    for s in range(6):
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(xs[s]), ys[s]).backward()
        opt.step()
    return torch.cat([p.detach().reshape(-1) for p in model.parameters()])


@pytest.mark.parametrize("algo", ["allreduce", "bytegrad", "allreduce_hier", "bytegrad_hier"])
def test_with_bagua_training_multi_gpu(algo):
    world = _world()
    res = run_ranks(_train, world, backend="nccl", args=(algo,), timeout=600)
    ref = _reference_weights(world)
    for flat, fused, _losses, extra in res:
        assert fused > 0, "training must run on the fused kernels"
        assert torch.equal(flat, res[0][0])
        tol = 2e-4 if algo.startswith("allreduce") else 5e-2
        assert (flat - ref).abs().max().item() < tol
        if algo.endswith("_hier"):
            assert extra["single_node"], "one box: the hierarchical communicator must have gone flat"


def test_hierarchical_allreduce_equals_flat_on_one_box():
    """`hierarchical=True` on one NVSwitch box runs the same fused all-reduce as the flat algorithm:
    the trained weights are bit-identical."""
    world = _world()
    flat = run_ranks(_train, world, backend="nccl", args=("allreduce",), timeout=600)
    hier = run_ranks(_train, world, backend="nccl", args=("allreduce_hier",), timeout=600)
    assert torch.equal(flat[0][0], hier[0][0])
    assert hier[0][1] > 0


def test_qadam_trains_on_gpus_and_switches_to_compressed_momentum():
    world = _world()
    res = run_ranks(_train, world, backend="nccl", args=("qadam",), timeout=600)
    for flat, fused, losses, extra in res:
        assert extra["compressed"], "after the warm-up the momentum buckets are exchanged compressed"
        assert fused > 0
        assert torch.isfinite(flat).all()
        assert torch.equal(flat, res[0][0]), "every rank applies the same averaged momentum"
        assert extra["final_loss_first_batch"] < losses[0]


def test_async_model_average_on_gpus_keeps_replicas_together():
    world = _world()
    res = run_ranks(_train, world, backend="nccl", args=("async",), timeout=600)
    ref = res[0][0]
    for flat, fused, losses, extra in res:
        assert extra["rounds"] > 0 and fused > 0
        assert torch.isfinite(flat).all()
        # replicas train on different data and are pulled together by the background averaging
        assert (flat - ref).abs().max().item() < 0.2
        assert extra["final_loss_first_batch"] < losses[0]


def _sym_pair(rank, world):
    """shift_one gossip on weights that live in the symmetric heap: partners read each other's
    bucket directly."""
    import bagua_core as bc
    import bagua_core_b200 as bb

    dev = torch.device("cuda", rank)
    stream = torch.cuda.Stream()
    comm = _mk_comm(rank, world, stream)
    assert comm.fused_available()
    comm.set_device_wait_ms(20000.0)
    backend = bc.BaguaCommBackendPy(10, rank)
    bb._C.set_tuning("pair_sym_min_bytes", 256 << 10)  # so that this bucket takes the direct-load kernel
    n = 16 * world * 8209
    x = comm.alloc_symmetric(n, torch.float32)
    assert x is not None and comm.is_symmetric(x)
    g = torch.Generator().manual_seed(40 + rank)
    x.copy_(torch.randn(n, generator=g))
    allx = [a.clone() for a in _gather_all(x.clone())]
    peer = torch.zeros_like(x)
    bt = bc.BaguaTensorPy(x, "w")
    b = bc.BaguaBucketPy("sym_gossip", [bt])
    b.append_decentralized_synchronous_op(comm, None, hierarchical=False, peer_selection_mode="shift_one",
                                          peer_weight=bc.BaguaTensorPy(peer, "p"))
    backend.register_ordered_buckets([b])
    cur = allx
    for step in range(3):
        ev = torch.cuda.Event()
        ev.record()
        backend.mark_communication_ready(bt, ev.cuda_event)
        backend.wait_pending_comm_ops()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        comm.check_device_status()
        p = bb._C.shift_one_peer(rank, world, step)
        assert torch.allclose(peer, (cur[rank] + cur[p]) / 2, atol=1e-6), step
        cur = [(cur[r] + cur[bb._C.shift_one_peer(r, world, step)]) / 2 for r in range(world)]
        x.copy_(peer)
        torch.cuda.synchronize()
        torch.distributed.barrier()
    launches = comm.fused_launches()
    backend.close()
    return launches


def test_symmetric_pair_average():
    world = _world()
    if world % 2:
        pytest.skip("shift_one needs an even number of ranks")
    res = run_ranks(_sym_pair, world, backend="nccl", timeout=300)
    assert all(r == 3 for r in res)
