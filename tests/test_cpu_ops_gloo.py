"""Multi-process CPU tests (gloo): every comm op of the engine against closed-form results.

Covers the reference's op semantics (bagua-core-internal/src/comm_ops/*.rs) on the host
transport; no GPU needed.
"""
import numpy as np
import pytest
import torch

from mp_util import run_ranks

SHAPES = [(1024, 1024), (4096,), (512, 256)]


def _make_comm(rank, world):
    import torch.distributed as dist

    import bagua_core as bc

    pg = dist.group.WORLD
    return bc.BaguaSingleCommunicatorPy(rank, world, -1, 0, "c10d:" + pg.group_name)


def _run_bucket(backend, bucket, tensors):
    backend.register_ordered_buckets([bucket])
    for t in tensors:
        backend.mark_communication_ready(t, 0)
    return backend.wait_pending_comm_ops()


def _config1(rank, world, flat):
    import bagua_core as bc

    g = torch.Generator().manual_seed(rank)
    if flat:
        total = sum(int(np.prod(s)) for s in SHAPES)
        storage = torch.empty(total)
        ts, off = [], 0
        for s in SHAPES:
            n = int(np.prod(s))
            v = storage[off:off + n].view(*s)
            v.copy_(torch.randn(*s, generator=g))
            ts.append(v)
            off += n
    else:
        ts = [torch.randn(*s, generator=g) for s in SHAPES]
    orig = [t.clone() for t in ts]
    comm = _make_comm(rank, world)
    backend = bc.BaguaCommBackendPy(100, -1)
    out = {}
    for algo in ("allreduce", "allreduce_sg", "bytegrad"):
        for t, o in zip(ts, orig):
            t.copy_(o)
        bts = [bc.BaguaTensorPy(t, f"{algo}_{i}") for i, t in enumerate(ts)]
        bucket = bc.BaguaBucketPy(f"bucket_{algo}", bts)
        if algo == "allreduce":
            bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True)
        elif algo == "allreduce_sg":
            bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True, scattergather=True)
        else:
            bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True,
                                                     scattergather=True, compression="MinMaxUInt8")
        n = _run_bucket(backend, bucket, bts)
        assert n == 1
        out[algo] = torch.cat([t.reshape(-1) for t in ts]).clone()
    out["orig"] = torch.cat([t.reshape(-1) for t in orig])
    backend.close()
    return out


@pytest.mark.parametrize("flat", [False, True])
def test_config1_allreduce_and_bytegrad(flat):
    world = 2
    res = run_ranks(_config1, world, args=(flat,))
    mean = sum(r["orig"] for r in res) / world
    for r in res:
        assert torch.equal(r["allreduce"], mean)  # exact: (a+b)/2 in fp32 either order
        assert torch.allclose(r["allreduce_sg"], mean, atol=0, rtol=0)
    # ByteGrad: per-chunk error bound 2*(max-min)/255 of the data that was quantised
    n = mean.numel()
    chunk = n // world
    for r in res:
        assert torch.equal(r["bytegrad"], res[0]["bytegrad"])  # all ranks agree bit for bit
        for c in range(world):
            sl = slice(c * chunk, (c + 1) * chunk)
            rng = max((x["orig"][sl].max() - x["orig"][sl].min()).item() for x in res)
            err = (r["bytegrad"][sl] - mean[sl]).abs().max().item()
            assert err <= 2 * rng / 255, (c, err, rng)


def _hier(rank, world):
    """hierarchical=True over (intranode = pairs, internode = leaders) equals the flat average."""
    import torch.distributed as dist

    import bagua_core as bc

    assert world == 4
    node = rank // 2
    intra_groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
    inter_group = dist.new_group([0, 2])
    intra = bc.BaguaSingleCommunicatorPy(rank % 2, 2, -1, 0, "c10d:" + intra_groups[node].group_name)
    inter = None
    if rank % 2 == 0:
        inter = bc.BaguaSingleCommunicatorPy(rank // 2, 2, -1, 0, "c10d:" + inter_group.group_name)
    g = torch.Generator().manual_seed(rank)
    x = torch.randn(4096, generator=g)
    orig = x.clone()
    bt = bc.BaguaTensorPy(x, "x")
    bucket = bc.BaguaBucketPy("b", [bt])
    bucket.append_centralized_synchronous_op(inter, intra, hierarchical=True, average=True)
    backend = bc.BaguaCommBackendPy(10, -1)
    _run_bucket(backend, bucket, [bt])
    backend.close()
    return orig, x.clone()


def test_hierarchical_equals_flat():
    res = run_ranks(_hier, 4)
    mean = sum(o for o, _ in res) / 4
    for _, x in res:
        assert torch.allclose(x, mean, atol=1e-6)


def _hier_single_node(rank, world, compression):
    """One node is the whole job: the intra-node communicator spans every rank, the inter-node one has
    one rank (the leader)."""
    import torch.distributed as dist

    import bagua_core as bc

    intra_group = dist.new_group(list(range(world)))
    inter_group = dist.new_group([0])
    intra = bc.BaguaSingleCommunicatorPy(rank, world, -1, 0, "c10d:" + intra_group.group_name)
    inter = bc.BaguaSingleCommunicatorPy(0, 1, -1, 0, "c10d:" + inter_group.group_name) if rank == 0 else None
    g = torch.Generator().manual_seed(rank)
    x = torch.randn(16 * world * 64, generator=g)
    orig = x.clone()
    bt = bc.BaguaTensorPy(x, "x")
    bucket = bc.BaguaBucketPy("b", [bt])
    bucket.append_centralized_synchronous_op(inter, intra, hierarchical=True, average=True, scattergather=True,
                                             compression=compression)
    backend = bc.BaguaCommBackendPy(10, -1)
    _run_bucket(backend, bucket, [bt])
    backend.close()
    return orig, x.clone()


@pytest.mark.parametrize("compression", [None, "MinMaxUInt8"])
def test_hierarchical_on_one_node_runs_flat_and_gives_the_two_level_result(monkeypatch, compression):
    """With one node, reduce-to-leader + leader's step + broadcast is replaced by one all-reduce and the
    leader's (one-rank, deterministic) step on every rank: bit-identical to the two-level path."""
    out = {}
    for flat in ("0", "1"):
        monkeypatch.setenv("BAGUA_B200_HIERARCHICAL_FLAT", flat)
        out[flat] = run_ranks(_hier_single_node, 3, args=(compression,))
    mean = sum(o for o, _ in out["1"]) / 3
    for r in range(3):
        assert torch.equal(out["0"][r][1], out["1"][r][1]), r
        assert torch.equal(out["1"][r][1], out["1"][0][1])
        tol = 1e-6 if compression is None else 2 * float(mean.max() - mean.min()) / 255
        assert (out["1"][r][1] - mean).abs().max().item() <= tol


def _decentralized(rank, world, mode, steps):
    import bagua_core as bc

    comm = _make_comm(rank, world)
    g = torch.Generator().manual_seed(rank)
    x = torch.randn(2048, generator=g)
    peer = torch.zeros_like(x)
    bx, bp = bc.BaguaTensorPy(x, "w"), bc.BaguaTensorPy(peer, "peer")
    bucket = bc.BaguaBucketPy("b", [bx])
    bucket.append_decentralized_synchronous_op(comm, None, hierarchical=False, peer_selection_mode=mode, peer_weight=bp)
    backend = bc.BaguaCommBackendPy(10, -1)
    hist = []
    for _ in range(steps):
        _run_bucket(backend, bucket, [bx])
        hist.append(peer.clone())
        x.copy_(peer)  # what the trainer does after the op
    state = bucket.ops_state()
    backend.close()
    return hist, state


@pytest.mark.parametrize("world", [2, 4])
def test_decentralized_shift_one(world):
    import bagua_core_b200 as b

    steps = 3
    res = run_ranks(_decentralized, world, args=("shift_one", steps))
    xs = [torch.randn(2048, generator=torch.Generator().manual_seed(r)) for r in range(world)]
    for s in range(steps):
        new = []
        for r in range(world):
            p = b._C.shift_one_peer(r, world, s)
            assert b._C.shift_one_peer(p, world, s) == r  # pairing is mutual
            new.append((xs[r] + xs[p]) / 2)
        for r in range(world):
            assert torch.allclose(res[r][0][s], new[r], atol=1e-6)
        xs = new
    assert res[0][1] == [[("step", steps)]]


def test_decentralized_all():
    res = run_ranks(_decentralized, 2, args=("all", 1))
    xs = [torch.randn(2048, generator=torch.Generator().manual_seed(r)) for r in range(2)]
    for r in range(2):
        assert torch.allclose(res[r][0][0], (xs[0] + xs[1]) / 2, atol=1e-6)


def _lp_ring(rank, world, steps):
    import bagua_core as bc

    comm = _make_comm(rank, world)
    n = 4096
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(n, generator=g)
    # replicas start equal to the true weights of self / left / right
    def init(r):
        return torch.randn(n, generator=torch.Generator().manual_seed(100 + r))

    w = init(rank)
    left = init((rank - 1) % world)
    right = init((rank + 1) % world)
    bx = bc.BaguaTensorPy(x, "x")
    bucket = bc.BaguaBucketPy("b", [bx])
    bucket.append_low_precision_decentralized_synchronous_op(
        comm, None, hierarchical=False, peer_selection_mode="ring", compression="MinMaxUInt8",
        weight=bc.BaguaTensorPy(w, "w"), left_peer_weight=bc.BaguaTensorPy(left, "l"),
        right_peer_weight=bc.BaguaTensorPy(right, "r"))
    backend = bc.BaguaCommBackendPy(10, -1)
    for s in range(steps):
        x.add_(0.01 * (s + 1))  # a local "optimizer step"
        _run_bucket(backend, bucket, [bx])
    backend.close()
    return x.clone(), w.clone(), left.clone(), right.clone()


@pytest.mark.parametrize("world", [2, 4])
def test_low_precision_ring(world):
    steps = 2
    res = run_ranks(_lp_ring, world, args=(steps,))
    for r in range(world):
        x, w, left, right = res[r]
        # after the op the bucket equals the rank's own replica ...
        assert torch.equal(x, w)
        # ... and the neighbours' replicas track the neighbours' weights exactly
        assert torch.allclose(left, res[(r - 1) % world][1], atol=1e-5)
        assert torch.allclose(right, res[(r + 1) % world][1], atol=1e-5)


def _async(rank, world):
    import bagua_core as bc

    comm = _make_comm(rank, world)
    x = torch.full((1000,), float(rank))
    bx = bc.BaguaTensorPy(x, "x")
    bucket = bc.BaguaBucketPy("b", [bx])
    bucket.append_decentralized_asynchronous_op(comm, None, peer_selection_mode="all", torch_stream=0)
    backend = bc.BaguaCommBackendPy(10, -1)
    _run_bucket(backend, bucket, [bx])
    backend.close()
    return x.clone()


def test_async_model_average():
    res = run_ranks(_async, 2)
    for x in res:
        assert torch.allclose(x, torch.full((1000,), 0.5))


def _collectives(rank, world):
    import bagua_core as bc

    comm = _make_comm(rank, world)
    T = lambda t, n="t": bc.BaguaTensorPy(t, n)  # noqa: E731
    out = {}
    a = torch.arange(8, dtype=torch.float32) + 10 * rank
    r = torch.zeros(8)
    comm.allreduce(T(a), T(r), 0)
    out["allreduce_sum"] = r.clone()
    b = a.clone()
    comm.allreduce_inplace(T(b), 10)
    out["allreduce_avg"] = b.clone()
    c = a.clone()
    comm.broadcast(T(c), 1)
    out["broadcast"] = c.clone()
    d = a.clone()
    comm.reduce_inplace(T(d), 0, 0)
    out["reduce"] = d.clone()
    e = a.clone()
    comm.alltoall_inplace(T(e))
    out["alltoall"] = e.clone()
    f = torch.zeros(8 * world)
    comm.allgather(T(a), T(f))
    out["allgather"] = f.clone()
    gsrc = a.clone()
    grecv = torch.zeros(8 // world)
    comm.reduce_scatter(T(gsrc), T(grecv), 0)
    out["reduce_scatter"] = grecv.clone()
    h = torch.zeros(8 * world) if rank == 0 else torch.zeros(1)
    comm.gather(T(a), T(h), 0)
    out["gather"] = h.clone()
    s_src = torch.arange(4 * world, dtype=torch.float32) if rank == 1 else torch.zeros(1)
    s_dst = torch.zeros(4)
    comm.scatter(T(s_src), T(s_dst), 1)
    out["scatter"] = s_dst.clone()
    # alltoall_v: rank r sends (p+1) elements to rank p
    sc = [p + 1 for p in range(world)]
    sd = [sum(sc[:p]) for p in range(world)]
    rc = [rank + 1] * world
    rd = [p * (rank + 1) for p in range(world)]
    sv = torch.arange(sum(sc), dtype=torch.float32) + 100 * rank
    rv = torch.zeros(sum(rc))
    comm.alltoall_v(T(sv), sc, sd, T(rv), rc, rd)
    out["alltoall_v"] = rv.clone()
    i64 = torch.arange(4, dtype=torch.int64) * (rank + 1)
    comm.allreduce_inplace(T(i64), 3)
    out["max_i64"] = i64.clone()
    u8 = torch.full((4,), rank + 1, dtype=torch.uint8)
    comm.allreduce_inplace(T(u8), 0)
    out["sum_u8"] = u8.clone()
    if rank == 0:
        comm.send(T(a), 1)
    else:
        z = torch.zeros(8)
        comm.recv(T(z), 0)
        out["recv"] = z.clone()
    # a root or peer outside the group is refused on the calling rank, before anything is sent
    refused = 0
    for call in (lambda: comm.broadcast(T(a.clone()), world), lambda: comm.reduce_inplace(T(a.clone()), -1, 0),
                 lambda: comm.gather_inplace(T(torch.zeros(8 * world)), 8, world + 3),
                 lambda: comm.scatter_inplace(T(torch.zeros(8 * world)), 8, -2),
                 lambda: comm.send(T(a.clone()), world), lambda: comm.recv(T(a.clone()), -1)):
        try:
            call()
        except RuntimeError as e:
            refused += "out of range" in str(e)
    out["refused"] = refused
    comm.barrier()
    return out


def test_collective_api():
    world = 2
    res = run_ranks(_collectives, world)
    base = torch.arange(8, dtype=torch.float32)
    a = [base + 10 * r for r in range(world)]
    for r in range(world):
        o = res[r]
        assert o["refused"] == 6
        assert torch.equal(o["allreduce_sum"], a[0] + a[1])
        assert torch.equal(o["allreduce_avg"], (a[0] + a[1]) / 2)
        assert torch.equal(o["broadcast"], a[1])
        assert torch.equal(o["allgather"], torch.cat(a))
        assert torch.equal(o["reduce_scatter"], (a[0] + a[1])[r * 4:(r + 1) * 4])
        assert torch.equal(o["alltoall"], torch.cat([a[p][r * 4:(r + 1) * 4] for p in range(world)]))
        assert torch.equal(o["scatter"], torch.arange(8, dtype=torch.float32)[r * 4:(r + 1) * 4])
        assert torch.equal(o["max_i64"], torch.arange(4, dtype=torch.int64) * 2)
        assert torch.equal(o["sum_u8"], torch.full((4,), 3, dtype=torch.uint8))
        expect_v = torch.cat([(torch.arange(3, dtype=torch.float32) + 100 * p)[sum(range(1, r + 1)):][:r + 1]
                              for p in range(world)])
        assert torch.equal(o["alltoall_v"], expect_v)
    assert torch.equal(res[0]["reduce"], a[0] + a[1])
    assert torch.equal(res[0]["gather"], torch.cat(a))
    assert torch.equal(res[1]["recv"], a[0])
