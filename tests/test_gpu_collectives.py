"""Peer-memory kernels for the communicator's own collectives (all-gather, all-to-all,
reduce-scatter, broadcast, reduce, gather, scatter, barrier): on one GPU through the single-launch emulation, and
on several GPUs against the library (NCCL) results.

Their signalling and index arithmetic are also covered on the CPU by
tests/test_cpu_protocol_model.py and tests/test_cpu_device_emulation.py."""
import os

import pytest
import torch

from mp_util import run_ranks

pytestmark = [pytest.mark.gpu]


def _arena(n, staging_mb=64):
    import bagua_core_b200 as bb

    a = bb._C.EmulatedArena(n, 0, staging_mb << 20)
    a.set_deadline_ms(5000.0)
    return a


def _rand(n, dt, seed):
    return torch.randn(n, generator=torch.Generator().manual_seed(seed)).to(dt).cuda()


CASES = [(16, 1), (4096 + 16, 3), (1 << 18, 8)]  # (elements per chunk, blocks per rank)


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("symmetric", [False, True])
def test_emulated_allgather(nranks, symmetric):
    arena = _arena(nranks)
    for chunk, blocks in CASES:
        xs = [_rand(chunk, torch.float32, 10 * chunk + r) for r in range(nranks)]
        outs = [torch.zeros(chunk * nranks, device="cuda") for _ in range(nranks)]
        arena.collective("allgather", xs, outs, symmetric=symmetric, blocks=blocks)
        ref = torch.cat(xs)
        for o in outs:
            assert torch.equal(o, ref)
        # in place: rank r's contribution already sits in chunk r of its buffer
        bufs = [torch.zeros(chunk * nranks, device="cuda") for _ in range(nranks)]
        for r in range(nranks):
            bufs[r][r * chunk:(r + 1) * chunk] = xs[r]
        views = [bufs[r][r * chunk:(r + 1) * chunk] for r in range(nranks)]
        arena.collective("allgather", views, bufs, symmetric=symmetric, blocks=blocks)
        for b in bufs:
            assert torch.equal(b, ref)


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("symmetric", [False, True])
def test_emulated_alltoall(nranks, symmetric):
    arena = _arena(nranks)
    for chunk, blocks in CASES:
        xs = [_rand(chunk * nranks, torch.float16, 7 * chunk + r) for r in range(nranks)]
        outs = [torch.zeros_like(x) for x in xs]
        arena.collective("alltoall", xs, outs, symmetric=symmetric, blocks=blocks)
        for r in range(nranks):
            ref = torch.cat([xs[q][r * chunk:(r + 1) * chunk] for q in range(nranks)])
            assert torch.equal(outs[r], ref)
    # in place goes through staging
    chunk = 4096
    xs = [_rand(chunk * nranks, torch.float32, 99 + r) for r in range(nranks)]
    ys = [x.clone() for x in xs]
    arena.collective("alltoall", ys, ys, blocks=4)
    for r in range(nranks):
        assert torch.equal(ys[r], torch.cat([xs[q][r * chunk:(r + 1) * chunk] for q in range(nranks)]))
    with pytest.raises(RuntimeError, match="in-place"):
        arena.collective("alltoall", ys, ys, symmetric=True, blocks=4)


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("unit", [16, 4, 1])
def test_emulated_alltoall_v(nranks, unit):
    """Per-pair sizes in multiples of `unit` bytes (16: whole vectors; 4 and 1: the narrower copy paths),
    some of them zero; receivers pull their segments out of the senders' buffers."""
    arena = _arena(nranks)
    for scale in (1, 300):
        table = [unit * scale * ((3 * s + 5 * d + scale) % 7) for s in range(nranks) for d in range(nranks)]
        sent = [sum(table[s * nranks:(s + 1) * nranks]) for s in range(nranks)]
        received = [sum(table[s * nranks + d] for s in range(nranks)) for d in range(nranks)]
        g = torch.Generator().manual_seed(scale + unit)
        xs = [torch.randint(0, 256, (max(sent[r], 16),), generator=g, dtype=torch.uint8).cuda() for r in range(nranks)]
        outs = [torch.full((received[r] + 32,), 7, dtype=torch.uint8, device="cuda") for r in range(nranks)]
        arena.alltoall_v(xs, outs, table)
        for d in range(nranks):
            parts = []
            for s in range(nranks):
                start = sum(table[s * nranks:s * nranks + d])
                parts.append(xs[s][start:start + table[s * nranks + d]])
            ref = torch.cat(parts)
            assert torch.equal(outs[d][:received[d]], ref), (nranks, unit, scale, d)
            assert torch.all(outs[d][received[d]:] == 7)  # nothing behind the last segment was touched


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("symmetric", [False, True])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_emulated_reduce_scatter(nranks, symmetric, dt):
    arena = _arena(nranks)
    tol = 1e-6 if dt == torch.float32 else 1.6e-2
    for chunk, blocks in CASES:
        xs = [_rand(chunk * nranks, dt, 3 * chunk + r) for r in range(nranks)]
        total = torch.stack([x.float() for x in xs]).sum(0)
        outs = [torch.zeros(chunk, dtype=dt, device="cuda") for _ in range(nranks)]
        arena.collective("reduce_scatter", xs, outs, symmetric=symmetric, average=True, blocks=blocks)
        for r in range(nranks):
            ref = total[r * chunk:(r + 1) * chunk] / nranks
            assert torch.allclose(outs[r].float(), ref, rtol=tol, atol=tol * max(1.0, ref.abs().max().item()))
        # in place (sum): the result replaces chunk r of rank r's input
        ys = [x.clone() for x in xs]
        views = [ys[r][r * chunk:(r + 1) * chunk] for r in range(nranks)]
        arena.collective("reduce_scatter", ys, views, symmetric=symmetric, blocks=blocks)
        for r in range(nranks):
            ref = total[r * chunk:(r + 1) * chunk]
            assert torch.allclose(views[r].float(), ref, rtol=tol, atol=tol * max(1.0, ref.abs().max().item()))


@pytest.mark.parametrize("nranks", [2, 3, 8])
@pytest.mark.parametrize("kind", ["broadcast_direct", "broadcast_twophase"])
def test_emulated_broadcast(nranks, kind):
    arena = _arena(nranks)
    for n, blocks in [(4, 1), (4096 + 4, 3), (1 << 20, 8)]:
        for root in {0, nranks - 1, nranks // 2}:
            bufs = [_rand(n, torch.float32, 5 * n + r) for r in range(nranks)]
            ref = bufs[root].clone()
            arena.collective(kind, [], bufs, root=root, blocks=blocks)
            for b in bufs:
                assert torch.equal(b, ref)


@pytest.mark.parametrize("nranks", [2, 3, 8])
def test_emulated_scatter_and_gather(nranks):
    arena = _arena(nranks)
    for chunk, blocks in CASES:
        for root in {0, nranks - 1}:
            big = [_rand(chunk * nranks, torch.float32, 13 * chunk + r) for r in range(nranks)]
            outs = [torch.zeros(chunk, device="cuda") for _ in range(nranks)]
            arena.collective("scatter", big, outs, root=root, blocks=blocks)
            for r in range(nranks):
                assert torch.equal(outs[r], big[root][r * chunk:(r + 1) * chunk])
            # gather them back into a fresh buffer on the root; other ranks' outputs stay as they were
            back = [torch.full((chunk * nranks,), -1.0, device="cuda") for _ in range(nranks)]
            arena.collective("gather", outs, back, root=root, blocks=blocks)
            assert torch.equal(back[root], big[root])
            for r in range(nranks):
                if r != root:
                    assert torch.equal(back[r], torch.full_like(back[r], -1.0))
            # in-place forms on the root
            ys = [b.clone() for b in big]
            views = [ys[r][r * chunk:(r + 1) * chunk] if r == root else torch.zeros(chunk, device="cuda")
                     for r in range(nranks)]
            arena.collective("scatter", ys, views, root=root, blocks=blocks)
            for r in range(nranks):
                assert torch.equal(views[r], big[root][r * chunk:(r + 1) * chunk])
            arena.collective("gather", views, ys, root=root, blocks=blocks)
            assert torch.equal(ys[root], big[root])


@pytest.mark.parametrize("nranks", [2, 3, 8])
@pytest.mark.parametrize("kind", ["reduce_direct", "reduce_twophase"])
@pytest.mark.parametrize("dt", [torch.float32, torch.float16])
def test_emulated_reduce(nranks, kind, dt):
    arena = _arena(nranks)
    tol = 1e-6 if dt == torch.float32 else 2e-3
    for n, blocks in [(8, 1), (4096 + 8, 3), (1 << 20, 8)]:
        root = n % nranks
        xs = [_rand(n, dt, 17 * n + r) for r in range(nranks)]
        ref = torch.stack([x.float() for x in xs]).mean(0)
        outs = [torch.full((n,), 7.0, dtype=dt, device="cuda") for _ in range(nranks)]
        arena.collective(kind, xs, outs, root=root, average=True, blocks=blocks)
        assert torch.allclose(outs[root].float(), ref, rtol=tol, atol=tol * max(1.0, ref.abs().max().item()))
        for r in range(nranks):
            if r != root:
                assert torch.equal(outs[r], torch.full_like(outs[r], 7.0))
        # in place: only the root's buffer changes
        ys = [x.clone() for x in xs]
        arena.collective(kind, ys, ys, root=root, blocks=blocks)
        assert torch.allclose(ys[root].float(), ref * nranks, rtol=tol, atol=tol * nranks * max(1.0, ref.abs().max().item()))
        for r in range(nranks):
            if r != root:
                assert torch.equal(ys[r], xs[r])


def test_emulated_collectives_interleaved_with_allreduce():
    """Different kernels back to back over the same staging and signal words."""
    nranks = 4
    arena = _arena(nranks)
    arena.collective("barrier", [], [])
    for rep in range(3):
        xs = [torch.full((1 << 14,), float(r + 1), device="cuda") for r in range(nranks)]
        arena.allreduce(xs, xs, True, "twoshot", 4)
        assert all(torch.allclose(x, torch.full_like(x, 2.5)) for x in xs)
        outs = [torch.zeros(nranks << 14, device="cuda") for _ in range(nranks)]
        arena.collective("allgather", xs, outs, blocks=3)
        assert all(torch.allclose(o, torch.full_like(o, 2.5)) for o in outs)
        arena.collective("barrier", [], [])
        bufs = [torch.full((1 << 16,), float(r), device="cuda") for r in range(nranks)]
        arena.collective("broadcast_twophase", [], bufs, root=2, blocks=5)
        assert all(torch.equal(b, torch.full_like(b, 2.0)) for b in bufs)
        rs = [torch.zeros(1 << 14, device="cuda") for _ in range(nranks)]
        arena.collective("reduce_scatter", bufs, rs, symmetric=(rep % 2 == 1), blocks=2)
        assert all(torch.equal(o, torch.full_like(o, 8.0)) for o in rs)
        arena.allreduce(xs, xs, False, "oneshot", 2)
        assert all(torch.allclose(x, torch.full_like(x, 10.0)) for x in xs)


# ---- several GPUs: peer-memory kernels against the library results -------------------------

def _mk_comm(rank, world, stream):
    import torch.distributed as dist

    import bagua_core as bc

    uid = [bc.BaguaSingleCommunicatorPy.generate_nccl_unique_id_str() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    return bc.BaguaSingleCommunicatorPy(rank, world, rank, stream.cuda_stream, uid[0])


def _p2p_vs_library(rank, world):
    import bagua_core as bc

    dev = torch.device("cuda", rank)
    stream = torch.cuda.Stream()
    comm = _mk_comm(rank, world, stream)
    assert comm.fused_available()
    comm.set_device_wait_ms(20000.0)
    T = bc.BaguaTensorPy
    checked = 0

    def both(fn):
        """Runs fn(comm) with library collectives, then with peer-memory kernels; returns both results."""
        out = []
        for p2p in (False, True):
            comm.set_p2p_collectives(p2p)
            before = comm.fused_launches()
            torch.cuda.synchronize()
            # buffers are made and filled on the communicator's stream: allocation, fill, collective
            # and any view taken of the result are then ordered with one another
            with torch.cuda.stream(stream):
                res = fn()
            stream.synchronize()
            comm.check_device_status()
            assert (comm.fused_launches() > before) == p2p
            out.append(res)
        comm.set_p2p_collectives(False)
        return out

    for chunk in (16, 4096 + 16, 1 << 20):
        g = torch.Generator().manual_seed(1000 * rank + chunk % 89)
        x = torch.randn(chunk, generator=g).to(dev)
        big = torch.randn(chunk * world, generator=g).to(dev)

        def allgather():
            out = torch.zeros(chunk * world, device=dev)
            comm.allgather(T(x, "s"), T(out, "r"))
            return out

        def allgather_inplace():
            buf = torch.zeros(chunk * world, device=dev)
            buf[rank * chunk:(rank + 1) * chunk] = x
            torch.cuda.synchronize()
            comm.allgather_inplace(T(buf, "b"))
            return buf

        def alltoall():
            out = torch.zeros_like(big)
            comm.alltoall(T(big, "s"), T(out, "r"))
            return out

        def alltoall_inplace():
            buf = big.clone()
            torch.cuda.synchronize()
            comm.alltoall_inplace(T(buf, "b"))
            return buf

        def reduce_scatter():
            out = torch.zeros(chunk, device=dev)
            comm.reduce_scatter(T(big, "s"), T(out, "r"), 10)
            return out

        def reduce_scatter_inplace():
            buf = big.clone()
            torch.cuda.synchronize()
            comm.reduce_scatter_inplace(T(buf, "b"), 0)
            return buf[rank * chunk:(rank + 1) * chunk]  # a view: read only after the caller has synchronised

        def broadcast():
            buf = big.clone()
            torch.cuda.synchronize()
            comm.broadcast(T(buf, "b"), world - 1)
            return buf

        def allreduce():
            buf = big.clone()
            torch.cuda.synchronize()
            comm.allreduce_inplace(T(buf, "b"), 10)
            return buf

        def gather():
            out = torch.full((chunk * world,), -1.0, device=dev)
            comm.gather(T(x, "s"), T(out, "r"), world - 1)
            return out if rank == world - 1 else torch.zeros(1, device=dev)

        def scatter():
            out = torch.zeros(chunk, device=dev)
            comm.scatter(T(big, "s"), T(out, "r"), 0)
            return out

        def reduce():
            buf = big.clone()
            torch.cuda.synchronize()
            comm.reduce_inplace(T(buf, "b"), 1 % world, 0)
            return buf

        for fn in (gather, scatter):
            lib, p2p = both(fn)
            assert torch.equal(lib, p2p), (fn.__name__, chunk)
            checked += 1
        lib, p2p = both(reduce)
        if rank == 1 % world:
            assert torch.allclose(lib, p2p, rtol=1e-5, atol=1e-5), ("reduce", chunk)
        else:
            assert torch.equal(p2p, big)  # only the root's buffer changes
        checked += 1

        for fn in (allgather, allgather_inplace, alltoall, alltoall_inplace, broadcast):
            lib, p2p = both(fn)
            assert torch.equal(lib, p2p), (fn.__name__, chunk)
            checked += 1
        for fn in (reduce_scatter, reduce_scatter_inplace, allreduce):
            lib, p2p = both(fn)
            assert torch.allclose(lib, p2p, rtol=1e-5, atol=1e-5), (fn.__name__, chunk)
            checked += 1

    # symmetric buffers: direct peer stores / loads, no staging
    n = 1 << 20
    sym_out = comm.alloc_symmetric(n * world, torch.float32)
    sym_in = comm.alloc_symmetric(n * world, torch.float32)
    assert sym_out is not None and sym_in is not None
    x = torch.randn(n, generator=torch.Generator().manual_seed(7 + rank)).to(dev)
    sym_in.copy_(torch.randn(n * world, generator=torch.Generator().manual_seed(70 + rank)))
    torch.cuda.synchronize()
    torch.distributed.barrier()

    def allgather_sym():
        comm.allgather(T(x, "s"), T(sym_out, "r"))
        return sym_out.clone()

    def reduce_scatter_sym():
        out = torch.zeros(n, device=dev)
        comm.reduce_scatter(T(sym_in, "s"), T(out, "r"), 0)
        return out

    lib, p2p = both(allgather_sym)
    assert torch.equal(lib, p2p)
    lib, p2p = both(reduce_scatter_sym)
    assert torch.allclose(lib, p2p, rtol=1e-5, atol=1e-5)
    checked += 2

    # all-to-all with per-pair sizes out of a symmetric send buffer: receivers pull their segments.
    # Ragged element counts (16-byte rows do not line up) and a single-byte dtype (odd lengths).
    def counts(src, dst, scale):
        return scale * (1 + (3 * src + 5 * dst) % 7) + (src + dst) % 3

    for dtype, scale in ((torch.float32, 1000), (torch.uint8, 333)):
        send_all = sym_in if dtype == torch.float32 else comm.alloc_symmetric(8 * 7 * 400, torch.uint8)
        if dtype == torch.uint8:
            send_all.copy_(torch.randint(0, 255, (send_all.numel(),), generator=torch.Generator().manual_seed(rank),
                                         dtype=torch.uint8))
            torch.cuda.synchronize()
            torch.distributed.barrier()
        sc = [counts(rank, q, scale) for q in range(world)]
        rc = [counts(q, rank, scale) for q in range(world)]
        sd = [sum(sc[:q]) + q for q in range(world)]  # one element of slack between segments
        rd = [sum(rc[:q]) for q in range(world)]
        assert sd[-1] + sc[-1] <= send_all.numel()

        def alltoall_v():
            out = torch.zeros(sum(rc) + 5, dtype=dtype, device=dev)
            comm.alltoall_v(T(send_all, "s"), sc, sd, T(out, "r"), rc, rd)
            return out

        lib, p2p = both(alltoall_v)
        assert torch.equal(lib, p2p), ("alltoall_v", dtype)
        checked += 1

    # barrier: returns only once every rank has arrived
    comm.set_p2p_collectives(True)
    for _ in range(3):
        comm.barrier()
    comm.set_p2p_collectives(False)
    return checked


@pytest.mark.multigpu
def test_p2p_collectives_match_the_library():
    world = min(torch.cuda.device_count(), int(os.environ.get("BAGUA_TEST_WORLD", "8")))
    res = run_ranks(_p2p_vs_library, world, backend="nccl", timeout=600)
    assert all(r == 37 for r in res)
