"""The fused communication kernels on ONE GPU: all ranks' grids run side by side in a single
cooperative launch (`EmulatedArena`), executing the same device code as the multi-GPU
kernels.  Results are checked against plain fp32 PyTorch math and against the host
implementation of the MinMaxUInt8 compressor."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _arena(n, staging_mb=64):
    import bagua_core_b200 as bb

    a = bb._C.EmulatedArena(n, 0, staging_mb << 20)
    a.set_deadline_ms(5000.0)
    return a


def _inputs(nranks, n, dt, seed=0):
    return [torch.randn(n, generator=torch.Generator().manual_seed(seed + r)).to(dt).cuda() for r in range(nranks)]


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("mode", ["oneshot", "twoshot", "symmetric"])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_emulated_allreduce(nranks, mode, dt):
    arena = _arena(nranks)
    for n, blocks in [(64, 1), (4096 + 8, 3), (1 << 20, 8)]:
        xs = _inputs(nranks, n, dt, seed=n)
        ref = torch.stack([x.float() for x in xs]).mean(0)
        outs = [torch.zeros_like(x) for x in xs]
        arena.allreduce(xs, outs, True, mode, blocks)
        tol = 1e-6 if dt == torch.float32 else 1.6e-2
        for o in outs:
            assert torch.allclose(o.float(), ref, rtol=tol, atol=tol * max(1.0, ref.abs().max().item()))
            assert torch.equal(o, outs[0])  # every rank holds the same bits
        # in place, sum
        ys = [x.clone() for x in xs]
        arena.allreduce(ys, ys, False, mode, blocks)
        for y in ys:
            assert torch.allclose(y.float(), ref * nranks, rtol=tol, atol=tol * nranks * max(1.0, ref.abs().max().item()))


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
def test_emulated_bulk_copy_allreduce_equals_the_load_store_kernel(nranks, dt):
    """The symmetric all-reduce whose tiles travel through the bulk-copy engine (shared-memory ring,
    mbarrier completion, bulk stores) gives the same bits as the kernel that uses ordinary loads and
    stores: sizes below one tile, ragged tails, slices that are empty, many tiles per block (the ring
    wraps several times), in place and out of place."""
    arena = _arena(nranks)
    ve = 4 if dt == torch.float32 else 8
    for n, blocks in [(ve * nranks, 1), (ve * 37, 3), (ve * (1024 * nranks + 3), 2), (ve * 100003, 5), (1 << 22, 4),
                      ((1 << 22) + ve * 13, 1)]:
        xs = _inputs(nranks, n, dt, seed=n % 1000)
        want = [torch.zeros_like(x) for x in xs]
        arena.allreduce(xs, want, True, "symmetric", blocks)
        outs = [torch.full_like(x, 7.0) for x in xs]
        arena.allreduce(xs, outs, True, "symmetric_tma", blocks)
        ref = torch.stack([x.float() for x in xs]).mean(0)
        tol = 1e-6 if dt == torch.float32 else 1.6e-2
        for o, w in zip(outs, want):
            assert torch.equal(o, w), (n, blocks)
            assert torch.allclose(o.float(), ref, rtol=tol, atol=tol * max(1.0, ref.abs().max().item()))
        ys = [x.clone() for x in xs]
        arena.allreduce(ys, ys, False, "symmetric_tma", blocks)  # in place, sum
        zs = [x.clone() for x in xs]
        arena.allreduce(zs, zs, False, "symmetric", blocks)
        for y, z in zip(ys, zs):
            assert torch.equal(y, z), (n, blocks)


def test_emulated_mixed_ops_reuse_staging_safely():
    """Back-to-back ops with different layouts over the same staging (the `done` chain)."""
    nranks = 4
    arena = _arena(nranks)
    expect = sum(range(1, nranks + 1)) / nranks
    for rep in range(4):
        for n, mode, blocks in [(1 << 12, "oneshot", 2), (1 << 18, "twoshot", 6), (256, "oneshot", 1),
                                (1 << 16, "symmetric", 4), (1 << 14, "twoshot", 3), (1 << 17, "symmetric_tma", 3)]:
            xs = [torch.full((n,), float(r + 1), device="cuda") for r in range(nranks)]
            arena.allreduce(xs, xs, True, mode, blocks)
            for x in xs:
                assert torch.allclose(x, torch.full_like(x, expect))
    assert arena.epoch() == 24


@pytest.mark.parametrize("symmetric", [False, True])
@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_emulated_pair_average(nranks, symmetric):
    import bagua_core_b200 as bb

    arena = _arena(nranks)
    n = (1 << 16) + 16
    xs = _inputs(nranks, n, torch.float32, seed=3)
    for step in range(3):
        peers = [bb._C.shift_one_peer(r, nranks, step) for r in range(nranks)]
        outs = [torch.zeros_like(x) for x in xs]
        arena.pair_average(xs, outs, peers, 4, symmetric)
        for r in range(nranks):
            assert torch.allclose(outs[r], (xs[r] + xs[peers[r]]) / 2, atol=1e-6)
        xs = outs


def _cpu_compress_roundtrip(t_cpu, n_chunks):
    import bagua_core as bc

    c = bc.BaguaTensorPy(t_cpu, "x").compress("MinMaxUInt8", n_chunks, -1)
    out = torch.empty_like(t_cpu)
    bc.BaguaTensorPy(out, "o").decompress_from("MinMaxUInt8", n_chunks, c)
    return out


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("dt", [torch.float32, torch.float16])
def test_emulated_bytegrad_matches_host_oracle(nranks, dt):
    arena = _arena(nranks)
    n = 16 * nranks * 1031
    xs = _inputs(nranks, n, dt, seed=11)
    # oracle: quantise every rank's bucket per chunk, average the dequantised values, quantise again
    deq = [_cpu_compress_roundtrip(x.cpu(), nranks).float() for x in xs]
    red = (torch.stack(deq).sum(0) / nranks).to(dt)
    expect = _cpu_compress_roundtrip(red, nranks)
    bs = [x.clone() for x in xs]
    arena.bytegrad(bs, True, 5)
    for b in bs:
        assert torch.equal(b, bs[0])
    got = bs[0].cpu()
    diff = (got.float() - expect.float()).abs()
    step = (red.float().max() - red.float().min()).item() / 255
    assert diff.max().item() <= step * 1.01 + 1e-6  # at most one quantisation level (rounding ties)
    assert (diff > step * 0.01).float().mean().item() < 0.01
    mean = torch.stack([x.float().cpu() for x in xs]).mean(0)
    chunk = n // nranks
    for c in range(nranks):
        sl = slice(c * chunk, (c + 1) * chunk)
        rng = max((x[sl].float().max() - x[sl].float().min()).item() for x in xs)
        assert (got[sl].float() - mean[sl]).abs().max().item() <= 2 * rng / 255 + 4e-3


@pytest.mark.parametrize("nranks", [2, 4])
def test_emulated_low_precision_ring(nranks):
    arena = _arena(nranks)
    n = 16 * 4099
    w0 = _inputs(nranks, n, torch.float32, seed=21)
    x = [w.clone() + 0.01 for w in w0]
    w = [t.clone() for t in w0]
    left = [w0[(r - 1) % nranks].clone() for r in range(nranks)]
    right = [w0[(r + 1) % nranks].clone() for r in range(nranks)]
    # oracle for one step
    d = [x[r] + left[r] / 3 + right[r] / 3 - w[r] * (5.0 / 3.0) for r in range(nranks)]
    q = [_cpu_compress_roundtrip(t.cpu(), 1).cuda() for t in d]
    arena.lp_ring(x, w, left, right, 4)
    for r in range(nranks):
        step = (d[r].max() - d[r].min()).item() / 255
        assert torch.equal(x[r], w[r])
        assert (x[r] - (w0[r] + q[r])).abs().max().item() <= step * 1.01 + 1e-5
        assert (left[r] - w[(r - 1) % nranks]).abs().max().item() <= 1e-5
        assert (right[r] - w[(r + 1) % nranks]).abs().max().item() <= 1e-5


def test_emulated_arena_rejects_oversized_ops():
    arena = _arena(2, staging_mb=1)
    xs = [torch.zeros(1 << 20, device="cuda") for _ in range(2)]
    with pytest.raises(RuntimeError, match="staging"):
        arena.allreduce(xs, xs, True, "oneshot", 2)


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("dt", [torch.float32, torch.float16])
def test_emulated_bytegrad_pipelined_equals_the_default_variant(nranks, dt, monkeypatch):
    """Same bytes and values, another schedule for the last two phases: the results must be bit-equal."""
    arena = _arena(nranks)
    n = 16 * nranks * 1031
    xs = _inputs(nranks, n, dt, seed=13)
    plain = [x.clone() for x in xs]
    monkeypatch.delenv("BAGUA_B200_BYTEGRAD_PIPELINE_MIN_CHUNK", raising=False)
    arena.bytegrad(plain, True, 5)
    piped = [x.clone() for x in xs]
    monkeypatch.setenv("BAGUA_B200_BYTEGRAD_PIPELINE_MIN_CHUNK", "0")
    arena.bytegrad(piped, True, 5)
    torch.cuda.synchronize()
    for a, b in zip(plain, piped):
        assert torch.equal(a, b)
    assert not torch.equal(piped[0], xs[0])
