"""Single-GPU numerics of the sm_100a tensor kernels against plain PyTorch fp32 references
(and against the engine's own host implementation, which defines the MinMaxUInt8 grid)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [1, 31, 32, 33, 1023, 4096, (1 << 20) + 1, 3 << 20]
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _tol(dt):
    return {torch.float32: 1e-6, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dt]


def _rand(n, dt, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g).to(dt).cuda()


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("dt", DTYPES)
def test_elementwise(n, dt):
    import bagua_core_b200.ops as ops

    x, y = _rand(n, dt, 1), _rand(n, dt, 2)
    xf, yf = x.float(), y.float()
    cases = [
        (lambda a: ops.add_inplace(a, y), xf + yf),
        (lambda a: ops.subtract_inplace(a, y), xf - yf),
        (lambda a: ops.addmul_inplace(a, y, -5.0 / 3.0), xf + yf * (-5.0 / 3.0)),
        (lambda a: ops.average_inplace(a, y), (xf + yf) / 2),
        (lambda a: ops.divide_inplace(a, 7.0), xf / 7.0),
    ]
    for fn, ref in cases:
        a = x.clone()
        fn(a)
        torch.cuda.synchronize()
        assert torch.allclose(a.float(), ref, rtol=_tol(dt), atol=_tol(dt)), (n, dt)


@pytest.mark.parametrize("offset", [0, 1, 3])
def test_elementwise_unaligned_views(offset):
    import bagua_core_b200.ops as ops

    base = _rand(5000 + offset, torch.float32, 3)
    x = base[offset:]
    y = _rand(5000, torch.float32, 4)
    ref = x.clone() + y
    ops.add_inplace(x, y)
    torch.cuda.synchronize()
    assert torch.allclose(x, ref, atol=1e-6)


@pytest.mark.parametrize("n_chunks,chunk", [(2, 48), (8, 4096), (3, 1000), (8, (1 << 18))])
@pytest.mark.parametrize("dt", DTYPES)
def test_reduce_chunk(n_chunks, chunk, dt):
    import bagua_core_b200.ops as ops

    x = _rand(n_chunks * chunk, dt, 5)
    for avg in (True, False):
        a = x.clone()
        ops.reduce_chunk_inplace(a, n_chunks, n_chunks - 1, average=avg)
        torch.cuda.synchronize()
        ref = x.float().view(n_chunks, chunk).sum(0)
        if avg:
            ref = ref / n_chunks
        got = a.view(n_chunks, chunk)[n_chunks - 1].float()
        assert torch.allclose(got, ref, rtol=_tol(dt) * 4, atol=_tol(dt) * 4)
        # other chunks untouched
        assert torch.equal(a.view(n_chunks, chunk)[: n_chunks - 1], x.view(n_chunks, chunk)[: n_chunks - 1])


def test_async_model_average():
    import bagua_core_b200.ops as ops

    for n in (5, 4096, (1 << 20) + 3):
        t, r, c = _rand(n, torch.float32, 6), _rand(n, torch.float32, 7), _rand(n, torch.float32, 8)
        ref = t + (r / 4.0 - c)
        ops.async_model_average(t, r, c, 4)
        torch.cuda.synchronize()
        assert torch.allclose(t, ref, atol=1e-5)


@pytest.mark.parametrize("n_chunks,chunk", [(1, 16), (1, 1000), (2, 48), (8, 4096), (4, 1 << 19), (3, 37)])
@pytest.mark.parametrize("dt", DTYPES)
def test_minmax_uint8_matches_host_and_bound(n_chunks, chunk, dt):
    import bagua_core as bc

    x = _rand(n_chunks * chunk, dt, 9)
    gpu_c = bc.BaguaTensorPy(x, "x").compress("MinMaxUInt8", n_chunks, -1)
    cpu_c = bc.BaguaTensorPy(x.cpu(), "x").compress("MinMaxUInt8", n_chunks, -1)
    g, c = gpu_c.to_numpy_u8(), cpu_c.to_numpy_u8()
    total = g.shape[0]
    off = total // n_chunks
    for i in range(n_chunks):
        # headers (min/max in the tensor dtype) and payloads agree with the host oracle
        esz = x.element_size()
        assert (g[i * off:i * off + 2 * esz] == c[i * off:i * off + 2 * esz]).all()
        pg, pc = g[i * off + 32:i * off + 32 + chunk], c[i * off + 32:i * off + 32 + chunk]
        # rounding of x*scale at exact .5 ties may differ by one level between FMA and non-FMA paths
        assert (abs(pg.astype(int) - pc.astype(int)) <= 1).all()
        assert (pg != pc).mean() < 0.01
    out = torch.empty_like(x)
    bc.BaguaTensorPy(out, "o").decompress_from("MinMaxUInt8", n_chunks, gpu_c)
    torch.cuda.synchronize()
    xf, of = x.float().view(n_chunks, chunk), out.float().view(n_chunks, chunk)
    rng = (xf.max(1).values - xf.min(1).values)
    err = (xf - of).abs().max(1).values
    slack = {torch.float32: 0.0, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dt] * xf.abs().max()
    assert (err <= rng / 255 * 0.51 + slack + 1e-6).all(), (err, rng / 255)


def test_minmax_uint8_target_chunk_only():
    import bagua_core as bc

    n_chunks, chunk = 4, 4096
    x = _rand(n_chunks * chunk, torch.float32, 10)
    full = bc.BaguaTensorPy(x, "x").compress("MinMaxUInt8", n_chunks, -1).to_numpy_u8()
    one = bc.BaguaTensorPy(x, "x").compress("MinMaxUInt8", n_chunks, 2).to_numpy_u8()
    off = full.shape[0] // n_chunks
    assert (full[2 * off:3 * off] == one[2 * off:3 * off]).all()


def test_sgd_flat_matches_torch():
    import bagua_core_b200.ops as ops

    n = (1 << 20) + 5
    p, g = _rand(n, torch.float32, 11), _rand(n, torch.float32, 12)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.SGD([ref_p], lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=True)
    buf = torch.zeros_like(p)
    for step in range(3):
        ref_p.grad = g.clone()
        opt.step()
        ops.sgd_momentum_flat(p, g, buf, 0.1, 0.9, 0.0, 1e-4, True, first_step=(step == 0))
    torch.cuda.synchronize()
    assert torch.allclose(p, ref_p.detach(), atol=1e-5, rtol=1e-5)


def test_device_wait_runs_out_and_reports():
    """A wait that nothing will ever satisfy ends by itself with a status record; the
    context stays usable."""
    import bagua_core_b200 as bb

    st = bb._C.debug_wait_timeout(0, 50.0)
    assert st["code"] == 2 and st["peer"] == 1 and st["epoch"] == 1
    x = torch.ones(16, device="cuda")
    assert float((x * 2).sum()) == 32.0


@pytest.mark.parametrize("n", [1, 17, 4096, 65536 + 3, (1 << 20) + 16])
@pytest.mark.parametrize("dt", DTYPES)
def test_kernels_stay_inside_their_buffers(n, dt):
    """Guard regions of a sentinel value on both sides of every operand must survive every
    kernel (a memory check that needs no external tool)."""
    import bagua_core as bc
    import bagua_core_b200.ops as ops

    guard = 64
    sentinel = 12345.0

    def guarded(seed):
        buf = torch.full((n + 2 * guard,), sentinel, dtype=dt, device="cuda")
        buf[guard:guard + n] = _rand(n, dt, seed)
        return buf, buf[guard:guard + n]

    def intact(buf):
        return bool((buf[:guard] == sentinel).all() and (buf[guard + n:] == sentinel).all())

    bx, x = guarded(21)
    by, y = guarded(22)
    ops.add_inplace(x, y)
    ops.addmul_inplace(x, y, 0.25)
    ops.average_inplace(x, y)
    ops.subtract_inplace(x, y)
    ops.divide_inplace(x, 3.0)
    if n % 2 == 0:
        ops.reduce_chunk_inplace(x, 2, 1, average=True)
    torch.cuda.synchronize()
    assert intact(bx) and intact(by)
    # compress into an engine buffer, decompress into a guarded output
    chunks = 2 if n % 2 == 0 else 1
    c = bc.BaguaTensorPy(x, "x").compress("MinMaxUInt8", chunks, -1)
    bo, o = guarded(23)
    bc.BaguaTensorPy(o, "o").decompress_from("MinMaxUInt8", chunks, c)
    torch.cuda.synchronize()
    assert intact(bx) and intact(bo)
    if dt == torch.float32:
        bm, mbuf = guarded(24)
        mbuf.zero_()
        ops.sgd_momentum_flat(x, y, mbuf, 0.01, 0.9)
        bt, t = guarded(25)
        ops.async_model_average(t, x, y, 4)
        torch.cuda.synchronize()
        assert intact(bx) and intact(by) and intact(bm) and intact(bt)


def test_pool_reuses_blocks():
    import bagua_core as bc
    import bagua_core_b200 as bb

    x = _rand(1 << 16, torch.float32, 13)
    bc.BaguaTensorPy(x, "x").compress("MinMaxUInt8", 1, -1)
    a = bb._C.pool_stats(0)["device_allocs"]
    for _ in range(5):
        bc.BaguaTensorPy(x, "x").compress("MinMaxUInt8", 1, -1)
    torch.cuda.synchronize()
    assert bb._C.pool_stats(0)["device_allocs"] == a


def test_pool_guard_regions_stay_intact_under_the_kernels_and_catch_a_stray_store():
    """Device pool blocks with guard regions: the compression kernels on ragged sizes leave every
    guard intact, and four bytes stored just past a block's capacity are found."""
    import bagua_core as bc
    import bagua_core_b200 as bb

    runtime = pytest.importorskip("cuda.bindings.runtime")
    C = bb._C
    was = C.pool_guard()
    torch.cuda.synchronize()
    C.pool_release_cached(0)
    C.pool_set_guard(True)
    try:
        kept = []
        for n in SIZES:
            for dt in (torch.float32, torch.float16):
                x = _rand(n, dt, n % 97)
                t = bc.BaguaTensorPy(x, "x")
                c = t.compress("MinMaxUInt8", 1, -1)
                back = bc.BaguaTensorPy(torch.empty_like(x), "back")
                back.decompress_from("MinMaxUInt8", 1, c)
                kept.append(c)
        assert C.pool_check_guards(0) == 0
        c = kept[-1]
        cap = C.pool_size_class(c.num_elements_allocated())
        (err,) = runtime.cudaMemset(c.data_ptr() + cap, 0, 4)  # inside the allocation: the rear guard
        assert int(err) == 0
        assert C.pool_check_guards(0) == 1
        (err,) = runtime.cudaMemset(c.data_ptr() + cap, 0xC5, 4)
        assert int(err) == 0
        assert C.pool_check_guards(0) == 0
        del kept, c
    finally:
        torch.cuda.synchronize()
        C.pool_release_cached(0)
        C.pool_set_guard(was)


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.uint8])
def test_multi_tensor_flatten_and_unflatten_in_one_launch(dt):
    """The staged-bucket copy kernel: ragged tensor sizes (tiles that hold many small tensors, tensors that
    span many tiles, odd byte counts and therefore odd offsets), gathered into a flat buffer and scattered
    back, bit-equal to torch.cat; bytes outside the packed range stay untouched."""
    import bagua_core_b200 as bb

    sizes = [1, 7, 0, 33, 4096, 5, (1 << 18) + 3, 1023, 16, (3 << 16) + 1, 2, 70001]
    g = torch.Generator().manual_seed(5)
    ts = []
    for i, n in enumerate(sizes):
        base = torch.randint(0, 255, (n + 3,), generator=g).to(torch.float32)
        t = base.to(dt).cuda()[i % 3:i % 3 + n]  # views at odd element offsets: every alignment class occurs
        ts.append(t.contiguous() if i % 2 else t)
    total = sum(t.numel() for t in ts)
    flat = torch.full((total + 64,), 77, dtype=dt, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    bb._C.k_multi_copy(ts, flat, True, stream)
    torch.cuda.synchronize()
    assert torch.equal(flat[:total], torch.cat([t.reshape(-1) for t in ts]))
    assert (flat[total:] == 77).all()
    # scatter back what a communication op would have left in the flat buffer
    flat[:total] = (flat[:total].float() * 0 + torch.arange(total, device="cuda") % 251).to(dt)
    want = flat[:total].clone()
    bb._C.k_multi_copy(ts, flat, False, stream)
    torch.cuda.synchronize()
    assert torch.equal(torch.cat([t.reshape(-1) for t in ts]), want)


def test_a_bucket_of_scattered_tensors_is_staged_with_the_copy_kernel():
    """Through the engine: a bucket whose tensors are not adjacent in memory is flattened into a pool
    buffer, handed to the op and copied back (here the op divides by the rank count of one: the round trip
    must leave every tensor's values in place and nothing else touched)."""
    import bagua_core as bc
    import bagua_core_b200 as bb

    torch.cuda.set_device(0)
    backing = torch.zeros(1 << 16, device="cuda")
    views = [backing[10:1000], backing[2000:2007], backing[4096:4096 + 12345], backing[30000:30001]]
    for i, v in enumerate(views):
        v.copy_(torch.arange(v.numel(), device="cuda") + 1000 * i)
    before = backing.clone()
    seen = []
    tensors = [bc.BaguaTensorPy(v, f"t{i}") for i, v in enumerate(views)]
    bucket = bc.BaguaBucketPy("scattered", tensors)
    stream = torch.cuda.Stream()
    uid = bc.BaguaSingleCommunicatorPy.generate_nccl_unique_id_str()
    comm = bc.BaguaSingleCommunicatorPy(0, 1, 0, stream.cuda_stream, uid)
    bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True)
    backend = bc.BaguaCommBackendPy(4, 0)
    backend.register_ordered_buckets([bucket])
    staged0 = bb._C.stats()["staged_copies"]
    torch.cuda.synchronize()
    for _ in range(2):  # the second round reuses the cached table
        for t in tensors:
            backend.mark_communication_ready(t, 0)
        assert backend.wait_pending_comm_ops() == 1
    stream.synchronize()
    assert bb._C.stats()["staged_copies"] == staged0 + 2
    assert torch.equal(backing, before)
    backend.close()


def test_bucket_time_line_records_one_span_per_bucket_and_the_marks():
    """Two device events bracket each bucket's work on the communication stream; marks can be dropped on any
    stream; times are relative to the first recorded event and ordered like the stream."""
    import bagua_core as bc
    import bagua_core_b200 as bb

    torch.cuda.set_device(0)
    x = torch.ones(1 << 20, device="cuda")
    y = torch.ones(1 << 10, device="cuda")
    tx, ty = bc.BaguaTensorPy(x, "x"), bc.BaguaTensorPy(y, "y")
    stream = torch.cuda.Stream()
    comm = bc.BaguaSingleCommunicatorPy(0, 1, 0, stream.cuda_stream, bc.BaguaSingleCommunicatorPy.generate_nccl_unique_id_str())
    buckets = [bc.BaguaBucketPy("first", [tx]), bc.BaguaBucketPy("second", [ty])]
    for b in buckets:
        b.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True)
    backend = bc.BaguaCommBackendPy(4, 0)
    backend.register_ordered_buckets(buckets)
    bb._C.timeline_collect()
    bb._C.set_bucket_timing(True)
    try:
        bb._C.timeline_mark("begin", torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        backend.mark_communication_ready(tx, 0)
        backend.mark_communication_ready(ty, 0)
        assert backend.wait_pending_comm_ops() == 2
        stream.synchronize()
        bb._C.timeline_mark("end", stream.cuda_stream)
    finally:
        bb._C.set_bucket_timing(False)
    spans = bb._C.timeline_collect()
    assert [(s["name"], s["kind"]) for s in spans] == [("begin", "mark"), ("first", "bucket"), ("second", "bucket"),
                                                      ("end", "mark")]
    assert spans[0]["start_ms"] == 0.0
    assert spans[1]["bytes"] == 4 << 20 and spans[2]["bytes"] == 4 << 10
    for s in spans:
        assert s["end_ms"] >= s["start_ms"] >= 0.0
    assert spans[1]["end_ms"] <= spans[2]["start_ms"] + 1e-3 and spans[2]["end_ms"] <= spans[3]["start_ms"] + 1e-3
    assert bb._C.timeline_collect() == []
    backend.close()
