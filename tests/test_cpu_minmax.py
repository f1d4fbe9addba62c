"""Properties of the MinMaxUInt8 compressor (host implementation = the oracle the GPU
kernels are compared against).  Reference numerics:
bagua-core-internal/kernels/bagua_kernels.cu:10,411-432,465-467."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

import bagua_core as bc
import bagua_core_b200 as bb


def _roundtrip(x, n_chunks):
    t = bc.BaguaTensorPy(x, "x")
    c = t.compress("MinMaxUInt8", n_chunks, -1)
    out = torch.empty_like(x)
    bc.BaguaTensorPy(out, "o").decompress_from("MinMaxUInt8", n_chunks, c)
    return c.to_numpy_u8(), out


def _python_oracle(chunk: np.ndarray):
    """Scalar restatement of the reference formulas in numpy float32/float64."""
    mn, mx = np.float32(chunk.min()), np.float32(chunk.max())
    denom = np.float32(np.float32(mx - mn) + np.float32(1e-7))
    scale = np.float32(np.float64(255.0) / np.float64(denom))
    upper = np.float32(np.rint(np.float32(mx * scale)))
    lower = np.float32(upper - np.float32(255.0))
    level = np.minimum(np.rint((chunk * scale).astype(np.float32)), upper)
    q = np.clip(level - lower, 0, 255).astype(np.uint8)
    deq = ((q.astype(np.float32) + lower) / scale).astype(np.float32)
    return mn, mx, q, deq


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 6), st.integers(1, 300), st.floats(1e-3, 1e3), st.floats(-100, 100), st.integers(0, 2 ** 31 - 1))
def test_layout_header_and_error_bound(n_chunks, chunk, spread, shift, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(n_chunks * chunk, generator=g) * spread + shift).float()
    buf, out = _roundtrip(x, n_chunks)
    total = bb._C.compressed_buffer_size(n_chunks, chunk, "F32")
    assert buf.shape[0] == total == (n_chunks * chunk + 31) // 32 * 32 + 32 * n_chunks
    off = total // n_chunks
    xs = x.numpy().reshape(n_chunks, chunk)
    os_ = out.numpy().reshape(n_chunks, chunk)
    for c in range(n_chunks):
        hdr = buf[c * off:c * off + 8].copy().view(np.float32)
        mn, mx, q, deq = _python_oracle(xs[c])
        assert hdr[0] == mn and hdr[1] == mx
        assert np.array_equal(buf[c * off + 32:c * off + 32 + chunk], q)
        assert np.array_equal(os_[c], deq)
        # worst-case error of the anchored grid: one level, (max-min)/255 (+ float slack)
        rng = float(mx - mn)
        assert np.abs(os_[c] - xs[c]).max() <= rng / 255 * 1.001 + 1e-6 * max(1.0, abs(float(mx)))


def test_zero_is_exactly_representable_when_the_range_spans_it():
    x = torch.tensor([-1.3, 0.0, 0.0, 2.9, 0.7, -0.2] * 8)
    _, out = _roundtrip(x, 1)
    assert (out[x == 0] == 0).all()


def test_constant_chunk_and_single_element():
    for v in (0.0, 3.5, -7.25):
        x = torch.full((40,), v)
        _, out = _roundtrip(x, 2)
        assert torch.allclose(out, x, atol=1e-6)
    _, out = _roundtrip(torch.tensor([2.0]), 1)
    assert abs(out.item() - 2.0) < 1e-6


def test_compress_is_idempotent_on_its_own_output():
    x = torch.randn(4096, generator=torch.Generator().manual_seed(5))
    _, once = _roundtrip(x, 4)
    _, twice = _roundtrip(once.clone(), 4)
    assert (once - twice).abs().max() <= (x.max() - x.min()) / 255 * 0.51


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_half_types_store_header_in_tensor_dtype(dt):
    x = torch.randn(256, generator=torch.Generator().manual_seed(6)).to(dt)
    buf, out = _roundtrip(x, 2)
    off = buf.shape[0] // 2
    for c in range(2):
        raw = buf[c * off:c * off + 4].copy()
        hdr = torch.from_numpy(raw.view(np.int16).copy()).view(dt)
        assert hdr[0] == x[c * 128:(c + 1) * 128].min() and hdr[1] == x[c * 128:(c + 1) * 128].max()
    rng = (x.float().max() - x.float().min()).item()
    assert (out.float() - x.float()).abs().max().item() <= rng / 255 * 1.1 + 0.02


def test_target_chunk_compresses_only_that_chunk():
    x = torch.randn(4 * 64, generator=torch.Generator().manual_seed(8))
    full = bc.BaguaTensorPy(x, "x").compress("MinMaxUInt8", 4, -1).to_numpy_u8()
    one = bc.BaguaTensorPy(x, "x").compress("MinMaxUInt8", 4, 1).to_numpy_u8()
    off = full.shape[0] // 4
    assert np.array_equal(full[off:off + 32 + 64][:8], one[off:off + 8])
    assert np.array_equal(full[off + 32:off + 32 + 64], one[off + 32:off + 32 + 64])


def test_rejects_bad_arguments():
    x = torch.randn(10)
    with pytest.raises(RuntimeError, match="n_chunks"):
        bc.BaguaTensorPy(x, "x").compress("MinMaxUInt8", 3, -1)
    with pytest.raises(RuntimeError, match="unsupported compression"):
        bc.BaguaTensorPy(x, "x").compress("TopK", 1, -1)
    with pytest.raises(RuntimeError):
        bc.BaguaTensorPy(torch.zeros(4, dtype=torch.int64), "i").compress("MinMaxUInt8", 1, -1)
