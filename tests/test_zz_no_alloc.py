"""The allocation-free compress entry point, called through its exported C symbol, must
produce exactly what the pooled `BaguaTensorPy.compress` produces — twice in a row, since
every call reuses the same built-in scratch array.  (Collected last on purpose.)"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import bagua_core_b200 as bb

    lib = ctypes.CDLL(bb.SO_PATH)
    fn = lib.bagua_no_alloc_compress_minmax_u8_f32
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    lib.bagua_no_alloc_compressed_size.restype = ctypes.c_size_t
    lib.bagua_no_alloc_compressed_size.argtypes = [ctypes.c_int64, ctypes.c_int]
    lib.bagua_no_alloc_last_error.restype = ctypes.c_char_p
    return lib


@pytest.mark.parametrize("n_chunks,chunk", [(8, 1 << 18), (3, 1000), (1, 4096)])
def test_no_alloc_compress_matches_pooled_compress_twice(n_chunks, chunk):
    import bagua_core as bc

    lib = _lib()
    torch.cuda.set_device(0)
    n = n_chunks * chunk
    size = lib.bagua_no_alloc_compressed_size(n, n_chunks)
    out = torch.zeros(size, dtype=torch.uint8, device="cuda")  # caller-owned output, allocated up front
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        x = torch.randn(n, generator=torch.Generator().manual_seed(40 + call)).cuda() * (call + 1)
        expect = bc.BaguaTensorPy(x, "x").compress("MinMaxUInt8", n_chunks, -1).to_numpy_u8()
        torch.cuda.synchronize()
        rc = lib.bagua_no_alloc_compress_minmax_u8_f32(x.data_ptr(), n, n_chunks, out.data_ptr(), size, stream)
        assert rc == 0, lib.bagua_no_alloc_last_error()
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert got.shape[0] == expect.shape[0]
        # compare what the format defines: per chunk the 8 header bytes {min,max} and the
        # payload (the bytes between header and payload and after the last payload are
        # padding that neither entry point writes)
        off = size // n_chunks
        for c in range(n_chunks):
            assert (got[c * off:c * off + 8] == expect[c * off:c * off + 8]).all(), f"call {call} chunk {c}: header"
            a, b = got[c * off + 32:c * off + 32 + chunk], expect[c * off + 32:c * off + 32 + chunk]
            assert (a == b).all(), f"call {call} chunk {c}: {(a != b).sum()} payload bytes differ"


def test_no_alloc_rejects_what_does_not_fit():
    lib = _lib()
    x = torch.zeros(16384, device="cuda")
    out = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    rc = lib.bagua_no_alloc_compress_minmax_u8_f32(x.data_ptr(), 16384, 16384, out.data_ptr(), 1 << 20, None)
    assert rc == -2 and b"scratch" in lib.bagua_no_alloc_last_error()
    rc = lib.bagua_no_alloc_compress_minmax_u8_f32(x.data_ptr(), 16384, 8, out.data_ptr(), 64, None)
    assert rc == -1 and b"too small" in lib.bagua_no_alloc_last_error()
    # an input pointer that cannot be read as float is refused before anything is launched
    rc = lib.bagua_no_alloc_compress_minmax_u8_f32(x.data_ptr() + 2, 1024, 8, out.data_ptr(), 1 << 20, None)
    assert rc == -1 and b"aligned" in lib.bagua_no_alloc_last_error()
