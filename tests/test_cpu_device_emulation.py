"""The device code of every fused communication kernel, run on the CPU.

The `*_body` device functions (`csrc/kernels/fused_allreduce_bodies.cuh`, `fused_collectives_bodies.cuh`,
`fused_bytegrad_body.cuh`, `fused_gossip_body.cuh`) are compiled by the host compiler with
-DBAGUA_HOST_EMULATION (`csrc/kernels/host_emulation.h`: one OS thread per CUDA thread, a block is one
warp of 32 threads with a barrier, GCC atomics for the PTX release/acquire instructions, warp
shuffles through a per-block exchange buffer) into tests/cpp/device_emulation.cc, which drives random
sequences of all-reduce (one-shot, two-shot, symmetric), pair average, ByteGrad, the low-precision
ring, all-gather, all-to-all (equal and per-pair sizes), reduce-scatter, broadcast, scatter, gather,
reduce and barrier —
staging and direct-peer-access forms, in-place forms — for N ranks x G blocks and checks every
result exactly (the quantising kernels against a scalar restatement of MinMaxUInt8).  Built with
-fsanitize=thread the same program checks that the signalling orders every payload access (no data
race report).  The one access pattern that is exempt has a name in the source: chunk headers, which
every block of a rank writes with the same value (`same_value_store` / `same_value_load`)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "bagua_core_b200", "csrc")
CUDA_INC = "/usr/local/cuda/include"


def _sanitizer_flags(sanitizer):
    flags = [f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer"]
    if sanitizer == "undefined":
        flags.append("-fno-sanitize-recover=undefined")  # the first report ends the program
    return flags


def _build(tmp_path, sanitizer):
    gxx = shutil.which("g++")
    if gxx is None or not os.path.exists(os.path.join(CUDA_INC, "cuda_runtime.h")):
        pytest.skip("needs g++ and the CUDA headers")
    exe = str(tmp_path / ("device_emulation_" + (sanitizer or "plain")))
    cmd = [gxx, "-std=c++20", "-O1", "-g", "-fno-strict-aliasing", "-DBAGUA_HOST_EMULATION", "-I", CSRC, "-I", CUDA_INC,
           os.path.join(ROOT, "tests", "cpp", "device_emulation.cc"), "-o", exe, "-lpthread"]
    if sanitizer:
        cmd[1:1] = _sanitizer_flags(sanitizer)
    build = subprocess.run(cmd, capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    return exe


def _run(exe, *args):
    run = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=600)
    out = run.stdout + run.stderr
    assert run.returncode == 0, out[-3000:]
    assert "0 wrong vectors, wait status 0, 0 failures" in out, out[-3000:]
    return out


def test_device_bodies_compute_every_collective_correctly(tmp_path):
    exe = _build(tmp_path, None)
    for nranks, blocks, ops, seed in [(2, 1, 150, 1), (3, 3, 150, 2), (4, 2, 200, 3), (5, 1, 100, 4), (8, 2, 120, 5),
                                      (8, 3, 80, 6)]:
        _run(exe, nranks, blocks, ops, seed)


def test_a_missing_rank_makes_the_others_time_out_and_return(tmp_path):
    """Failure detection of the device code without a GPU: one rank never runs; every wait of the
    others is bounded, so they record what they waited for and return instead of hanging."""
    exe = _build(tmp_path, None)
    for nranks, absent in [(2, 1), (4, 2), (8, 0)]:
        run = subprocess.run([exe, str(nranks), "2", "30", "1", str(absent), "300"], capture_output=True, text=True,
                             timeout=120)
        assert run.returncode == 3, run.stdout + run.stderr
        assert f"rank {absent} absent, every other rank returned" in run.stdout
        assert "wait status code 0" not in run.stdout


def test_alltoall_v_reports_sizes_that_sender_and_receiver_disagree_on(tmp_path):
    """Rank 0 announces a longer segment than rank 1 expects: rank 1 records status code 4 with the
    sender's rank, still receives exactly the bytes it asked for, and every rank returns."""
    exe = _build(tmp_path, None)
    for nranks in (2, 5):
        run = subprocess.run([exe, str(nranks), "2", "1", "3", "-1", "30000", "1"], capture_output=True, text=True,
                             timeout=240)
        assert run.returncode == 1, run.stdout + run.stderr
        assert "0 wrong vectors, wait status 4, 1 failures" in run.stdout, run.stdout + run.stderr


def test_device_bodies_are_race_free_under_thread_sanitizer(tmp_path):
    exe = _build(tmp_path, "thread")
    for nranks, blocks, ops, seed in [(2, 1, 80, 1), (4, 2, 80, 2), (3, 3, 60, 3)]:
        out = _run(exe, nranks, blocks, ops, seed)
        assert "WARNING: ThreadSanitizer" not in out, out[-3000:]


def test_device_bodies_stay_in_bounds_under_address_sanitizer(tmp_path):
    """The memory checker for device code that needs no GPU: every buffer of the emulation is a heap
    block of its own, so a load or store of a body outside staging, input or output is reported.  (Stores
    inside a buffer but outside the op's extent are caught by the poison check of every run.)"""
    exe = _build(tmp_path, "address")
    for nranks, blocks, ops, seed in [(2, 1, 80, 11), (4, 2, 80, 12), (8, 2, 60, 13)]:
        out = _run(exe, nranks, blocks, ops, seed)
        assert "ERROR: AddressSanitizer" not in out, out[-3000:]


def test_device_bodies_keep_every_vector_access_aligned(tmp_path):
    """A 16-byte load or store at an address that is not a multiple of 16 is a fault on the GPU and
    passes silently on an x86 host.  The CUDA vector types keep their alignment under the host compiler
    (`alignof(uint4) == 16`), so the alignment check of the undefined-behaviour sanitizer sees every
    such access of the bodies: ragged sizes, odd chunk counts and the per-pair all-to-all offsets
    included.  The other checks of that sanitizer (shift widths, signed overflow in index arithmetic,
    indexing past a fixed-size array) come with it.  The program stops at the first report."""
    exe = _build(tmp_path, "undefined")
    for nranks, blocks, ops, seed in [(2, 1, 150, 21), (3, 3, 120, 22), (5, 1, 100, 23), (8, 2, 100, 24)]:
        out = _run(exe, nranks, blocks, ops, seed)
        assert "runtime error" not in out, out[-3000:]


@pytest.mark.parametrize("sanitizer", [None, "address", "undefined"])
def test_model_op_kernels_match_the_host_restatement(tmp_path, sanitizer):
    """The fused bias+ReLU and max-pool kernels (`csrc/kernels/model_ops_bodies.cuh`), run thread for
    thread on grids of a few blocks of 256 threads, against `csrc/kernels/model_ops_cpu.cc`; the second
    build runs them under AddressSanitizer (every tensor is a heap block of exactly its size)."""
    gxx = shutil.which("g++")
    if gxx is None or not os.path.exists(os.path.join(CUDA_INC, "cuda_runtime.h")):
        pytest.skip("needs g++ and the CUDA headers")
    exe = str(tmp_path / "model_ops_emulation")
    cmd = [gxx, "-std=c++20", "-O1", "-g", "-fno-strict-aliasing", "-DBAGUA_HOST_EMULATION", "-I", CSRC, "-I", CUDA_INC,
           os.path.join(ROOT, "tests", "cpp", "model_ops_emulation.cc"), os.path.join(CSRC, "kernels", "model_ops_cpu.cc"),
           "-o", exe, "-lpthread"]
    if sanitizer:
        cmd[1:1] = _sanitizer_flags(sanitizer)
    build = subprocess.run(cmd, capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0 and "0 failures" in run.stdout, run.stdout + run.stderr
    assert "ERROR: AddressSanitizer" not in run.stdout + run.stderr
    assert "runtime error" not in run.stdout + run.stderr
