"""The signalling protocol of the fused kernels, checked as a host-thread model (same
epoch words, `done` chain and acquire/release structure; see tests/cpp/protocol_model.cc).
This is where ordering mistakes in the protocol itself would show: the model is a test
program of its own (built here with g++), not part of the engine's library."""
import json
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "bagua_core_b200", "csrc")
CPP = os.path.join(ROOT, "tests", "cpp")


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    gxx = shutil.which("g++")
    cuda_inc = "/usr/local/cuda/include"
    if gxx is None or not os.path.exists(os.path.join(cuda_inc, "cuda_runtime_api.h")):
        pytest.skip("needs g++ and the CUDA headers")
    exe = str(tmp_path_factory.mktemp("protocol") / "protocol_model")
    cmd = [gxx, "-std=c++17", "-O2", "-I", CSRC, "-I", CPP, "-I", cuda_inc, os.path.join(CPP, "protocol_model_main.cc"),
           os.path.join(CPP, "protocol_model.cc"), "-o", exe, "-lpthread"]
    build = subprocess.run(cmd, capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-2000:]

    def check(nranks, blocks, n_ops, seed=0, use_done_chain=True, slow_rank=-1, mix=False):
        run = subprocess.run([exe, str(nranks), str(blocks), str(n_ops), str(seed), str(int(use_done_chain)),
                              str(slow_rank), str(int(mix))], capture_output=True, text=True, timeout=300)
        assert run.returncode == 0, run.stderr[-2000:]
        return json.loads(run.stdout.strip().splitlines()[-1])

    return check


@pytest.mark.parametrize("nranks,blocks", [(2, 1), (2, 3), (3, 2), (4, 4), (8, 2)])
def test_random_schedules_never_corrupt_or_hang(model, nranks, blocks):
    for seed in range(3):
        r = model(nranks, blocks, 60, seed=seed)
        assert r == {"errors": 0, "timeouts": 0, "ops": 60}, (nranks, blocks, seed, r)


@pytest.mark.parametrize("nranks,blocks", [(2, 1), (2, 3), (3, 2), (4, 2), (5, 3), (8, 4)])
def test_every_collective_kernel_in_random_order(model, nranks, blocks):
    """Random sequences over all kernels of the communicator (all-reduces, all-gather, all-to-all,
    reduce-scatter through staging and with direct peer access, both broadcasts, barrier), each
    with the kernels' own index arithmetic: every value that arrives is the expected one."""
    for seed in range(3):
        r = model(nranks, blocks, 80, seed=seed, mix=True)
        assert r == {"errors": 0, "timeouts": 0, "ops": 80}, (nranks, blocks, seed, r)


def test_mixed_sequences_need_the_done_chain(model):
    errors = sum(model(4, 2, 200, seed=s, use_done_chain=False, mix=True)["errors"] for s in range(4))
    assert errors > 0


def test_adversarial_delay_is_safe_with_the_done_chain_and_unsafe_without(model):
    """A rank that lingers in the copy-out of a two-shot op while its peer starts a one-shot op
    over the same staging addresses: the `done` chain is exactly what keeps that safe."""
    safe = model(2, 1, 20, seed=1, use_done_chain=True, slow_rank=0)
    assert safe["errors"] == 0 and safe["timeouts"] == 0
    unsafe = model(2, 1, 20, seed=1, use_done_chain=False, slow_rank=0)
    assert unsafe["errors"] > 0
