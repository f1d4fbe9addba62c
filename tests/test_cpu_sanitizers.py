"""Host runtime under ThreadSanitizer: a C++ stress program (tests/cpp/runtime_stress.cc) that
drives the scheduler, channels, buckets and pools from several threads is compiled with
-fsanitize=thread together with the engine's own sources and must finish with exit code 0
and without a sanitizer report.  (This covers the host half of the engine; the device code runs under the
same sanitizers in tests/test_cpu_device_emulation.py.)"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "bagua_core_b200", "csrc")
SOURCES = ["runtime/backend.cc", "runtime/timeline.cc", "tensor/tensor.cc", "pool/resource_pool.cc", "ops/ops.cc", "telemetry/telemetry.cc",
           "kernels/cpu_kernels.cc"]


def _nccl_include():
    import torch

    site = os.path.dirname(os.path.dirname(torch.__file__))
    inc = os.path.join(site, "nvidia", "nccl", "include")
    return inc if os.path.exists(os.path.join(inc, "nccl.h")) else "/usr/include"


@pytest.mark.parametrize("sanitizer", ["thread"] + (["address"] if os.environ.get("BAGUA_TEST_ASAN") else []))
def test_runtime_stress_is_clean_under_sanitizer(tmp_path, sanitizer):
    gxx = shutil.which("g++")
    cuda_inc = "/usr/local/cuda/include"
    if gxx is None or not os.path.exists(os.path.join(cuda_inc, "cuda_runtime_api.h")):
        pytest.skip("needs g++ and the CUDA headers")
    exe = str(tmp_path / f"stress_{sanitizer}")
    cmd = [gxx, "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", "-I", CSRC, "-I",
           cuda_inc, "-I", _nccl_include(), "-I", os.path.join(ROOT, "tests", "cpp"),
           os.path.join(ROOT, "tests", "cpp", "runtime_stress.cc"), os.path.join(ROOT, "tests", "cpp", "protocol_model.cc"),
           os.path.join(ROOT, "tests", "cpp", "stubs.cc")] + [os.path.join(CSRC, s) for s in SOURCES] + [
               "-o", exe, "-L/usr/local/cuda/lib64", "-lcudart", "-lpthread"]
    build = subprocess.run(cmd, capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, LD_LIBRARY_PATH="/usr/local/cuda/lib64:" + os.environ.get("LD_LIBRARY_PATH", ""))
    run = subprocess.run([exe], capture_output=True, text=True, env=env, timeout=300)
    out = run.stdout + run.stderr
    assert run.returncode == 0, out[-3000:]
    assert "0 failures" in out
    assert "WARNING: ThreadSanitizer" not in out and "ERROR: AddressSanitizer" not in out, out[-3000:]


@pytest.mark.parametrize("sanitizer", ["address", "thread"])
def test_multicast_slab_setup_against_a_stand_in_driver(tmp_path, sanitizer):
    """`csrc/comm/nvls.cc` (the set-up of symmetric memory with an NVSwitch multicast mapping) without a GPU:
    ranks are threads, the CUDA runtime and driver are a stand-in that counts what it hands out.  Every
    driver call is made to fail on the first and on the last rank in turn; all ranks must then give up at
    the same step with nothing left allocated, mapped, bound or open (tests/cpp/nvls_setup.cc)."""
    gxx = shutil.which("g++")
    cuda_inc = "/usr/local/cuda/include"
    if gxx is None or not os.path.exists(os.path.join(cuda_inc, "cuda.h")):
        pytest.skip("needs g++ and the CUDA headers")
    exe = str(tmp_path / f"nvls_setup_{sanitizer}")
    cmd = [gxx, "-std=c++20", "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", "-I", CSRC, "-I", cuda_inc,
           os.path.join(ROOT, "tests", "cpp", "nvls_setup.cc"), os.path.join(CSRC, "comm", "nvls.cc"),
           os.path.join(CSRC, "pool", "resource_pool.cc"), "-o", exe, "-L/usr/local/cuda/lib64", "-lcudart", "-lpthread"]
    build = subprocess.run(cmd, capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, LD_LIBRARY_PATH="/usr/local/cuda/lib64:" + os.environ.get("LD_LIBRARY_PATH", ""))
    run = subprocess.run([exe], capture_output=True, text=True, env=env, timeout=300)
    out = run.stdout + run.stderr
    assert run.returncode == 0, out[-3000:]
    assert "63 cases" in out and " 0 failures" in out, out[-2000:]
    assert "WARNING: ThreadSanitizer" not in out and "ERROR: AddressSanitizer" not in out, out[-3000:]
