"""In-tree build of the native extension (C++ runtime + sm_100a kernels).

`build()` compiles every source under `csrc/` with ninja through
`torch.utils.cpp_extension.load` (CUDA files with
`-gencode arch=compute_100a,code=sm_100a`, which bypasses torch's own arch list) and
copies the resulting shared object next to this file as `_bagua_core_b200.so`.  The
package imports that file directly, so a machine that receives the built tree needs
neither a compiler nor a JIT cache.  nvcc cross-compiles: no GPU is needed to build.

Counterpart of the reference's build script (bagua-core-internal/build.rs:1-90), which
compiles its kernels for every architecture nvcc lists and links Aluminum/MPI/NCCL.
"""
from __future__ import annotations

import os
import shutil
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
EXT_NAME = "_bagua_core_b200"
SO_PATH = os.path.join(PKG_DIR, EXT_NAME + ".so")
BUILD_DIR = os.path.join(PKG_DIR, "build")

SOURCES = [
    "bindings.cc",
    "runtime/backend.cc",
    "runtime/timeline.cc",
    "pool/resource_pool.cc",
    "tensor/tensor.cc",
    "comm/communicator.cc",
    "comm/arena.cc",
    "comm/nvls.cc",
    "comm/nccl_transport.cc",
    "comm/c10d_transport.cc",
    "comm/solo_transport.cc",
    "ops/ops.cc",
    "telemetry/telemetry.cc",
    "capi/capi.cc",
    "kernels/cpu_kernels.cc",
    "kernels/elementwise.cu",
    "kernels/minmax_uint8.cu",
    "kernels/multi_copy.cu",
    "kernels/fused_allreduce.cu",
    "kernels/fused_allreduce_ce.cu",
    "kernels/fused_bytegrad.cu",
    "kernels/fused_gossip.cu",
    "kernels/fused_collectives.cu",
    "kernels/fused_nvls.cu",
    "kernels/fused_emu.cc",
    "kernels/no_alloc.cu",
    "kernels/model_ops.cu",
    "kernels/model_ops_cpu.cc",
]


def _nccl_paths():
    """Header and library of the NCCL build torch itself links (same process, same symbols)."""
    import torch

    site = os.path.dirname(os.path.dirname(torch.__file__))
    inc = os.path.join(site, "nvidia", "nccl", "include")
    lib = os.path.join(site, "nvidia", "nccl", "lib")
    if os.path.exists(os.path.join(inc, "nccl.h")) and os.path.exists(os.path.join(lib, "libnccl.so.2")):
        return inc, lib
    return "/usr/include", "/usr/lib/x86_64-linux-gnu"


def _shared_libstdcxx_flags():
    """Linker flags that pin the system's shared libstdc++.so.6 (empty if it cannot be found)."""
    for d in ("/usr/lib/x86_64-linux-gnu", "/usr/lib64", "/lib/x86_64-linux-gnu", "/usr/lib/aarch64-linux-gnu"):
        if os.path.exists(os.path.join(d, "libstdc++.so.6")):
            return [f"-L{d}", "-l:libstdc++.so.6"]
    return []


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def is_stale() -> bool:
    if not os.path.exists(SO_PATH):
        return True
    so_mtime = os.path.getmtime(SO_PATH)
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".cc", ".cu", ".h", ".cuh")) and os.path.getmtime(os.path.join(root, f)) > so_mtime:
                return True
    return False


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile (if anything changed) and return the path of the shared object."""
    if not force and not is_stale():
        return SO_PATH
    from torch.utils import cpp_extension

    os.makedirs(BUILD_DIR, exist_ok=True)
    nccl_inc, nccl_lib = _nccl_paths()
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 8))
    cpp_extension.load(
        name=EXT_NAME,
        sources=sources(),
        extra_cflags=["-O2", "-std=c++17", "-fvisibility=hidden", "-Wno-attributes"],
        extra_cuda_cflags=[
            "-O3",
            "-std=c++17",
            "-gencode",
            "arch=compute_100a,code=sm_100a",
            "-lineinfo",
            "-Xcompiler",
            "-fvisibility=hidden",
        ],
        extra_include_paths=[nccl_inc, CSRC],
        # The shared C++ runtime is named explicitly and first.  Some toolchain wrappers
        # resolve a bare -lstdc++ to the static archive; an extension carrying its own copy
        # of libstdc++ next to the one torch uses has two sets of locale facets, and the
        # first number streamed into a std::ostream crashes.
        extra_ldflags=_shared_libstdcxx_flags()
        + [f"-L{nccl_lib}", "-l:libnccl.so.2", f"-Wl,-rpath,{nccl_lib}", "-lcudart"],
        build_directory=BUILD_DIR,
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    built = os.path.join(BUILD_DIR, EXT_NAME + ".so")
    tmp = SO_PATH + ".tmp"
    shutil.copyfile(built, tmp)
    os.replace(tmp, SO_PATH)
    return SO_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
