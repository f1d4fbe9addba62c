"""Loader of the native extension.

The shared object is built in-tree by `bagua_core_b200._build.build()` and imported from
its file path.  If it is missing and a CUDA toolchain is present it is built on first
import; otherwise importing fails loudly — there is no pure-Python fallback for the
communication engine.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import torch  # noqa: F401  (loads libtorch / libc10 / NCCL before the extension)

from . import _build

_MOD_NAME = "bagua_core_b200." + _build.EXT_NAME


def _load():
    if _MOD_NAME in sys.modules:
        return sys.modules[_MOD_NAME]
    path = _build.SO_PATH
    if not os.path.exists(path):
        import shutil

        if shutil.which("nvcc") is None:
            raise ImportError(
                f"{path} is missing and nvcc is not on PATH; build it with "
                "`python -m bagua_core_b200._build` on a machine with the CUDA toolkit"
            )
        _build.build()
    spec = importlib.util.spec_from_file_location(_MOD_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[_MOD_NAME] = mod
    spec.loader.exec_module(mod)
    return mod


C = _load()
SO_PATH = _build.SO_PATH


def _drop_multicast_bindings():
    # A process must not die while its memory is bound to an NVSwitch multicast object that
    # other GPUs still use; communicators that were never destroyed are covered here.
    try:
        C.release_multicast_slabs()
    except Exception:
        pass


import atexit  # noqa: E402

atexit.register(_drop_multicast_bindings)
