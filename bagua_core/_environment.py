"""Library preloading, kept for parity with the reference's package shell
(python/bagua_core/_environment.py:5-8 preloads a bundled libnccl.so before the native
module is imported).  Here NCCL is the copy that ships with torch: importing torch maps it,
so the native extension resolves its NCCL symbols against the same library."""


def _preload_libraries() -> None:
    import torch  # noqa: F401  (maps libtorch, libc10 and torch's libnccl.so.2)
