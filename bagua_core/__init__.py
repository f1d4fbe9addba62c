"""Drop-in `bagua_core` module: the four classes and `show_version` of the reference's
pyo3 module (bagua-core-py/src/lib.rs:506-514; python/bagua_core/__init__.py:1-4),
served by the B200-native engine."""
from ._environment import _preload_libraries

_preload_libraries()

from bagua_core_b200 import (  # noqa: E402  # noqa: F401
    BaguaBucketPy,
    BaguaCommBackendPy,
    BaguaSingleCommunicatorPy,
    BaguaTensorPy,
    show_version,
)
from .version import __version__  # noqa: F401
