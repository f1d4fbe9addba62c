"""bagua_core_b200 — a Blackwell-native distributed-training communication engine with
the capabilities and Python API of BaguaSys/bagua-core.

Layers (top to bottom):

* ``bagua_core_b200.parallel``  – ``with_bagua``-style model wrapper, bucketing, the
  training algorithms (gradient all-reduce, ByteGrad, decentralized, low-precision
  decentralized, QAdam, async model average);
* ``bagua_core_b200.models``    – benchmark model definitions (VGG-16, BERT-large,
  ResNet-50, MLP);
* ``bagua_core_b200.ops``       – Python entry points of the sm_100a tensor kernels;
* the native extension          – scheduler, tensors/buckets, communicators, peer arena,
  fused communication kernels (``BaguaCommBackendPy`` etc., re-exported here and by the
  ``bagua_core`` compatibility package).
"""
from ._native import C as _C
from ._native import SO_PATH

BaguaSingleCommunicatorPy = _C.BaguaSingleCommunicatorPy
BaguaTensorPy = _C.BaguaTensorPy
BaguaBucketPy = _C.BaguaBucketPy
BaguaCommBackendPy = _C.BaguaCommBackendPy
show_version = _C.show_version

__version__ = "0.1.0"

# reduction-op codes of the `op` arguments (reference: datatypes/mod.rs:24-38)
class ReduceOp:
    SUM, PROD, MIN, MAX, LOR, LAND, LXOR, BOR, BAND, BXOR, AVG = range(11)


__all__ = [
    "BaguaSingleCommunicatorPy",
    "BaguaTensorPy",
    "BaguaBucketPy",
    "BaguaCommBackendPy",
    "show_version",
    "ReduceOp",
    "__version__",
]
