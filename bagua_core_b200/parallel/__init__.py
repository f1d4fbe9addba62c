"""Data-parallel training layer: process groups, flat buckets, `with_bagua` and the algorithms."""
from .algorithms import (  # noqa: F401
    Algorithm,
    AsyncModelAverageAlgorithm,
    ByteGradAlgorithm,
    DecentralizedAlgorithm,
    GradientAllReduceAlgorithm,
    LowPrecisionDecentralizedAlgorithm,
    QAdamAlgorithm,
    QAdamOptimizer,
)
from .bucket import BaguaBucket, BaguaTensor, split_into_buckets  # noqa: F401
from .collectives import (  # noqa: F401
    ReduceOp,
    allgather,
    allgather_inplace,
    allreduce,
    allreduce_inplace,
    alltoall,
    alltoall_inplace,
    alltoall_v,
    barrier,
    broadcast,
    gather,
    gather_inplace,
    recv,
    reduce,
    reduce_inplace,
    reduce_scatter,
    reduce_scatter_inplace,
    scatter,
    scatter_inplace,
    send,
)
from .communication import (  # noqa: F401
    BaguaProcessGroup,
    destroy_process_group,
    get_local_rank,
    get_process_group,
    get_rank,
    get_world_size,
    init_process_group,
)
from .distributed import BaguaModule, with_bagua  # noqa: F401
from .optim import FlatSGD  # noqa: F401
