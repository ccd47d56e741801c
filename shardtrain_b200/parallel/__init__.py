"""Legacy synchronous tensor / sequence parallelism (the runtime has its own split-phase path)."""
from shardtrain_b200.parallel.mappings import (  # noqa: F401
    TPGroup, copy_to_tp, gather_sequence, reduce_from_tp, reduce_scatter_sequence,
)
from shardtrain_b200.parallel.model import TensorParallelPlan, parallelize_tp_sp  # noqa: F401
