from .spec import (CollectiveSpecBroadcast, CollectiveSpecPartial, CollectiveSpecSplit,  # noqa: F401
                   CollectiveSpecUnique)
from .tensor import CollectiveTensor  # noqa: F401
from .quantized import (ColumnParallelQLinear, RowParallelQLinear, shard_gptq_column,  # noqa: F401
                        shard_gptq_row)
from .fused import FusedAllReduce  # noqa: F401
from . import dispatch as _dispatch  # noqa: F401
