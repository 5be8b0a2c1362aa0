"""Expert-parallel placement rules and runtime bootstrap helpers.

The placement is the reference's (intranode_dispatch.cu:133-134): experts are
block-partitioned over ranks, and ranks ``[g * dp_size, (g + 1) * dp_size)`` form a
DP group that holds the same tokens.
"""

from .placement import (
    EPLayout as EPLayout,
)
from .runtime import (
    finalize_runtime as finalize_runtime,
    init_runtime_from_torch as init_runtime_from_torch,
)
