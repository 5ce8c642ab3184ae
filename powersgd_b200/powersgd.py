"""Import-path parity with the reference's `powersgd.powersgd` module."""
from .aggregators import (  # noqa: F401
    Aggregator,
    AllReduce,
    BasicConfig,
    BasicPowerSGD,
    Config,
    PowerSGD,
    batch_transpose,
    view_as_matrix,
)
from .plan import avg_compressed_size  # noqa: F401
