"""powersgd_b200 — PowerSGD low-rank gradient compression, built for B200 (sm_100a).

Public surface (same names as the reference's `powersgd` package, powersgd/__init__.py:3-7):
`PowerSGD`, `Config`, `AllReduce`, `Aggregator`, `optimizer_step`.
"""
from .aggregators import Aggregator, AllReduce, BasicConfig, BasicPowerSGD, Config, PowerSGD
from .optim import optimizer_step
from .utils import params_in_optimizer

__version__ = "0.1.0"

__all__ = [
    "Aggregator",
    "AllReduce",
    "BasicConfig",
    "BasicPowerSGD",
    "Config",
    "PowerSGD",
    "optimizer_step",
    "params_in_optimizer",
]
