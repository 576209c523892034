"""Optimizer shell of the layer (interface of MOLE/optim/mixed_optim.py)."""
from .mixed_optim import CPUAdam, MOLEMixedAdam  # noqa: F401
