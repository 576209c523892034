"""mole_b200 -- B200-native (sm_100a) implementation of the MOLE MoE-layer hot path.

``MOLEModule`` keeps the reference's Python surface (MOLE/moe/layer.py); underneath, PyTorch
host code calls ``libmole_b200.so`` (C ABI in ``include/mole_b200.h``).  Importing the package
loads that library and fails loudly when it has not been built (``python mole_b200/build.py``).
"""
from . import _lib, ops                      # noqa: F401  (loads the shared library)
from .moe.layer import MOLEModule            # noqa: F401
from .moe.functions import BatchFusedFWD, pfetchbwd   # noqa: F401
from .utils.Ugate import MOLETopk            # noqa: F401

__all__ = ["MOLEModule", "MOLETopk", "BatchFusedFWD", "pfetchbwd", "ops"]
