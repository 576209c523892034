"""Import alias: the reference's setup.py (setup.py:10,21) packages the code as ``MOLE``.
``MOLE.moe.layer``, ``MOLE.utils.*`` and ``MOLE.core`` resolve to the modules of ``mole_b200``."""
import importlib
import sys

import mole_b200

_ALIASES = ["moe", "moe.layer", "moe.functions", "utils", "utils.Ugate", "utils.Uparam",
            "utils.Ustream", "utils.Udist", "utils.Uact", "utils.Utimer", "utils.Uscheduler",
            "optim", "optim.mixed_optim", "core"]
for _name in _ALIASES:
    sys.modules[f"{__name__}.{_name}"] = importlib.import_module(f"mole_b200.{_name}")
# the reference's scheduler imports the layer module under this name (MOLE/utils/Uscheduler.py:2)
sys.modules[f"{__name__}.moe.MOLE"] = sys.modules[f"{__name__}.moe.layer"]
moe, utils, core = mole_b200.moe, mole_b200.utils, sys.modules[f"{__name__}.core"]
optim = sys.modules[f"{__name__}.optim"]
