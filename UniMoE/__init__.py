"""Import alias: the reference's own sources import the package as ``UniMoE`` (e.g.
MOLE/moe/layer.py:3-13).  ``UniMoE.moe.layer``, ``UniMoE.utils.*`` and ``UniMoE.core`` resolve to
the modules of ``mole_b200``."""
import importlib
import sys

import mole_b200

_ALIASES = ["moe", "moe.layer", "moe.functions", "utils", "utils.Ugate", "utils.Uparam",
            "utils.Ustream", "utils.Udist", "utils.Uact", "utils.Utimer", "core"]
for _name in _ALIASES:
    sys.modules[f"{__name__}.{_name}"] = importlib.import_module(f"mole_b200.{_name}")
moe, utils, core = mole_b200.moe, mole_b200.utils, sys.modules[f"{__name__}.core"]
