"""Activation names of the expert FFN (interface of MOLE/utils/Uact.py).

The layer only stores the callable; the activation itself runs inside the FC1 epilogue of the
grouped GEMM and its derivative inside the dX2 epilogue.
"""
import torch.nn.functional as F

_FWD = {"gelu": F.gelu, "relu": F.relu}


def build_activation_fwd(act: str):
    try:
        return _FWD[act]
    except KeyError:
        raise ValueError(f"unsupported activation {act!r}; the fused epilogues cover 'gelu' and 'relu'")


def build_activation_bwd(act: str):
    if act not in _FWD:
        raise ValueError(f"unsupported activation {act!r}")
    return None
