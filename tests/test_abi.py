"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "mole_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(mole_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_groups():
    names = declared_symbols()
    for must in ("mole_gate_route_fwd", "mole_dispatch_fwd", "mole_combine_fwd", "mole_ffn_fwd",
                 "mole_ffn_bwd", "mole_all2all", "mole_pool_fetch", "mole_ctx_create"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from mole_b200 import _lib
    for name in declared_symbols():
        assert hasattr(_lib.lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(declared_symbols())


def test_no_torch_types_in_signatures():
    code = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)     # comments stripped
    assert "at::" not in code and "Tensor" not in code and "torch" not in code.lower()
    assert "#include <stdint.h>" in code and code.count("#include") == 1


def test_argument_validation_needs_no_gpu():
    from mole_b200 import _lib
    lib = _lib.lib
    assert lib.mole_version() >= 100
    assert _lib.capacity_stride(1) == 128 and _lib.capacity_stride(320) == 384
    assert _lib.capacity_stride(640) == 640
    n = C.c_int64()
    assert lib.mole_route_workspace_bytes(4096, 8, 2, C.byref(n)) == 0 and n.value > 0
    assert lib.mole_route_workspace_bytes(4096, 1000, 2, C.byref(n)) == -1      # too many experts
    assert b"E=1000" in lib.mole_last_error_string()
    assert lib.mole_route_workspace_bytes(4096, 8, 9, C.byref(n)) == -1         # k > E
    d = _lib.FfnDesc(dtype=1, act=0, gelu_bwd=0, M=1000, F=4096, L=8, n_src=1, Cs=128, e_begin=0,
                     e_end=8, n_slots=8, n_grad_slots=0, accumulate=0, compact=0, backend=0)
    assert lib.mole_ffn_workspace_bytes(C.byref(d), C.byref(n)) == -1           # M % 64 != 0
    d.M = 192                                                                   # bf16 needs % 128
    assert lib.mole_ffn_workspace_bytes(C.byref(d), C.byref(n)) == -4
    d.M = 1024
    assert lib.mole_ffn_workspace_bytes(C.byref(d), C.byref(n)) == 0 and n.value > 0
    d.Cs = 100
    assert lib.mole_ffn_workspace_bytes(C.byref(d), C.byref(n)) == -1
    with pytest.raises(_lib.MoleError):
        _lib.check(lib.mole_ffn_workspace_bytes(C.byref(d), C.byref(n)))


def test_product_package_never_imports_the_oracle():
    for path in (ROOT / "mole_b200").rglob("*.py"):
        src = path.read_text()
        assert "oracle" not in src, f"{path} mentions the oracle"
