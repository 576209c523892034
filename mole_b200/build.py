"""Builds ``libmole_b200.so`` in-tree with nvcc for sm_100a.

Run as ``python mole_b200/build.py`` (add ``-v`` for ptxas resource usage); it is loaded by path,
not through the package, because importing the package needs the library it builds.  The library is
a plain C-ABI shared object: no torch headers, no pybind.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT_DIR = HERE / "lib"
LIB = OUT_DIR / "libmole_b200.so"
SOURCES = ["route.cu", "dispatch.cu", "gate_mma.cu", "gemm_simt.cu", "gemm_tc.cu", "ffn.cu", "runtime.cu", "adam.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the CUDA library cannot be built")


def _nccl_include() -> list[str]:
    site = Path(sysconfig.get_paths()["purelib"]) / "nvidia" / "nccl" / "include"
    return ["-I", str(site)] if (site / "nccl.h").exists() else []


def _stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.iterdir()) + [HERE.parent / "include" / "mole_b200.h"])
    return newest > LIB.stat().st_mtime


def build(verbose: bool = False, force: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    OUT_DIR.mkdir(exist_ok=True)
    obj_dir = HERE / "_obj"
    obj_dir.mkdir(exist_ok=True)
    common = [nvcc, *ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", *_nccl_include()]
    if verbose:
        common += ["-Xptxas", "-v"]

    def compile_one(src: str) -> Path:
        obj = obj_dir / (src + ".o")
        cmd = common + ["-c", str(CSRC / src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(f"--- {src}\n{res.stdout}{res.stderr}")
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    link = [nvcc, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-ldl"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("linking libmole_b200.so failed")
    return LIB


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force=True)
    print(path)
