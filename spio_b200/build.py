"""Build libspio_b200.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

Run as ``python -m spio_b200.build`` or call :func:`build`.  nvcc cross-compiles for
sm_100a, so no GPU is needed to build.  Plays the role of the reference's Cython build
of its driver shim (setup.py:27-51); the kernels themselves were JIT-only there.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = PKG_DIR / "lib" / "obj"
LIB_PATH = LIB_DIR / "libspio_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-diag-suppress", "177"]


def find_nvcc() -> str:
    """Locate nvcc: $CUDA_HOME, then PATH, then /usr/local/cuda."""
    cands = []
    if os.environ.get("CUDA_HOME"):
        cands.append(Path(os.environ["CUDA_HOME"]) / "bin" / "nvcc")
    which = shutil.which("nvcc")
    if which:
        cands.append(Path(which))
    cands.append(Path("/usr/local/cuda/bin/nvcc"))
    for c in cands:
        if c.exists():
            return str(c)
    raise RuntimeError("nvcc not found; set CUDA_HOME")


def _sources():
    """(source, object, extra flags) for every translation unit."""
    units = [(CSRC / "gw8_capi.cu", OBJ_DIR / "gw8_capi.o", [])]
    for r in range(1, 6):
        units.append((CSRC / "gw8_inst.cu", OBJ_DIR / f"gw8_inst_r{r}.o", [f"-DGW8_R={r}"]))
    units.append((CSRC / "gw8_tc_inst.cu", OBJ_DIR / "gw8_tc_inst.o", []))
    units.append((CSRC / "jit_driver.cpp", OBJ_DIR / "jit_driver.o", []))
    units.append((CSRC / "layernorm_2d.cu", OBJ_DIR / "layernorm_2d.o", []))
    units.append((CSRC / "dp_exchange.cu", OBJ_DIR / "dp_exchange.o", []))
    return units


def _newest_input() -> float:
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    deps += list(CSRC.glob("*.cpp")) + [PKG_DIR.parent / "include" / "spio_b200.h"]
    return max(p.stat().st_mtime for p in deps if p.exists())


def is_current() -> bool:
    """True when the library exists and is newer than every source."""
    return LIB_PATH.exists() and LIB_PATH.stat().st_mtime >= _newest_input()


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(map(str, cmd))}\n{res.stdout}\n{res.stderr}")
    return res.stdout + res.stderr


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every translation unit (in parallel) and link the shared library."""
    if not force and is_current():
        return LIB_PATH
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    flags = ARCH_FLAGS + COMMON_FLAGS + (["-Xptxas", "-v"] if ptxas_info else [])

    def compile_one(unit):
        src, obj, extra = unit
        return _run([nvcc, *flags, *extra, "-c", str(src), "-o", str(obj)], verbose)

    units = _sources()
    with ThreadPoolExecutor(max_workers=min(len(units), os.cpu_count() or 2)) as ex:
        logs = list(ex.map(compile_one, units))
    if ptxas_info:
        print("\n".join(logs))
    objs = [str(obj) for _, obj, _ in units]
    _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB_PATH), *objs, "-ldl"], verbose)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas-info" in sys.argv)
    print(path)
