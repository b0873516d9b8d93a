"""Build the CUDA library in-tree for sm_100a: ``python build.py`` (nvcc only, no GPU needed)."""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIBRARY = HERE / "lib" / "libhygemm_b200.so"
SOURCES = ["hg_quant.cu", "hg_gemm_simt.cu", "hg_gemm_tc.cu", "hg_runtime.cu", "hg_tp.cu", "hg_clip.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-shared", "-cudart", "static"]


def stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "hygemm.h"]
    return any(d.stat().st_mtime > built for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel into ``lib/libhygemm_b200.so``; returns its path."""
    if not force and not stale():
        return LIBRARY
    LIBRARY.parent.mkdir(exist_ok=True)
    cmd = ["nvcc", *FLAGS, *(["-Xptxas", "-v"] if verbose else []), *[str(CSRC / s) for s in SOURCES], "-o", str(LIBRARY)]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode:
        raise RuntimeError("nvcc failed building libhygemm_b200.so")
    return LIBRARY


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
