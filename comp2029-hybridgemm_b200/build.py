"""Build the CUDA library in-tree for sm_100a: ``python build.py`` (nvcc only, no GPU needed)."""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIBRARY = HERE / "lib" / "libhygemm_b200.so"
TRACE_LIBRARY = HERE / "lib" / "libhygemm_b200_trace.so"   # same sources with -DHG_TRACE (per-CTA time stamps)
SOURCES = ["hg_quant.cu", "hg_gemm_simt.cu", "hg_gemm_tc.cu", "hg_runtime.cu", "hg_tp.cu", "hg_clip.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-shared", "-cudart", "static"]


def stale(library: Path = LIBRARY) -> bool:
    if not library.exists():
        return True
    built = library.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "hygemm.h"]
    return any(d.stat().st_mtime > built for d in deps)


def build_library(force: bool = False, verbose: bool = False, trace: bool = False) -> Path:
    """Compile every kernel into ``lib/libhygemm_b200.so`` (``trace``: the diagnostic twin
    ``lib/libhygemm_b200_trace.so``, whose GEMM kernel records per-CTA time stamps); returns its path."""
    library = TRACE_LIBRARY if trace else LIBRARY
    if not force and not stale(library):
        return library
    library.parent.mkdir(exist_ok=True)
    cmd = ["nvcc", *FLAGS, *(["-DHG_TRACE=1"] if trace else []), *(["-Xptxas", "-v"] if verbose else []),
           *[str(CSRC / s) for s in SOURCES], "-o", str(library)]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode:
        raise RuntimeError(f"nvcc failed building {library.name}")
    return library


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
