"""In-tree build of libkda_b200.so (nvcc, sm_100a only).

``python -m kda_ascendc_b200.build`` compiles the three CUDA sources under
``csrc/`` into ``kda_ascendc_b200/libkda_b200.so``.  nvcc cross-compiles without a
GPU, so the same command serves the build check on a CPU-only machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libkda_b200.so"
SOURCES = ["kda_c_api.cu", "kda_k1_sm100.cu", "kda_k2_sm100.cu", "kda_k2la_sm100.cu", "kda_k2m_sm100.cu", "kda_k2t_sm100.cu", "kda_recurrent_sm100.cu", "kda_fold_sm100.cu", "kda_peer_sm100.cu",
           "kda_selftest.cu", "kda_static_scratch.cu"]
HEADERS = ["kda_common.cuh", "kda_kernels.h", "../../include/kda_b200.h"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = sources() + [(CSRC / h).resolve() for h in HEADERS]
    return any(d.exists() and d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    tmp = LIB_PATH.with_suffix(".so.tmp%d" % os.getpid())
    cmd += ["-o", str(tmp), *[str(s) for s in sources()]]
    proc = subprocess.run(cmd, cwd=str(CSRC), capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), proc.stderr[-4000:]))
    if verbose:
        sys.stderr.write(proc.stderr)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
