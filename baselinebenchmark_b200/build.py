"""Builds libmoba_b200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
SOURCES = ["api.cu", "gate.cu", "routes.cu", "attend_mma.cu", "attend_tc5.cu", "attend_bwd.cu", "attend_bwd_tc5.cu", "attend_bwd_dkdv_tc5.cu", "route_static.cu", "nccl_dl.cu"]
LIB = PKG / "libmoba_b200.so"


def nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def build(verbose: bool = False, force: bool = False) -> Path:
    srcs = [PKG / "csrc" / s for s in SOURCES]
    deps = srcs + list((PKG / "csrc").glob("*.cuh")) + [ROOT / "include" / "moba_b200.h"]
    if not force and LIB.exists() and all(LIB.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return LIB
    cmd = [nvcc(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
           "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", str(ROOT / "include"), "-I", str(PKG / "csrc"),
           "-o", str(LIB)] + [str(s) for s in srcs] + ["-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libmoba_b200.so")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force=True))
