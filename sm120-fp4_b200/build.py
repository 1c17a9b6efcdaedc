"""Build recipe of the CUDA library: nvcc, sm_100a only, one shared object next to the package.

    python sm120-fp4_b200/build.py [--verbose]

The shared object exports the C ABI declared in include/b200moe.h and nothing else that a caller needs.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libb200moe.so"
SOURCES = ["capi.cu", "layout_quant.cu", "route.cu", "decode.cu", "decode_tc.cu", "prefill.cu", "ep.cu", "umma_probe.cu", "stream_probe.cu"]
FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr", "-Xptxas", "-v"]


DIAG = "--diag" in sys.argv or os.environ.get("B200MOE_DIAG") == "1"
if DIAG:
    # diagnostic build (libb200moe_diag.so, loaded with B200MOE_LIB=<path>): per-worker cycle counters in the decode kernel,
    # ablation switches of the prefill GEMM, and the entry points of include/b200moe_diag.h. Not the library that ships.
    FLAGS += ["-DB200_TIMERS", "-DB200_PF_ABLATE", "-DB200_DIAGNOSTICS"]
    LIB = PKG / "libb200moe_diag.so"


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()] + sorted(p for p in CSRC.glob("*.cu") if p.name not in SOURCES)


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def build(verbose: bool = False, force: bool = False) -> Path:
    if not force and not stale():
        return LIB
    objs = []
    out_dir = PKG / ("build_diag" if DIAG else "build")
    out_dir.mkdir(exist_ok=True)
    procs = []
    for src in sources():
        obj = out_dir / (src.stem + ".o")
        objs.append(obj)
        if obj.exists() and obj.stat().st_mtime > max(p.stat().st_mtime for p in [src] + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))) and not force:
            continue
        cmd = [nvcc(), *FLAGS, "-c", str(src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, pr in procs:
        log, _ = pr.communicate()
        if verbose or pr.returncode:
            print(f"--- {src.name}\n{log}", file=sys.stderr)
        if pr.returncode:
            raise RuntimeError(f"nvcc failed on {src.name}")
    cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode:
        print(r.stdout, file=sys.stderr)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
