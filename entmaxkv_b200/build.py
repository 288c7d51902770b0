"""Build recipe of ``libentmaxkv_b200.so`` (nvcc, sm_100a only, in-tree)."""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libentmaxkv_b200.so")
SOURCES = ["ekv_cache.cu", "ekv_topk.cu", "ekv_gaussian.cu", "ekv_decode.cu", "ekv_exchange.cu",
           "ekv_fused_small.cu", "ekv_stream_topk.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put /usr/local/cuda/bin on PATH")


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "entmaxkv_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    """Compile every kernel for sm_100a into one shared library; returns its path."""
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS]
    if ptxas_info:
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("EKV_NVCC_EXTRA", "").split()      # e.g. -DEKV_FUSED_TIMING for a development build
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB]
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose or ptxas_info:
        sys.stderr.write(res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build_library(force=True, verbose=True, ptxas_info="--ptxas" in sys.argv))
