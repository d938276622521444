"""Builds libfastdms_b200.so (the C-ABI library) in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libfastdms_b200.so"
SOURCES = ["store_decode.cu", "attn_decode.cu", "expiry.cu", "pack_prefill.cu", "metadata.cu", "kv_quant.cu",
           "elementwise.cu", "allreduce.cu", "prefix_attention.cu", "skinny_gemm.cu", "linear_allreduce.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared", "--use_fast_math", "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the fastdms_b200 CUDA library cannot be built")
    return exe


def needs_build() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) +
                 [PKG.parent / "include" / "fastdms_b200.h"])
    return newest > LIB.stat().st_mtime


PROBE_LIB = PKG / "libfastdms_b200_probe.so"


def build(force: bool = False, verbose: bool = False, probe: bool = False) -> Path:
    """Compile every kernel for sm_100a into one shared library next to the package.  `probe=True`
    builds a second library, libfastdms_b200_probe.so, whose attention kernels record phase timestamps
    (-DFDMS_ATTN_PROBE); load it by setting FDMS_B200_LIB to its path."""
    if probe:
        cmd = [_nvcc(), *NVCC_FLAGS, "-DFDMS_ATTN_PROBE", "-o", str(PROBE_LIB), *[str(CSRC / s) for s in SOURCES]]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            print(proc.stdout, proc.stderr)
            raise RuntimeError(f"nvcc failed with exit code {proc.returncode}")
        return PROBE_LIB
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(LIB), *[str(CSRC / s) for s in SOURCES]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        print(proc.stdout)
        print(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {proc.returncode}")
    (PKG / "build_ptxas.log").write_text(proc.stderr)
    return LIB


if __name__ == "__main__":
    import sys
    if "--probe" in sys.argv:
        print(build(probe=True))
    else:
        build(force=True, verbose=True)
