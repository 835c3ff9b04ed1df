"""Build libdeepity_b200.so (CUDA kernels + C ABI + host networks) in-tree with nvcc.

    python -m deepity_b200.build [--force]

Targets sm_100a only.  The library links the CUDA runtime statically and resolves the
driver's tensor-map encoder at run time, so it has no link-time dependency beyond libstdc++.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OUT = os.path.join(PKG, "libdeepity_b200.so")

SOURCES = ["dpc_core.cu", "dpc_tc.cu", "dpc_static.cu", "dpc_conv.cu",
           os.path.join("host", "pc_network.cpp"), os.path.join("host", "conv_network.cpp")]
HEADERS = ["dpc_internal.h", "dpc_math.cuh", "dpc_simt.cuh", os.path.join("host", "pc_network.h"),
           os.path.join("host", "conv_network.h"),
           os.path.join(ROOT, "include", "deepity_b200.h")]


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA 12.9 toolkit is required to build")
    return cand


def up_to_date() -> bool:
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + \
           [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS] + \
           [os.path.abspath(__file__)]
    deps += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".cu"))]
    return all(os.path.getmtime(d) <= t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return OUT
    cmd = [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
        "-std=c++17", "-ftz=true", "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2",
        "-I", os.path.join(ROOT, "include"), "-I", CSRC,
        *[os.path.join(CSRC, s) for s in SOURCES],
        "-o", OUT,
    ]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    print("[deepity_b200] building", OUT, file=sys.stderr)
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
