"""Build libdeepity_b200.so (CUDA kernels + C ABI + host networks) in-tree with nvcc, and
libDeepityCUDA.so, the plugin an unmodified reference host loads for DEVICE_GPU.

    python -m deepity_b200.build [--force] [--plugin]

Targets sm_100a only.  The libraries link the CUDA runtime statically and resolve the
driver's tensor-map encoder at run time, so they have no link-time dependency beyond libstdc++.

The plugin implements the reference's backend interface, so its vtable object is compiled
against the reference's own interface header: it needs the reference checkout (environment
variable DEEPITY_REFERENCE, else the default location below) and a sleef.h (the reference's headers
include it; the one shipped inside torch's include tree is used).  Without the checkout the
plugin is skipped and a previously built libDeepityCUDA.so is used as is.
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


PLUGIN_OUT = os.path.join(PKG, "libDeepityCUDA.so")
PLUGIN_DIR = os.path.join(CSRC, "plugin")


def reference_include() -> str | None:
    root = os.environ.get("DEEPITY_REFERENCE", "/root/reference")
    inc = os.path.join(root, "include")
    return inc if os.path.exists(os.path.join(inc, "deepity", "backend", "IComputeBackend.h")) else None


def build_plugin(force: bool = False) -> str | None:
    """libDeepityCUDA.so: deepity_cuda_plugin.cpp (host compiler, reference interface header) +
    b200_backend.cu (nvcc).  Returns its path, or None when it cannot be built here and no
    earlier build exists."""
    inc = reference_include()
    if inc is None:
        return PLUGIN_OUT if os.path.exists(PLUGIN_OUT) else None
    srcs = [os.path.join(PLUGIN_DIR, f) for f in os.listdir(PLUGIN_DIR)] + \
           [os.path.join(CSRC, "dpc_tcgen05.cuh"), os.path.abspath(__file__)]
    if not force and os.path.exists(PLUGIN_OUT) and \
            all(os.path.getmtime(f) <= os.path.getmtime(PLUGIN_OUT) for f in srcs):
        return PLUGIN_OUT
    import sysconfig
    torch_inc = os.path.join(sysconfig.get_paths()["purelib"], "torch", "include")
    obj_dir = os.path.join(PKG, "build")
    os.makedirs(obj_dir, exist_ok=True)
    vtable_o = os.path.join(obj_dir, "deepity_cuda_plugin.o")
    print("[deepity_b200] building", PLUGIN_OUT, file=sys.stderr)
    subprocess.run(["g++", "-std=c++20", "-O2", "-march=x86-64-v3", "-fopenmp", "-fPIC",
                    "-fvisibility=hidden", "-I", inc, "-I", torch_inc, "-I", PLUGIN_DIR,
                    "-c", os.path.join(PLUGIN_DIR, "deepity_cuda_plugin.cpp"), "-o", vtable_o],
                   check=True)
    subprocess.run([nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
                    "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2",
                    "-I", CSRC, os.path.join(PLUGIN_DIR, "b200_backend.cu"), vtable_o,
                    "-Xlinker", "-lgomp", "-o", PLUGIN_OUT], check=True)
    return PLUGIN_OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--plugin" in sys.argv:
        print(build_plugin(force="--force" in sys.argv))
