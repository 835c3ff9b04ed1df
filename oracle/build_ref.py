"""Build the oracle: the reference's own CPU train-step path, compiled where it lies.

Test infrastructure only.  Compiles the reference sources for the Simple /
DirectKP / Full / SimpleConv predictive-coding networks and the CPU backend straight
from the reference checkout (environment variable ``DEEPITY_REFERENCE``, else the
default of ``reference_root()``), together with ``ref_driver.cpp`` and
``ref_conv_driver.cpp`` (flat C interfaces) and ``shim_kernels.cpp`` (scalar
restatements of the few Highway / scalar-SLEEF symbols this image lacks), into
``oracle/_ref/libdeepity_ref.so``.  The reference's own CMake build cannot run
offline (it fetches SLEEF, Highway, oneDNN, CUTLASS and nanobind), so the handful
of source files are handed to g++ directly.  oneDNN and MKL paths are off; GEMMs
go to the OpenBLAS bundled with scipy, vector SLEEF symbols come from
``libtorch_cpu``.

Outputs go only to ``oracle/_ref/`` (git-ignored).  Nothing is copied from the
reference into this repository.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libdeepity_ref.so")

REF_SOURCES = [
    "src/networks/DirectKPPCNetwork.cpp",
    "src/networks/SimplePCNetwork.cpp",
    "src/networks/FullPCNetwork.cpp",
    "src/networks/SimpleConvPCNetwork.cpp",
    "src/layers/SimpleConvPCLayer.cpp",
    "src/layers/DirectKPPCLayer.cpp",
    "src/layers/SimplePCLayer.cpp",
    "src/layers/FullPCLayer.cpp",
    "src/backend/CPUBackend.cpp",
    "src/backend/Backend.cpp",
    "src/backend/CUDAPluginLoader.cpp",
]


def reference_root() -> str | None:
    root = os.environ.get("DEEPITY_REFERENCE", "/root/reference")
    return root if os.path.isdir(os.path.join(root, "src", "networks")) else None


def site_packages() -> str:
    return sysconfig.get_paths()["purelib"]


def build(verbose: bool = True) -> str | None:
    """Compile the oracle if the reference checkout is present.

    Returns the path of the shared library, or None when the reference is not
    available (then a previously built library, if any, is used as is).
    """
    root = reference_root()
    if root is None:
        return OUT if os.path.exists(OUT) else None
    sp = site_packages()
    blas = glob.glob(os.path.join(sp, "scipy.libs", "libscipy_openblas*.so"))
    if not blas:
        raise RuntimeError("scipy's bundled OpenBLAS not found")
    torch_lib = os.path.join(sp, "torch", "lib")
    srcs = [os.path.join(root, s) for s in REF_SOURCES]
    mine = [os.path.join(HERE, "ref_driver.cpp"), os.path.join(HERE, "ref_conv_driver.cpp"),
            os.path.join(HERE, "shim_kernels.cpp")]
    newest = max(os.path.getmtime(p) for p in srcs + mine + [os.path.abspath(__file__)])
    if os.path.exists(OUT) and os.path.getmtime(OUT) >= newest:
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [
        "g++", "-std=c++20", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared",
        # the host as a CUDA-enabled build of the reference compiles it: DEVICE_GPU networks bind
        # device arenas and reach their backend through the plugin loader (no CUDA header needed)
        "-DDEEPITY_USE_CUDA",
        "-I", os.path.join(HERE, "shim"),
        "-I", os.path.join(root, "include"),
        "-I", os.path.join(root, "src", "backend"),
        "-I", os.path.join(sp, "torch", "include"),
        *mine, *srcs,
        "-o", OUT,
        "-L", torch_lib, "-ltorch_cpu", "-lc10",
        blas[0],
        "-ldl",
        f"-Wl,-rpath,{torch_lib}",
        f"-Wl,-rpath,{os.path.dirname(blas[0])}",
    ]
    if verbose:
        print("[oracle] building", OUT, file=sys.stderr)
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build())
