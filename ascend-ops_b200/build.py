"""In-tree build of the B200 decode operator library.

Produces, next to the Python package:
  ascend910a_extras/lib/libb200ops.so          CUDA kernels + C ABI (no torch dependency)
  ascend910a_extras/ascend910a_extras_C.*.so   torch extension calling the C ABI

The reference builds the same two layers with CMake: the aclnn op library through
csrc/opdev/build.sh and the pybind module from csrc/ffi/*.cpp (CMakeLists.txt:39-113).
Here it is two direct compiler invocations: nvcc for sm_100a (cross-compiles without a
GPU) and g++ against the installed torch headers.

Usage: python build.py [--force] [--no-torch-ext] [--verbose]
"""
from __future__ import annotations

import argparse
import concurrent.futures
import hashlib
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent
CSRC = HERE / "csrc"
PKG = HERE / "ascend910a_extras"
LIB_DIR = PKG / "lib"
OBJ_DIR = HERE / "build"
INCLUDE = REPO / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    f"-I{INCLUDE}", f"-I{CSRC}",
]


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"command failed ({proc.returncode}): {' '.join(str(c) for c in cmd)}")
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout + proc.stderr)


def _stamp(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _headers():
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted(INCLUDE.glob("*.h"))


def build_cuda_library(force=False, verbose=False):
    """Compile every csrc/*.cu for sm_100a and link libb200ops.so."""
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    out = LIB_DIR / "libb200ops.so"
    stamp_file = OBJ_DIR / "libb200ops.stamp"
    stamp = _stamp(sources + _headers(), " ".join(NVCC_FLAGS))
    if not force and out.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return out
    nvcc = os.environ.get("NVCC", "nvcc")
    hdr_stamp = _stamp(_headers(), " ".join(NVCC_FLAGS))

    def compile_one(src):
        obj = OBJ_DIR / (src.stem + ".o")
        ostamp = OBJ_DIR / (src.stem + ".stamp")
        s = _stamp([src], hdr_stamp)
        if not force and obj.exists() and ostamp.exists() and ostamp.read_text() == s:
            return obj
        _run([nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)], verbose)
        ostamp.write_text(s)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=int(os.environ.get("MAX_JOBS", "8"))) as ex:
        objs = list(ex.map(compile_one, sources))
    _run([nvcc, "-shared", "-o", str(out), *map(str, objs), "-gencode",
          "arch=compute_100a,code=sm_100a", "-cudart", "static"], verbose)
    stamp_file.write_text(stamp)
    return out


def build_torch_extension(force=False, verbose=False):
    """Compile csrc/torch_ext.cpp into the module ascend910a_extras_C next to ops.py."""
    import torch
    from torch.utils import cpp_extension

    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    out = PKG / f"ascend910a_extras_C{suffix}"
    src = CSRC / "torch_ext.cpp"
    stamp_file = OBJ_DIR / "torch_ext.stamp"
    stamp = _stamp([src] + sorted(INCLUDE.glob("*.h")), torch.__version__)
    if not force and out.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return out
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    includes = cpp_extension.include_paths() + [sysconfig.get_paths()["include"], str(INCLUDE),
                                                os.path.join(cuda_home, "include")]
    lib_paths = cpp_extension.library_paths()
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=ascend910a_extras_C",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-DUSE_CUDA",
           *[f"-isystem{p}" for p in includes], str(src), "-o", str(out),
           f"-L{LIB_DIR}", "-lb200ops", "-Wl,-rpath,$ORIGIN/lib",
           *[f"-L{p}" for p in lib_paths], *[f"-Wl,-rpath,{p}" for p in lib_paths],
           "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python"]
    _run(cmd, verbose)
    stamp_file.write_text(stamp)
    return out


def build_all(force=False, verbose=False, torch_ext=True):
    lib = build_cuda_library(force, verbose)
    ext = build_torch_extension(force, verbose) if torch_ext else None
    return lib, ext


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--no-torch-ext", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ns = ap.parse_args()
    built = build_all(ns.force, ns.verbose, not ns.no_torch_ext)
    print("built:", *[str(b) for b in built if b])
