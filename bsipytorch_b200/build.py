"""In-tree build of the native parts.

* ``libbsi_b200.so``  -- the C-ABI library (``include/bsi_b200.h``): hand-written CUDA for
  sm_100a only, no torch dependency, static CUDA runtime, so a C / cgo / JNI / ctypes caller
  can load it on its own.
* ``bsi_ops*.so``     -- the pybind11 extension that mirrors the reference's ``bsi_ops``
  module on top of that library (torch tensors in, capsules out).

Both land next to this file; object files go to ``bsipytorch_b200/build/``. A target is
rebuilt only when one of its inputs changed (content hash), so calling ``build()`` at import
time of a test run is cheap.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libbsi_b200.so")
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
EXT = os.path.join(PKG, "bsi_ops" + EXT_SUFFIX)

CUDA_SOURCES = ["common.cu", "pack.cu", "ewah.cu", "dot.cu", "dot_tcgen05.cu", "dot_bmma.cu", "peer.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _hash(paths, extra="") -> str:
    h = hashlib.sha1(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(os.path.basename(p).encode())
            h.update(f.read())
    return h.hexdigest()


def _stamp_ok(stamp, want, *outputs) -> bool:
    if not all(os.path.exists(o) for o in outputs) or not os.path.exists(stamp):
        return False
    with open(stamp) as f:
        return f.read().strip() == want


def _headers():
    hs = [os.path.join(CSRC, n) for n in os.listdir(CSRC) if n.endswith((".cuh", ".h"))]
    hs.append(os.path.join(ROOT, "include", "bsi_b200.h"))
    return hs


def build_lib(verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = _headers()
    objs, jobs = [], []
    for name in CUDA_SOURCES:
        src = os.path.join(CSRC, name)
        obj = os.path.join(OBJ, name[:-3] + ".o")
        stamp = obj + ".stamp"
        want = _hash([src] + headers, " ".join(NVCC_FLAGS))
        objs.append(obj)
        if not _stamp_ok(stamp, want, obj):
            jobs.append((src, obj, stamp, want))

    def compile_one(job):
        src, obj, stamp, want = job
        cmd = ["nvcc"] + NVCC_FLAGS + ["-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        with open(stamp, "w") as f:
            f.write(want)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(compile_one, jobs))
    link_stamp = os.path.join(OBJ, "libbsi_b200.stamp")
    want = _hash(objs)
    if jobs or not _stamp_ok(link_stamp, want, LIB):
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        with open(link_stamp, "w") as f:
            f.write(_hash(objs))
    return LIB


def build_ext(verbose: bool = False) -> str:
    """The pybind11 ``bsi_ops`` module: plain C++ against libtorch, linked to libbsi_b200.so."""
    build_lib(verbose)
    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "bsi_ops_module.cpp")
    stamp = os.path.join(OBJ, "bsi_ops.stamp")
    want = _hash([src, os.path.join(ROOT, "include", "bsi_b200.h")], torch.__version__ + EXT_SUFFIX)
    if _stamp_ok(stamp, want, EXT):
        return EXT
    os.makedirs(OBJ, exist_ok=True)
    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"], "-I", os.path.join(ROOT, "include")]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-DTORCH_EXTENSION_NAME=bsi_ops", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-Wno-attributes"] + inc + [
           src, "-o", EXT,
           "-L" + PKG, "-lbsi_b200", "-Wl,-rpath,$ORIGIN",
           "-L" + torch_lib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda", "-ltorch_python",
           "-Wl,-rpath," + torch_lib]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    with open(stamp, "w") as f:
        f.write(want)
    return EXT


def build(verbose: bool = False):
    return build_lib(verbose), build_ext(verbose)


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
