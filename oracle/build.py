"""Build recipe for the checkers under ``oracle/``.

Test infrastructure only: nothing in the shipped package imports this module.

Two artefacts, both git-ignored:

* ``oracle/_build/libbsi_oracle.so`` -- the C restatement (``bsi_oracle.c``), compiled
  with ``-march=native`` for the host it runs on; it is rebuilt when the source or the
  host CPU changes, so a library built on one machine is never executed on another.
* ``oracle/_ref/ref_kernels.so`` -- the reference's own CUDA kernels
  (``bsi_ops/csrc/cuda/bsi_cuda_kernels.cu`` and the five ``.cuh`` files it includes),
  compiled for sm_100a straight from the reference checkout. Only built where that
  checkout exists.
* ``oracle/_ref/benchmarks/*.py`` -- the reference's caller scripts (layer replacement,
  dot microbenchmark, tensor-core check, apples-to-apples benchmark), staged unmodified so
  that the GPU tests can run them over this library on a machine without the checkout.
  Git-ignored like the rest of ``_ref``: they never enter the history.

The reference checkout is looked for in ``$BSI_REFERENCE_DIR`` or, when that is unset, in a
directory named ``reference`` beside this repository; when neither exists both steps are skipped.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
REF_DIR = os.path.join(HERE, "_ref")
ORACLE_SO = os.path.join(BUILD_DIR, "libbsi_oracle.so")
REF_SO = os.path.join(REF_DIR, "ref_kernels.so")
REFERENCE_CHECKOUT = os.environ.get("BSI_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
REF_KERNEL_TU = os.path.join(REFERENCE_CHECKOUT, "bsi_ops", "csrc", "cuda", "bsi_cuda_kernels.cu")
REF_CALLERS_DIR = os.path.join(REF_DIR, "benchmarks")
REF_CALLERS = ["verify_accuracy_bsi.py", "benchmark_dot_kernel_micro.py", "verify_tc_dot_correctness.py",
               "benchmark_apples_to_apples_bsi.py"]


def _host_tag() -> str:
    model, flags = "", ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name") and not model:
                    model = line.split(":", 1)[1].strip()
                elif line.startswith("flags") and not flags:
                    flags = line.split(":", 1)[1].strip()
                if model and flags:
                    break
    except OSError:
        pass
    return hashlib.sha1((model + "|" + flags).encode()).hexdigest()[:16]


def _digest(paths) -> str:
    h = hashlib.sha1()
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def build_oracle(force: bool = False) -> str:
    """Compile ``bsi_oracle.c`` for this host (no-op when up to date)."""
    src = os.path.join(HERE, "bsi_oracle.c")
    stamp = os.path.join(BUILD_DIR, "libbsi_oracle.stamp")
    want = _digest([src]) + ":" + _host_tag()
    if not force and os.path.exists(ORACLE_SO) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return ORACLE_SO
    os.makedirs(BUILD_DIR, exist_ok=True)
    cmd = ["gcc", "-O3", "-march=native", "-std=c99", "-fopenmp", "-fPIC", "-shared",
           "-o", ORACLE_SO, src, "-lm"]
    subprocess.run(cmd, check=True)
    with open(stamp, "w") as f:
        f.write(want)
    return ORACLE_SO


def build_ref(force: bool = False):
    """Compile the reference kernels where the reference checkout is present.

    Returns the path of the library, or None when there is neither a checkout nor a
    previously built library."""
    if not os.path.exists(REF_KERNEL_TU):
        return REF_SO if os.path.exists(REF_SO) else None
    srcdir = os.path.dirname(REF_KERNEL_TU)
    srcs = [REF_KERNEL_TU] + sorted(
        os.path.join(srcdir, n) for n in os.listdir(srcdir) if n.endswith(".cuh"))
    stamp = os.path.join(REF_DIR, "ref_kernels.stamp")
    want = _digest(srcs)
    if not force and os.path.exists(REF_SO) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["nvcc", "-O3", "-std=c++20", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC", "-w", "-o", REF_SO, REF_KERNEL_TU]
    subprocess.run(cmd, check=True)
    with open(stamp, "w") as f:
        f.write(want)
    return REF_SO


def stage_reference_callers():
    """Copy the reference's caller scripts, byte for byte, into ``oracle/_ref/benchmarks`` (where the
    checkout is present). Returns the directory, or None when there is nothing staged."""
    import shutil
    src_dir = os.path.join(REFERENCE_CHECKOUT, "bsi_ops", "benchmarks")
    if os.path.isdir(src_dir):
        os.makedirs(REF_CALLERS_DIR, exist_ok=True)
        for name in REF_CALLERS:
            src = os.path.join(src_dir, name)
            if os.path.exists(src):
                shutil.copyfile(src, os.path.join(REF_CALLERS_DIR, name))
    return REF_CALLERS_DIR if os.path.isdir(REF_CALLERS_DIR) else None


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
    print(stage_reference_callers())
