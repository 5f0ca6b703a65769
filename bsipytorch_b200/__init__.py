"""B200-native (sm_100a) implementation of the bit-sliced-index (BSI) tensor-dot path.

* ``bsipytorch_b200.bsi_ops``  -- pybind11 module with the reference's ``bsi_ops`` CUDA entry points
* ``bsipytorch_b200.capi``     -- ctypes view of the C ABI (``include/bsi_b200.h``)
* ``bsipytorch_b200.linear``   -- ``BSIQuantizedLinear`` / ``quantize_model_bsi`` (the reference's layer
  replacement, ``bsi_ops/benchmarks/verify_accuracy_bsi.py``)

There is no CPU or eager fallback: importing ``bsi_ops`` fails loudly when the native libraries have
not been built (``python -m bsipytorch_b200.build``).
"""
from __future__ import annotations

import importlib
import os
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))


def _load_bsi_ops():
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    try:
        return importlib.import_module("bsipytorch_b200.bsi_ops")
    except ImportError as e:  # pragma: no cover - exercised only on a broken install
        raise ImportError(
            "bsipytorch_b200: the native extension is missing or does not load (" + str(e) + "). "
            "Build it in-tree with `python -m bsipytorch_b200.build`; there is no fallback path.") from e


def __getattr__(name):
    if name == "bsi_ops":
        mod = _load_bsi_ops()
        globals()["bsi_ops"] = mod
        return mod
    raise AttributeError(name)


def install_as_bsi_ops():
    """Make ``import bsi_ops`` resolve to this implementation, for unmodified reference scripts."""
    mod = _load_bsi_ops()
    sys.modules["bsi_ops"] = mod
    return mod
