"""Loader of the fixtures the reference's own kernels produced (tests/golden/ref_fixed76.npz)."""
import os

import numpy as np
import torch

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_fixed76.npz")
MODES_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_modes.npz")
DOT_CASES = ("c1", "fc1", "fc2")


def load():
    return np.load(PATH)


def load_modes():
    """Variable-slice mode, row-scale dots and outlier clipping through the reference's kernels."""
    return np.load(MODES_PATH)


def f16(g, key):
    return torch.from_numpy(g[key].copy()).view(torch.float16)


def case_inputs(g, name):
    """(queries as a torch tensor in their original dtype, keys float32)."""
    dt = str(g[f"{name}_q_dtype"])
    raw = g[f"{name}_q"]
    if dt == "torch.float32":
        q = torch.from_numpy(raw.copy())
    else:
        q = torch.from_numpy(raw.copy()).view(torch.float16 if dt == "torch.float16" else torch.bfloat16)
    k = torch.from_numpy(g[f"{name}_k_f16bits"].copy()).view(torch.float16).float()
    return q, k
