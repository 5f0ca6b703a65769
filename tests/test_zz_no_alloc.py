"""The allocation-free EWAH encoder (bsi_b200_ewah_encode_static) against the regular one.

Some hosts of this library cannot allocate device memory on its behalf and cannot let it allocate
either -- a plugin inside a process whose memory manager already owns the GPU, a binding that only
holds its input and output buffers, a loop that must stay free of cudaMalloc/cudaFree because they
serialise the device. For them the encoder's scratch (per-slice popcounts and sizes) sits in a fixed
array inside the library. This file checks, through the C ABI, that it produces exactly what the
caller-scratch entry point produces, twice in a row on different inputs (the array is shared between
calls and keeps the previous call's contents), and that it refuses more slices than the array holds.

Collected last on purpose, so that a run that stops at the first failure has already run every other
test. It passes on its own in a fresh process as well as after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import _capi_helpers as H
from bsipytorch_b200 import capi

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _words(S, W, seed):
    rng = np.random.default_rng(seed)
    w = rng.integers(1, 2 ** 63, (S, W), dtype=np.uint64)
    w[rng.random((S, W)) < 0.5] = 0
    w[::3] = 0                                   # whole slices empty -> compressible
    w[1::7, : W // 2] = np.uint64(0xFFFFFFFFFFFFFFFF)
    return torch.from_numpy(w.view(np.int64)).to(DEV)


def _encode_static(words, threshold):
    S, W = words.shape
    cap = S * (W + 1)
    out = torch.zeros(max(cap, 1), dtype=torch.int64, device=DEV)
    off = torch.zeros(S, dtype=torch.int64, device=DEV)
    length = torch.zeros(S, dtype=torch.int32, device=DEV)
    flags = torch.zeros(S, dtype=torch.int32, device=DEV)
    total = torch.zeros(1, dtype=torch.int64, device=DEV)
    rc = capi.lib().bsi_b200_ewah_encode_static(capi.ptr(words), S, W, C.c_double(threshold), capi.ptr(out), cap,
                                                capi.ptr(off), capi.ptr(length), capi.ptr(flags), capi.ptr(total),
                                                capi.stream_ptr())
    capi.check(rc, "bsi_b200_ewah_encode_static")
    return out[: int(total.item())], off, length, flags


def test_static_scratch_encoder_matches_regular_encoder_twice():
    # second call: fewer slices and a different width, so stale counts/sizes of the first call sit
    # right behind the part of the array the second call uses
    for S, W, thr, seed in [(700, 32, 0.5, 1), (90, 129, 0.2, 2)]:
        words = _words(S, W, seed)
        want = H.ewah_encode(words, thr)
        got = _encode_static(words, thr)
        for a, b in zip(got, want):
            assert torch.equal(a, b)          # integer streams: exact equality is the tolerance
        assert torch.equal(H.ewah_decode(got[0], got[1], got[2], W), words)


def test_static_scratch_encoder_at_its_slice_limit():
    # exactly as many slices as the array holds: the counts fill their half, the sizes end at the array's last word
    S, W = capi.EWAH_STATIC_MAX_SLICES, 4
    words = _words(S, W, 3)
    want = H.ewah_encode(words, 0.5)
    got = _encode_static(words, 0.5)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert torch.equal(H.ewah_decode(got[0], got[1], got[2], W), words)


def test_static_scratch_encoder_rejects_oversized_requests():
    L = capi.lib()
    w = torch.zeros(4, 4, dtype=torch.int64, device=DEV)
    rc = L.bsi_b200_ewah_encode_static(capi.ptr(w), capi.EWAH_STATIC_MAX_SLICES + 1, 4, C.c_double(0.5), capi.ptr(w),
                                       16, capi.ptr(w), capi.ptr(w), capi.ptr(w), capi.ptr(w), None)
    assert rc == capi.ERR_UNSUPPORTED
    assert b"exceeds the built-in scratch" in L.bsi_b200_last_error()
