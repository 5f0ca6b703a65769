"""numpy front end of the C restatement in ``bsi_oracle.c``.

Test infrastructure only: the shipped package never imports this module. It is the
checker used by the tests, the smoke check and the benchmark's CPU baseline.

Arrays are numpy; shapes follow the reference: ``words[Q, S, W]`` uint64,
``chunk_scales[Q, chunks]`` float32, ``Bw[R, Sb]`` float32, ``out[Q, R]`` float32.
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

import importlib.util

_HERE = os.path.dirname(os.path.abspath(__file__))
# oracle/build.py, loaded by path: the checker's folder stays off sys.path (a top-level `build` or
# `oracle` module there would shadow other packages in child processes)
_spec = importlib.util.spec_from_file_location("bsi_oracle_build", os.path.join(_HERE, "build.py"))
_build = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_build)

_lib = None


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(_build.build_oracle())
        i64, i32, f32, f64, u64, i8 = C.c_longlong, C.c_int32, C.c_float, C.c_double, C.c_ulonglong, C.c_int8
        P = C.POINTER
        L.bsi_or_round_half_away.restype = i64
        L.bsi_or_round_half_away.argtypes = [f64]
        L.bsi_or_compute_shift.restype = C.c_int
        L.bsi_or_compute_shift.argtypes = [u64, f64, C.c_int, C.c_int, f32]
        L.bsi_or_quantize_pack.restype = None
        L.bsi_or_quantize_pack.argtypes = [P(f32), i64, i64, C.c_int, C.c_int, C.c_int, f32,
                                           P(i32), P(f32), P(i8), P(u64)]
        L.bsi_or_slice_popcount.argtypes = [P(u64), i64, i64, P(u64)]
        L.bsi_or_compress_flags.argtypes = [P(u64), i64, i64, f64, P(i32)]
        L.bsi_or_ewah_size.argtypes = [P(u64), i64, i64, P(i32), P(u64)]
        L.bsi_or_ewah_emit.argtypes = [P(u64), i64, i64, P(i32), P(u64), P(u64), P(i32)]
        L.bsi_or_ewah_decode.argtypes = [P(u64), i64, i64, P(u64)]
        L.bsi_or_dot_popc.argtypes = [P(u64), P(f32), i64, C.c_int, i64, P(u64), P(f32), C.c_int,
                                      i64, i64, f32, P(f32), P(i32)]
        L.bsi_or_dot_i8.argtypes = [P(i8), P(f32), i64, P(i8), P(f32), i64, i64, i64, f32,
                                    P(f32), P(i32)]
        L.bsi_or_cpu_build.restype = C.c_void_p
        L.bsi_or_cpu_build.argtypes = [P(f32), i64, i64, C.c_int]
        L.bsi_or_cpu_free.argtypes = [C.c_void_p]
        L.bsi_or_cpu_dot.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, P(f64)]
        L.bsi_or_num_threads.restype = C.c_int
        _lib = L
    return _lib


def round_half_away(x: float) -> int:
    return int(lib().bsi_or_round_half_away(float(x)))


def compute_shift(max_abs: int, fixed_bits: int, sum_abs: float = 0.0, count: int = 0,
                  clip_k: float = 0.0) -> int:
    return int(lib().bsi_or_compute_shift(int(max_abs), float(sum_abs), int(count),
                                          int(fixed_bits), float(clip_k)))


def quantize_pack(x, decimal_places: int, bits: int, chunk_mode: bool, clip_k: float = 0.0):
    """x: [Q, D] float32 (half/bfloat16 inputs are widened by the caller, which is exact).

    Returns dict(shifts, scales, qvals[Q,D] int8, words[Q,bits,W] uint64)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    Q, D = x.shape
    W = max(1, (D + 63) // 64)
    chunks = (D + 255) // 256
    sshape = (Q, chunks) if chunk_mode else (Q,)
    shifts = np.zeros(sshape, np.int32)
    scales = np.ones(sshape, np.float32)
    qvals = np.zeros((Q, D), np.int8)
    words = np.zeros((Q, bits, W), np.uint64)
    lib().bsi_or_quantize_pack(_p(x, C.c_float), Q, D, int(decimal_places), int(bits),
                               1 if chunk_mode else 0, float(clip_k),
                               _p(shifts, C.c_int32), _p(scales, C.c_float),
                               _p(qvals, C.c_int8), _p(words, C.c_ulonglong))
    return dict(shifts=shifts, scales=scales, qvals=qvals, words=words)


def slice_weights(bits: int, row_scale=None):
    """Base two's-complement slice weights (+-2^i, top negative), optionally times a per-row scale.

    Reference: bsi_vector_cuda.cpp:1028-1043 (queries) and :1148-1157 (keys)."""
    w = np.array([(-1.0 if i == bits - 1 else 1.0) * float(1 << i) for i in range(bits)], np.float32)
    if row_scale is None:
        return w
    return (w[None, :] * np.asarray(row_scale, np.float32)[:, None]).astype(np.float32)


def pad_i8(qvals, chunks: int):
    Q, D = qvals.shape
    out = np.zeros((Q, chunks * 256), np.int8)
    out[:, :D] = qvals
    return out


def slice_popcount(words):
    words = np.ascontiguousarray(words, np.uint64)
    S, W = words.shape
    counts = np.zeros(S, np.uint64)
    lib().bsi_or_slice_popcount(_p(words, C.c_ulonglong), S, W, _p(counts, C.c_ulonglong))
    return counts


def compress_flags(counts, W: int, threshold: float):
    counts = np.ascontiguousarray(counts, np.uint64)
    flags = np.zeros(counts.shape[0], np.int32)
    lib().bsi_or_compress_flags(_p(counts, C.c_ulonglong), counts.shape[0], int(W),
                                float(threshold), _p(flags, C.c_int32))
    return flags


def ewah_encode(words, flags):
    """words [S, W], flags [S] -> (stream uint64[total], off int64[S], length int32[S])."""
    words = np.ascontiguousarray(words, np.uint64)
    flags = np.ascontiguousarray(flags, np.int32)
    S, W = words.shape
    sizes = np.zeros(S, np.uint64)
    lib().bsi_or_ewah_size(_p(words, C.c_ulonglong), S, W, _p(flags, C.c_int32), _p(sizes, C.c_ulonglong))
    off = np.zeros(S, np.uint64)
    if S > 1:
        off[1:] = np.cumsum(sizes)[:-1]
    total = int(sizes.sum())
    stream = np.zeros(max(total, 1), np.uint64)
    length = np.zeros(S, np.int32)
    lib().bsi_or_ewah_emit(_p(words, C.c_ulonglong), S, W, _p(flags, C.c_int32),
                           _p(off, C.c_ulonglong), _p(stream, C.c_ulonglong), _p(length, C.c_int32))
    return stream[:total], off.astype(np.int64), length


def ewah_decode(stream, W: int):
    stream = np.ascontiguousarray(stream, np.uint64)
    out = np.zeros(W, np.uint64)
    lib().bsi_or_ewah_decode(_p(stream, C.c_ulonglong), stream.shape[0], int(W), _p(out, C.c_ulonglong))
    return out


def dot_popc(A, qs, B, Bw, scale_inv: float, want_iacc: bool = False):
    """Weighted-popcount form. qs is [Q, chunks] (chunk scales) or [Q] (row scales)."""
    A = np.ascontiguousarray(A, np.uint64)
    B = np.ascontiguousarray(B, np.uint64)
    qs = np.ascontiguousarray(qs, np.float32)
    Bw = np.ascontiguousarray(Bw, np.float32)
    Q, Sa, W = A.shape
    R, Sb, W2 = B.shape
    assert W == W2 and W % 4 == 0
    chunks = W // 4
    stride = chunks if qs.ndim == 2 else 0
    out = np.zeros((Q, R), np.float32)
    iacc = np.zeros((Q, R, chunks), np.int32) if want_iacc else None
    lib().bsi_or_dot_popc(_p(A, C.c_ulonglong), _p(qs, C.c_float), stride, Sa, W,
                          _p(B, C.c_ulonglong), _p(Bw, C.c_float), Sb, R, Q,
                          float(np.float32(scale_inv)), _p(out, C.c_float), _p(iacc, C.c_int32))
    return (out, iacc) if want_iacc else out


def dot_i8(a8, qs, k8, bw0, scale_inv: float, want_iacc: bool = False):
    """Integer-product form on the clamped values; a8 [Q, 256*chunks], k8 [R, 256*chunks]."""
    a8 = np.ascontiguousarray(a8, np.int8)
    k8 = np.ascontiguousarray(k8, np.int8)
    qs = np.ascontiguousarray(qs, np.float32)
    bw0 = np.ascontiguousarray(bw0, np.float32)
    Q, Dp = a8.shape
    R = k8.shape[0]
    chunks = Dp // 256
    stride = chunks if qs.ndim == 2 else 0
    out = np.zeros((Q, R), np.float32)
    iacc = np.zeros((Q, R, chunks), np.int32) if want_iacc else None
    lib().bsi_or_dot_i8(_p(a8, C.c_int8), _p(qs, C.c_float), stride, _p(k8, C.c_int8),
                        _p(bw0, C.c_float), Q, R, chunks, float(np.float32(scale_inv)),
                        _p(out, C.c_float), _p(iacc, C.c_int32))
    return (out, iacc) if want_iacc else out


def scale_inv(decimal_places: int) -> np.float32:
    """float(1 / 10^(dq + dk)), as bsi_cuda.cpp:710-711,753 computes it."""
    t = 2 * int(decimal_places)
    return np.float32(1.0 / (10.0 ** t)) if t > 0 else np.float32(1.0)


def fixed_dot(xq, xk, decimal_places: int = 2, bits_q: int = 7, bits_k: int = 6,
              want_iacc: bool = False, via: str = "i8", clip_k: float = 0.0, chunk_scale: bool = True):
    """End to end: queries xq [Q, D], keys xk [R, D] (float32) -> out [Q, R] float32.

    Queries get per-256-element chunk scales when ceil(D/64) is a multiple of 4, else a
    per-row scale (bsi_vector_cuda.cpp:980-994); keys always get a per-row scale."""
    xq = np.ascontiguousarray(xq, np.float32)
    xk = np.ascontiguousarray(xk, np.float32)
    D = xq.shape[1]
    W = max(1, (D + 63) // 64)
    chunk = chunk_scale and (W % 4 == 0)          # BSI_FIXED_CHUNK_SCALE=0 gives one scale per query row
    qa = quantize_pack(xq, decimal_places, bits_q, chunk, clip_k)
    kb = quantize_pack(xk, decimal_places, bits_k, False, clip_k)
    Bw = slice_weights(bits_k, kb["scales"])
    si = scale_inv(decimal_places)
    if via == "popc":
        assert chunk
        return dot_popc(qa["words"], qa["scales"], kb["words"], Bw, si, want_iacc)
    chunks = (D + 255) // 256
    return dot_i8(pad_i8(qa["qvals"], chunks), qa["scales"], pad_i8(kb["qvals"], chunks),
                  Bw[:, 0].copy(), si, want_iacc)


def cpu_dot(xq, xk, decimal_places: int = 2, threads: int = 0):
    """The reference's CPU (bsiCPP-semantics) path: float64 [Q, R]."""
    xq = np.ascontiguousarray(xq, np.float32)
    xk = np.ascontiguousarray(xk, np.float32)
    L = lib()
    hq = L.bsi_or_cpu_build(_p(xq, C.c_float), xq.shape[0], xq.shape[1], int(decimal_places))
    hk = L.bsi_or_cpu_build(_p(xk, C.c_float), xk.shape[0], xk.shape[1], int(decimal_places))
    out = np.zeros((xq.shape[0], xk.shape[0]), np.float64)
    try:
        L.bsi_or_cpu_dot(hq, hk, int(decimal_places), int(threads), _p(out, C.c_double))
    finally:
        L.bsi_or_cpu_free(hq)
        L.bsi_or_cpu_free(hk)
    return out


class CpuKeyset:
    """Prebuilt CPU key set, so that a timed loop measures the dot and the query build only
    (as the reference's batch_dot_product_prebuilt does, bsiFunctions.cpp:651-701)."""

    def __init__(self, xk, decimal_places: int):
        xk = np.ascontiguousarray(xk, np.float32)
        self.dp = int(decimal_places)
        self.R = xk.shape[0]
        self.h = lib().bsi_or_cpu_build(_p(xk, C.c_float), xk.shape[0], xk.shape[1], self.dp)

    def dot(self, xq, threads: int = 0):
        xq = np.ascontiguousarray(xq, np.float32)
        L = lib()
        hq = L.bsi_or_cpu_build(_p(xq, C.c_float), xq.shape[0], xq.shape[1], self.dp)
        out = np.zeros((xq.shape[0], self.R), np.float64)
        try:
            L.bsi_or_cpu_dot(hq, self.h, self.dp, int(threads), _p(out, C.c_double))
        finally:
            L.bsi_or_cpu_free(hq)
        return out

    def __del__(self):
        try:
            lib().bsi_or_cpu_free(self.h)
        except Exception:
            pass


def num_threads() -> int:
    return int(lib().bsi_or_num_threads())


# ---- variable-slice mode (the reference without BSI_FIXED_BITS*: no shift, slice count from the data) ------------
def decimal_ints(x, decimal_places: int):
    """half_away(double(float(x)) * 10^dp) as int64 (bsi_cuda_kernels_quant.cuh:24-29, 110-121)."""
    t = np.ascontiguousarray(x, np.float32).astype(np.float64) * (10.0 ** int(decimal_places))
    return np.where(t >= 0, np.floor(t + 0.5), -np.floor(-t + 0.5)).astype(np.int64)


def variable_slices(max_abs: int) -> int:
    """bit_width(max |v|) + 2, 2 when everything is zero, at most 64 (bsi_vector_cuda.cpp:746-754)."""
    max_abs = int(max_abs)
    return min(64, max(1, max_abs.bit_length()) + 2) if max_abs else 2


def variable_pack(x, decimal_places: int, per_row: bool = False):
    """Variable-slice builder. Queries (per_row=False): one slice count for the batch
    (bsi_vector_cuda.cpp:1086-1101); keys (per_row=True): `row_slices` holds every row's own count, the words
    are stored at the widest row's width. Words are the low S bits of the two's-complement integers
    (bsi_cuda_kernels_pack.cuh:129-174); a row's slice weights are +2^i, with the top slice negative when the row
    holds a negative value (bsi_vector_cuda.cpp:1156-1162).

    Returns dict(ints[rows, D] int64, S, row_slices[rows], words[rows, S, W] uint64, weights[rows, S] float32)."""
    v = decimal_ints(x, decimal_places)
    rows, D = v.shape
    W = max(1, (D + 63) // 64)
    row_max = np.abs(v).max(axis=1) if D else np.zeros(rows, np.int64)
    S = variable_slices(int(row_max.max()) if rows else 0)
    row_slices = np.array([variable_slices(int(m)) for m in row_max], np.int32) if per_row else np.full(rows, S, np.int32)
    words = np.zeros((rows, S, W), np.uint64)
    u = v.astype(np.uint64)                       # two's complement bit pattern
    for s in range(S):
        bit = ((u >> np.uint64(s)) & np.uint64(1)).astype(np.uint64)
        for w in range(W):
            seg = bit[:, w * 64:(w + 1) * 64]
            sh = np.arange(seg.shape[1], dtype=np.uint64)
            words[:, s, w] = (seg << sh[None, :]).sum(axis=1, dtype=np.uint64)
    base = np.array([float(1 << i) for i in range(S)], np.float32)
    twos = base.copy()
    twos[S - 1] = -twos[S - 1]
    neg = (v < 0).any(axis=1)
    weights = np.where(neg[:, None], twos[None, :], base[None, :]).astype(np.float32)
    return dict(ints=v, S=S, row_slices=row_slices, words=words, weights=weights, negative=neg)


def variable_dot(xq, xk, decimal_places: int = 2):
    """out[q][r] = float32(sum_d vq[q][d] * vk[r][d]) * float32(1 / 10^(2 dp)): what the reference's weighted
    popcount sum (bsi_cuda_kernels_dot.cuh:597-654) gives while its float32 partial sums stay below 2^24 (every
    product of a count, a power of two and an integer is then exact); asserts that bound."""
    vq, vk = decimal_ints(xq, decimal_places), decimal_ints(xk, decimal_places)
    bound = np.abs(vq).astype(np.int64) @ np.abs(vk).astype(np.int64).T
    assert int(bound.max(initial=0)) < (1 << 24), "outside the range where the reference's float32 accumulation is exact"
    exact = vq @ vk.T
    return exact.astype(np.float32) * scale_inv(decimal_places)


def variable_dot_popc(qa, kb, decimal_places: int = 2):
    """Slow cross-check of variable_dot from the slices and weights themselves (small shapes only)."""
    A, Aw, B, Bw = qa["words"], qa["weights"], kb["words"], kb["weights"]
    Q, Sa, W = A.shape
    R, Sb, _ = B.shape
    out = np.zeros((Q, R), np.float64)
    for i in range(Sa):
        for j in range(Sb):
            both = A[:, None, i, :] & B[None, :, j, :]
            cnt = np.zeros((Q, R), np.int64)
            for w in range(W):
                cnt += np.array([[bin(int(x)).count("1") for x in row] for row in both[:, :, w]], np.int64)
            out += cnt * (Aw[:, i].astype(np.float64)[:, None] * Bw[:, j].astype(np.float64)[None, :])
    return out.astype(np.float32) * scale_inv(decimal_places)
