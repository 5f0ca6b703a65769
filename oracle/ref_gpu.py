"""ctypes harness over the reference's own CUDA kernels (``oracle/_ref/ref_kernels.so``).

Test infrastructure only. The library is the reference's ``bsi_cuda_kernels.cu`` compiled
unmodified for sm_100a by ``oracle/build.py``; this module re-does the few lines of host
orchestration that sit above its ``extern "C" launch_*`` functions
(bsi_vector_cuda.cpp:401-557 for queries, :581-656 + :1108-1157 for keys, :900-952 for EWAH,
bsi_cuda.cpp:658-815 for the dot) so that its outputs can be compared with ours on a GPU.

The dot launcher reads its mode from the environment on first use (dot.cuh:2664-2724), so the
fixed76 recipe of the reference's README is exported before the library is loaded. The TMA
variant (BSI_TC_TMA=1) is left off: its mbarrier wait has no bound (dot.cuh:2026-2046).
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_SO = os.path.join(_HERE, "_ref", "ref_kernels.so")

_FIXED76_ENV = {
    "BSI_TC_DOT": "1", "BSI_TC_FIXED_INT": "1", "BSI_TC_CPASYNC": "1", "BSI_FIXED_BITS_KEYS": "6",
    "BSI_FIXED_BITS_QUERIES": "7", "BSI_FIXED_CHUNK_SCALE": "1", "BSI_TC_R_SWEEP": "4", "BSI_TC_TMA": "0",
}

_lib = None


def available() -> bool:
    return os.path.exists(REF_SO) and torch.cuda.is_available()


def lib():
    global _lib
    if _lib is None:
        for k, v in _FIXED76_ENV.items():
            os.environ.setdefault(k, v)
        _lib = C.CDLL(REF_SO)
    return _lib


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dtype_code(x):
    return {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[x.dtype]


def pack_queries_chunk(x, decimal_places=2, bits=7, clip_k=0.0):
    """Reference query builder, chunk-scale mode. Returns (words[Q,bits,W] int64, shifts, scales)."""
    L = lib()
    x = x.contiguous()
    Q, d = x.shape
    W = (d + 63) // 64
    chunks = (d + 255) // 256
    dev = x.device
    words = torch.zeros(Q, bits, W, dtype=torch.int64, device=dev)
    shifts = torch.empty(Q, chunks, dtype=torch.int32, device=dev)
    scales = torch.empty(Q, chunks, dtype=torch.float32, device=dev)
    dec = C.c_double(10.0 ** decimal_places)
    L.launch_compute_chunk_shift_scale_from_input(
        _p(x), C.c_int(_dtype_code(x)), C.c_int64(Q), C.c_int64(d), C.c_int(chunks), dec, C.c_int(bits),
        C.c_float(clip_k), _p(shifts), _p(scales), _stream())
    L.launch_quantize_shift_pack_chunk_batch(
        _p(x), C.c_int(_dtype_code(x)), C.c_int64(Q), C.c_int64(d), C.c_int(chunks), C.c_int(bits), C.c_int(W),
        C.c_ulonglong((1 << bits) - 1), dec, C.c_int(bits), _p(shifts), _p(words), _stream())
    return words, shifts, scales


def pack_rows(x, decimal_places=2, bits=6, clip_k=0.0):
    """Reference fixed-bit per-row builder (the key path). Returns (words, shifts, scales, ints)."""
    L = lib()
    x = x.contiguous()
    R, d = x.shape
    W = (d + 63) // 64
    dev = x.device
    ints = torch.empty(R, d, dtype=torch.int64, device=dev)
    shifts = torch.empty(R, dtype=torch.int32, device=dev)
    scales = torch.empty(R, dtype=torch.float32, device=dev)
    words = torch.zeros(R, bits, W, dtype=torch.int64, device=dev)
    L.launch_quantize_round_to_int64_batch(_p(x), C.c_int(_dtype_code(x)), C.c_int64(R), C.c_int64(d),
                                           C.c_double(10.0 ** decimal_places), _p(ints), _stream())
    L.launch_compute_row_shift_scale(_p(ints), C.c_int64(R), C.c_int64(d), C.c_int(bits), C.c_float(clip_k),
                                     _p(shifts), _p(scales), _stream())
    L.launch_apply_row_shift_clamp(_p(ints), C.c_int64(R), C.c_int64(d), _p(shifts), C.c_int(bits), _stream())
    L.launch_pack_bits_all_ballot_batch(_p(ints), C.c_int(R), C.c_longlong(d), C.c_int(bits), C.c_int(W),
                                        C.c_ulonglong((1 << bits) - 1), _p(words), _stream())
    return words, shifts, scales, ints


def slice_weights(bits, rows, device, row_scales=None):
    w = torch.tensor([(-1.0 if i == bits - 1 else 1.0) * float(1 << i) for i in range(bits)],
                     dtype=torch.float32, device=device)
    w = w.unsqueeze(0).expand(rows, bits)
    if row_scales is not None:
        w = w * row_scales.unsqueeze(1)
    return w.contiguous()


def dot_fixed76(A_words, A_chunk_scales, B_words, Bw, scale_inv):
    """Reference fixed76 chunk-scale dot (packed-entry argument pattern). Returns out [Q, R] float32."""
    L = lib()
    Q, Sa, W = A_words.shape
    R, Sb, _ = B_words.shape
    dev = A_words.device
    Aw = slice_weights(Sa, Q, dev)
    out = torch.zeros(Q, R, dtype=torch.float32, device=dev)
    L.launch_popcount_weighted_keys_literal_fused_multiq(
        _p(A_words), _p(Aw), _p(A_chunk_scales), C.c_int(A_chunk_scales.shape[1]), C.c_int(Sa), C.c_int(W),
        _p(B_words), _p(Bw), C.c_int(Sb), C.c_int(R), C.c_int(Q), C.c_int(8), C.c_int(4), None, None,
        C.c_float(float(scale_inv)), C.c_int(R), _p(out), _stream())
    return out


def ewah_encode(words2d, threshold):
    """Reference EWAH encode of words [S, W]. Returns (stream, off, length, flags, counts)."""
    L = lib()
    words2d = words2d.contiguous()
    S, W = words2d.shape
    dev = words2d.device
    counts = torch.empty(S, dtype=torch.int64, device=dev)
    flags = torch.empty(S, dtype=torch.int32, device=dev)
    sizes = torch.empty(S, dtype=torch.int64, device=dev)
    L.launch_slice_popcount_sum(_p(words2d), C.c_int(S), C.c_int(W), _p(counts), _stream())
    L.launch_compress_flags_from_density(_p(counts), C.c_int(S), C.c_int(W), C.c_double(threshold), _p(flags), _stream())
    L.launch_ewah_size(_p(words2d), C.c_int(S), C.c_int(W), _p(flags), _p(sizes), _stream())
    incl = sizes.cumsum(0)
    total = int(incl[-1].item())
    off = torch.zeros(S, dtype=torch.int64, device=dev)
    off[1:] = incl[:-1]
    stream = torch.empty(total, dtype=torch.int64, device=dev)
    length = torch.empty(S, dtype=torch.int32, device=dev)
    L.launch_ewah_emit(_p(words2d), C.c_int(S), C.c_int(W), _p(flags), _p(off), _p(stream), _p(length), _stream())
    return stream, off, length, flags, counts


def ewah_decode(stream, off, length, W):
    L = lib()
    S = off.shape[0]
    out = torch.empty(S, W, dtype=torch.int64, device=stream.device)
    off_h = off.cpu().tolist()
    len_h = length.cpu().tolist()
    for s in range(S):
        L.launch_ewah_decompress(C.c_void_p(stream.data_ptr() + 8 * off_h[s]), C.c_int(len_h[s]), C.c_int(W),
                                 C.c_void_p(out.data_ptr() + 8 * s * W), _stream())
    return out


def pack_plain(x, decimal_places, slices):
    """Reference variable-slice builder on the GPU: round to int64, then the ballot packer
    (bsi_vector_cuda.cpp:1074-1131). Returns (words [rows, slices, W] int64, ints [rows, d] int64)."""
    L = lib()
    x = x.contiguous()
    rows, d = x.shape
    W = (d + 63) // 64
    dev = x.device
    ints = torch.empty(rows, d, dtype=torch.int64, device=dev)
    words = torch.zeros(rows, slices, W, dtype=torch.int64, device=dev)
    L.launch_quantize_round_to_int64_batch(_p(x), C.c_int(_dtype_code(x)), C.c_int64(rows), C.c_int64(d),
                                           C.c_double(10.0 ** decimal_places), _p(ints), _stream())
    mask = (1 << slices) - 1 if slices < 64 else (1 << 64) - 1
    L.launch_pack_bits_all_ballot_batch(_p(ints), C.c_int(rows), C.c_longlong(d), C.c_int(slices), C.c_int(W),
                                        C.c_ulonglong(mask), _p(words), _stream())
    return words, ints


def dot_generic(A_words, Aw, B_words, Bw, scale_inv, tensor_core=True):
    """Reference generic-S dot with float slice weights and no chunk scales (the variable-slice path,
    bsi_cuda.cpp:433-656 -> dot.cuh:211-1283 with BSI_TC_DOT=1, :58-188 with 0). Returns out [Q, R] float32."""
    L = lib()
    Q, Sa, W = A_words.shape
    R, Sb, _ = B_words.shape
    out = torch.zeros(Q, R, dtype=torch.float32, device=A_words.device)
    old = os.environ.get("BSI_TC_DOT")
    os.environ["BSI_TC_DOT"] = "1" if tensor_core else "0"      # re-read on every launch (dot.cuh:2642)
    try:
        L.launch_popcount_weighted_keys_literal_fused_multiq(
            _p(A_words), _p(Aw.contiguous()), None, C.c_int(0), C.c_int(Sa), C.c_int(W),
            _p(B_words), _p(Bw.contiguous()), C.c_int(Sb), C.c_int(R), C.c_int(Q), C.c_int(8), C.c_int(4), None, None,
            C.c_float(float(scale_inv)), C.c_int(R), _p(out), _stream())
        torch.cuda.synchronize()
    finally:
        if old is None:
            os.environ.pop("BSI_TC_DOT", None)
        else:
            os.environ["BSI_TC_DOT"] = old
    return out
