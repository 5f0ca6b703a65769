"""Thin helpers that call the C ABI (through ctypes) on torch CUDA tensors."""
import ctypes as C

import torch

from bsipytorch_b200 import capi

_DT = {torch.float32: capi.DTYPE_F32, torch.float16: capi.DTYPE_F16, torch.bfloat16: capi.DTYPE_BF16}


def quantize_pack(x, decimal_places=2, bits=7, chunk_mode=True, want_q8=True, clip_k=0.0):
    assert x.is_cuda and x.dim() == 2
    x = x.contiguous()
    rows, D = x.shape
    W = max(1, (D + 63) // 64)
    chunks = (D + 255) // 256
    dev = x.device
    words = torch.zeros(rows, bits, W, dtype=torch.int64, device=dev)
    sshape = (rows, chunks) if chunk_mode else (rows,)
    scales = torch.ones(sshape, dtype=torch.float32, device=dev)
    shifts = torch.zeros(sshape, dtype=torch.int32, device=dev)
    ld8 = max(chunks, 1) * 256
    q8 = torch.full((rows, ld8), 99, dtype=torch.int8, device=dev) if want_q8 else None
    if clip_k > 0.0:
        rc = capi.lib().bsi_b200_quantize_pack_clip(capi.ptr(x), _DT[x.dtype], rows, D, D, decimal_places, bits,
                                                    1 if chunk_mode else 0, C.c_float(clip_k), capi.ptr(words),
                                                    capi.ptr(scales), capi.ptr(shifts), capi.ptr(q8), ld8,
                                                    capi.stream_ptr())
    else:
        rc = capi.lib().bsi_b200_quantize_pack(capi.ptr(x), _DT[x.dtype], rows, D, D, decimal_places, bits,
                                               1 if chunk_mode else 0, capi.ptr(words), capi.ptr(scales),
                                               capi.ptr(shifts), capi.ptr(q8), ld8, capi.stream_ptr())
    capi.check(rc, "bsi_b200_quantize_pack")
    return dict(words=words, scales=scales, shifts=shifts, q8=q8)


def recombine_i8(words):
    rows, bits, W = words.shape
    chunks = (W + 3) // 4
    q8 = torch.full((rows, chunks * 256), 99, dtype=torch.int8, device=words.device)
    rc = capi.lib().bsi_b200_recombine_i8(capi.ptr(words), rows, bits, W, capi.ptr(q8), chunks * 256,
                                          capi.stream_ptr())
    capi.check(rc, "bsi_b200_recombine_i8")
    return q8


def dot_i8(a8, qs, k8, bw0, scale_inv, engine=capi.ENGINE_AUTO, want_iacc=False):
    Q, lda = a8.shape
    R, ldk = k8.shape
    chunks = lda // 256
    stride = chunks if qs.dim() == 2 else 0
    out = torch.full((Q, R), float("nan"), dtype=torch.float32, device=a8.device)
    iacc = torch.full((Q, R, chunks), -2 ** 31, dtype=torch.int32, device=a8.device) if want_iacc else None
    rc = capi.lib().bsi_b200_dot_i8(capi.ptr(a8), lda, capi.ptr(qs), stride, capi.ptr(k8), ldk, capi.ptr(bw0),
                                    Q, R, chunks, C.c_float(float(scale_inv)), capi.ptr(out), R, capi.ptr(iacc),
                                    engine, capi.stream_ptr())
    capi.check(rc, "bsi_b200_dot_i8")
    return (out, iacc) if want_iacc else out


def dot_words(A, qs, B, Bw, scale_inv, want_iacc=False):
    Q, Sa, W = A.shape
    R, Sb, _ = B.shape
    chunks = W // 4
    stride = chunks if qs.dim() == 2 else 0
    out = torch.full((Q, R), float("nan"), dtype=torch.float32, device=A.device)
    iacc = torch.full((Q, R, chunks), -2 ** 31, dtype=torch.int32, device=A.device) if want_iacc else None
    rc = capi.lib().bsi_b200_dot_words(capi.ptr(A), capi.ptr(qs), stride, Sa, W, capi.ptr(B), capi.ptr(Bw), Sb,
                                       R, Q, C.c_float(float(scale_inv)), R, capi.ptr(out), capi.ptr(iacc),
                                       capi.stream_ptr())
    capi.check(rc, "bsi_b200_dot_words")
    return (out, iacc) if want_iacc else out


def ewah_encode(words2d, threshold):
    """One-call encoder. Returns (stream, off, length, flags) as torch tensors."""
    S, W = words2d.shape
    dev = words2d.device
    L = capi.lib()
    scratch = torch.empty(max(int(L.bsi_b200_ewah_scratch_bytes(S)), 8), dtype=torch.uint8, device=dev)
    cap = S * (W + 1)
    out = torch.zeros(max(cap, 1), dtype=torch.int64, device=dev)
    off = torch.zeros(S, dtype=torch.int64, device=dev)
    length = torch.zeros(S, dtype=torch.int32, device=dev)
    flags = torch.zeros(S, dtype=torch.int32, device=dev)
    total = torch.zeros(1, dtype=torch.int64, device=dev)
    rc = L.bsi_b200_ewah_encode(capi.ptr(words2d), S, W, C.c_double(threshold), capi.ptr(scratch), scratch.numel(),
                                capi.ptr(out), cap, capi.ptr(off), capi.ptr(length), capi.ptr(flags),
                                capi.ptr(total), capi.stream_ptr())
    capi.check(rc, "bsi_b200_ewah_encode")
    return out[: int(total.item())], off, length, flags


def ewah_steps(words2d, threshold):
    """The four separate entry points, as the reference chains them."""
    S, W = words2d.shape
    dev = words2d.device
    L = capi.lib()
    counts = torch.zeros(S, dtype=torch.int64, device=dev)
    flags = torch.zeros(S, dtype=torch.int32, device=dev)
    sizes = torch.zeros(S, dtype=torch.int64, device=dev)
    off = torch.zeros(S, dtype=torch.int64, device=dev)
    total = torch.zeros(1, dtype=torch.int64, device=dev)
    capi.check(L.bsi_b200_ewah_flags(capi.ptr(words2d), S, W, C.c_double(threshold), capi.ptr(counts),
                                     capi.ptr(flags), capi.stream_ptr()))
    capi.check(L.bsi_b200_ewah_size(capi.ptr(words2d), S, W, capi.ptr(flags), capi.ptr(sizes), capi.stream_ptr()))
    capi.check(L.bsi_b200_ewah_offsets(capi.ptr(sizes), S, capi.ptr(off), capi.ptr(total), capi.stream_ptr()))
    out = torch.zeros(max(int(total.item()), 1), dtype=torch.int64, device=dev)
    length = torch.zeros(S, dtype=torch.int32, device=dev)
    capi.check(L.bsi_b200_ewah_emit(capi.ptr(words2d), S, W, capi.ptr(flags), capi.ptr(off), capi.ptr(out),
                                    capi.ptr(length), capi.stream_ptr()))
    return out[: int(total.item())], off, length, flags, counts, sizes


def ewah_decode(stream, off, length, W):
    S = off.shape[0]
    out = torch.full((S, W), -1, dtype=torch.int64, device=off.device)
    if stream.numel() == 0:
        stream = torch.zeros(1, dtype=torch.int64, device=off.device)
    capi.check(capi.lib().bsi_b200_ewah_decode(capi.ptr(stream), capi.ptr(off), capi.ptr(length), S, W,
                                               capi.ptr(out), capi.stream_ptr()))
    return out


def as_u64(t):
    """int64 torch tensor -> numpy uint64 (same bits)."""
    return t.detach().cpu().numpy().view("uint64")
