"""ctypes binding of the C ABI declared in ``include/bsi_b200.h``.

This is the binding a non-C++ host would write; the tests call the kernels through it with raw
device pointers taken from torch tensors. Loading fails loudly when ``libbsi_b200.so`` is absent.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libbsi_b200.so")

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE, ERR_TIMEOUT = 0, 1, 2, 3, 4, 5
DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
ENGINE_AUTO, ENGINE_TCGEN05, ENGINE_SIMT, ENGINE_BMMA = 0, 1, 2, 3
EWAH_STATIC_MAX_SLICES = 65536

_vp, _i64, _i32, _f32, _f64 = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_double

# name -> (restype, argtypes); every symbol the header declares.
SIGNATURES = {
    "bsi_b200_status_string": (C.c_char_p, [_i32]),
    "bsi_b200_last_error": (C.c_char_p, []),
    "bsi_b200_version": (_i32, []),
    "bsi_b200_device_status": (_i32, [C.POINTER(_i32)]),
    "bsi_b200_quantize_pack": (_i32, [_vp, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i64, _vp]),
    "bsi_b200_quantize_pack_clip": (_i32, [_vp, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _f32, _vp, _vp, _vp, _vp, _i64, _vp]),
    "bsi_b200_decimal_absmax": (_i32, [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _vp, _vp]),
    "bsi_b200_pack_plain": (_i32, [_vp, _i32, _i64, _i64, _i64, _i32, _i32, _vp, _vp, _vp, _i64, _vp]),
    "bsi_b200_quantize_pack_norms": (_i32, [_vp, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _f32, _vp, _vp, _vp, _vp, _i64, _vp, _vp]),
    "bsi_b200_register_query_bounds": (_i32, [_vp, _vp, _i64]),
    "bsi_b200_unregister_query_bounds": (_i32, [_vp]),
    "bsi_b200_register_key_bounds": (_i32, [_vp, _vp, _i64, _i32]),
    "bsi_b200_unregister_key_bounds": (_i32, [_vp]),
    "bsi_b200_debug_exact_int_tiles": (_i32, [_vp]),
    "bsi_b200_recombine_i8": (_i32, [_vp, _i64, _i32, _i64, _vp, _i64, _vp]),
    "bsi_b200_dot_i8": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _f32, _vp, _i64, _vp, _i32, _vp]),
    "bsi_b200_linear_i8": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _f32, _vp, _i64, _i32, _vp]),
    "bsi_b200_linear_i8_act": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _f32, _vp, _i64, _i32, _i32, _vp]),
    "bsi_b200_linear_i8_scatter": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _f32, _i32, _vp, _i64, _i64, _i32, _i32, _vp]),
    "bsi_b200_quantize_pack_multi": (_i32, [_vp, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _vp, _i64, _i32, _vp, _i64, _vp]),
    "bsi_b200_linear_i8_requant": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _f32, _i32, _i32, _i32, _i32,
                                          _i32, _vp, _i64, _vp, _i64, _vp]),
    "bsi_b200_add_layernorm_pack": (_i32, [_vp, _vp, _vp, _vp, _f32, _i32, _i64, _i64, _vp, _i32, _i32, _i32, _vp, _i64, _i32, _vp, _i64, _vp]),
    "bsi_b200_peer_alloc": (_i32, [_i64, _vp, _vp]),
    "bsi_b200_peer_free": (_i32, [_vp]),
    "bsi_b200_peer_open": (_i32, [_vp, _vp]),
    "bsi_b200_peer_close": (_i32, [_vp]),
    "bsi_b200_peer_barrier": (_i32, [_vp, _i32, _i32, _i64, _vp]),
    "bsi_b200_dot_words": (_i32, [_vp, _vp, _i64, _i32, _i64, _vp, _vp, _i32, _i64, _i64, _f32, _i64, _vp, _vp, _vp]),
    "bsi_b200_ewah_flags": (_i32, [_vp, _i64, _i64, _f64, _vp, _vp, _vp]),
    "bsi_b200_ewah_size": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp]),
    "bsi_b200_ewah_offsets": (_i32, [_vp, _i64, _vp, _vp, _vp]),
    "bsi_b200_ewah_emit": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "bsi_b200_ewah_decode": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp, _vp]),
    "bsi_b200_ewah_scratch_bytes": (_i64, [_i64]),
    "bsi_b200_ewah_encode": (_i32, [_vp, _i64, _i64, _f64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _vp]),
    "bsi_b200_ewah_encode_static": (_i32, [_vp, _i64, _i64, _f64, _vp, _i64, _vp, _vp, _vp, _vp, _vp]),
    "bsi_b200_cast_bias": (_i32, [_vp, _i64, _vp, _i64, _i64, _vp, _i64, _i32, _vp]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} not found: build it with `python -m bsipytorch_b200.build` "
                          "(there is no fallback path)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class BsiError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        L = lib()
        super().__init__(f"{what}: {L.bsi_b200_status_string(code).decode()} ({L.bsi_b200_last_error().decode()})")


def check(code, what="bsi_b200 call"):
    if code != OK:
        raise BsiError(code, what)


def ptr(t):
    """Device (or host) address of a torch tensor / None."""
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def exact_int_tiles() -> int:
    """(warp, tile) pairs of the paired tensor-core kernel that took the integer route since the last call."""
    v = C.c_ulonglong(0)
    check(lib().bsi_b200_debug_exact_int_tiles(C.byref(v)), "bsi_b200_debug_exact_int_tiles")
    return v.value


def device_status() -> int:
    v = C.c_int(0)
    check(lib().bsi_b200_device_status(C.byref(v)), "bsi_b200_device_status")
    return v.value
