// Fused quantise + bit-slice pack kernels (queries: per-256-element chunk scale; keys: per-row
// scale), the slice -> int8 recombination, and the cast+bias layer epilogue.
//
// One warp owns one 256-element chunk of one row: lane L holds elements 8L..8L+7, read with one
// 16-byte (f16/bf16) or two 16-byte (f32) loads, so a warp reads 512 B / 1 KiB contiguously.
// The largest |v| of the chunk is reduced with shuffles, the 8 clamped values of a lane are
// bit-transposed in registers (8x8), and byte s of the result is the lane's byte of slice s:
// byte (L % 8) of word (L / 8) of the chunk. The int8 image is written 8 bytes per lane.
//
// Arithmetic follows the reference bit for bit (bsi_cuda_kernels_quant.cuh:24-29, 82-108,
// 291-341, 414-488): v = half_away(double(float(x)) * 10^dp); bits = 64 - clz(max|v|);
// shift = clamp(bits - (b-1), 0, 62); q = sign(v) * ((|v| + (shift ? 1 << (shift-1) : 0)) >> shift),
// clamped to [-2^(b-1), 2^(b-1)-1].
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace bsi {
namespace {

typedef unsigned long long u64;

template <typename T>
__device__ __forceinline__ float to_float(T v) { return static_cast<float>(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ long long round_half_away(double x) {
    if (x >= 0.0) return static_cast<long long>(floor(x + 0.5));
    return -static_cast<long long>(floor(-x + 0.5));
}

__device__ __forceinline__ u64 uabs(long long v) { return static_cast<u64>(v >= 0 ? v : -v); }

// half_away(double(f) * 10^dp) in integer arithmetic, bit for bit the value the float64 expression
// gives. With f = m * 2^e (m < 2^24) and mult = 10^dp < 2^27 the product m * mult has at most 51
// bits, so the float64 multiply is exact, and so is the + 0.5 before the floor wherever it can change
// the result; half-away rounding of the exact value is (|P| + 2^(s-1)) >> s. NaN gives 0 and
// magnitudes of 2^63 or more saturate, which is what the float64 -> int64 conversion does.
// mult == 0 selects the float64 path (decimal_places outside [0, 8]).
__device__ __forceinline__ long long decimal_round(float f, double dec_scale, uint32_t mult) {
    if (mult == 0u) return round_half_away(static_cast<double>(f) * dec_scale);
    const uint32_t bits = __float_as_uint(f);
    const uint32_t exp = (bits >> 23) & 0xffu;
    uint32_t man = bits & 0x7fffffu;
    const bool neg = (bits >> 31) != 0u;
    u64 mag;
    if (exp == 255u) {
        mag = man ? 0ull : 0x7fffffffffffffffull;
    } else {
        int e;
        if (exp == 0u) {
            e = -149;
        } else {
            man |= 0x800000u;
            e = static_cast<int>(exp) - 150;
        }
        const u64 P = static_cast<u64>(man) * static_cast<u64>(mult);
        if (e >= 0) {
            mag = (e >= 63 || (P >> (63 - e)) != 0ull) ? (P ? 0x7fffffffffffffffull : 0ull) : (P << e);
        } else {
            const int sh = -e;
            mag = sh >= 53 ? 0ull : ((P + (1ull << (sh - 1))) >> sh);
        }
    }
    return neg ? -static_cast<long long>(mag) : static_cast<long long>(mag);
}

__device__ __forceinline__ u64 warp_max_u64(u64 v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const u64 o = __shfl_xor_sync(0xffffffffu, v, off);
        v = o > v ? o : v;
    }
    return v;
}

__device__ __forceinline__ int shift_for(u64 max_abs, int bits) {
    const int width = max_abs ? (64 - __clzll(static_cast<long long>(max_abs))) : 0;
    int shift = width - (bits - 1);
    shift = shift < 0 ? 0 : shift;
    return shift > 62 ? 62 : shift;
}

// Transposes the 8x8 bit matrix held in x (row e = byte e, LSB first): afterwards bit e of
// byte s is the former bit s of byte e.
__device__ __forceinline__ u64 transpose8x8(u64 x) {
    u64 t;
    t = (x ^ (x >> 7)) & 0x00AA00AA00AA00AAull;
    x = x ^ t ^ (t << 7);
    t = (x ^ (x >> 14)) & 0x0000CCCC0000CCCCull;
    x = x ^ t ^ (t << 14);
    t = (x ^ (x >> 28)) & 0x00000000F0F0F0F0ull;
    x = x ^ t ^ (t << 28);
    return x;
}

// Loads the 8 elements [col, col+8) of a row as float; elements at or beyond D read as 0.
template <typename T>
__device__ __forceinline__ void load8(const T* __restrict__ row, int64_t col, int64_t D, bool vec_ok,
                                      float (&f)[8]) {
    if (vec_ok && col + 8 <= D) {
        if constexpr (sizeof(T) == 2) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row + col));
            const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = to_float(h[e]);
        } else {
            const float4 a = __ldg(reinterpret_cast<const float4*>(row + col));
            const float4 b = __ldg(reinterpret_cast<const float4*>(row + col) + 1);
            f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
            f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
        }
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = (col + e < D) ? to_float(row[col + e]) : 0.0f;
    }
}

// Writes the lane's 8 clamped values (one byte each in `packed`): int8 image and bit slices.
__device__ __forceinline__ void store_packed(u64 packed, int bits, int lane, int64_t chunk, int64_t W,
                                             u64* __restrict__ words_row, int8_t* __restrict__ q8_row) {
    if (q8_row != nullptr) {
        *reinterpret_cast<u64*>(q8_row + chunk * 256 + lane * 8) = packed;
    }
    if (words_row != nullptr) {
        const int64_t word = chunk * 4 + (lane >> 3);
        if (word < W) {
            const u64 t = transpose8x8(packed);
            uint8_t* dst = reinterpret_cast<uint8_t*>(words_row + word) + (lane & 7);
            for (int s = 0; s < bits; ++s) {
                dst[static_cast<size_t>(s) * static_cast<size_t>(W) * 8u] =
                    static_cast<uint8_t>(t >> (8 * s));
            }
        }
    }
}

// Quantises the lane's 8 integers with `shift`, clamps, writes slices and the int8 image.
__device__ __forceinline__ void emit_chunk(const long long (&v)[8], int shift, int bits, int lane,
                                           int64_t chunk, int64_t W, u64* __restrict__ words_row,
                                           int8_t* __restrict__ q8_row) {
    const long long qmax = (1ll << (bits - 1)) - 1ll;
    const long long qmin = -(1ll << (bits - 1));
    const u64 round_add = shift > 0 ? (1ull << (shift - 1)) : 0ull;
    u64 packed = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const u64 uq = (uabs(v[e]) + round_add) >> shift;
        long long q = v[e] < 0 ? -static_cast<long long>(uq) : static_cast<long long>(uq);
        q = q < qmin ? qmin : q;
        q = q > qmax ? qmax : q;
        packed |= (static_cast<u64>(q) & 0xffull) << (8 * e);
    }
    store_packed(packed, bits, lane, chunk, W, words_row, q8_row);
}

// 32-bit variant of the quantiser for the common case (10^dp <= 127 and every |x| of the warp's chunk
// below 2^23, so that every product and magnitude fits 32 bits). Same integers as the 64-bit path.
__device__ __forceinline__ uint32_t decimal_round_mag32(uint32_t fbits, uint32_t mult) {
    const uint32_t exp = (fbits >> 23) & 0xffu;
    const uint32_t man = (fbits & 0x7fffffu) | (exp ? 0x800000u : 0u);
    const uint32_t sh = 150u - exp;  // >= 1 on this path; denormals get sh = 150
    const uint32_t P = man * mult;   // < 2^31
    return sh >= 32u ? 0u : ((P + (1u << (sh - 1u))) >> sh);
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_pack_chunk_kernel(
    const T* __restrict__ x, int64_t rows, int64_t D, int64_t ldx, double dec_scale, uint32_t dec_mult, int bits,
    int64_t chunks, int64_t W, u64* __restrict__ words, float* __restrict__ scales,
    int32_t* __restrict__ shifts, int8_t* __restrict__ q8, int64_t ld8, int vec_ok) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (unit >= rows * chunks) return;
    const int64_t row = unit / chunks;
    const int64_t chunk = unit - row * chunks;

    float f[8];
    load8<T>(x + row * ldx, chunk * 256 + lane * 8, D, vec_ok != 0, f);
    u64* words_row = words != nullptr ? words + row * bits * W : nullptr;
    int8_t* q8_row = q8 != nullptr ? q8 + row * ld8 : nullptr;

    bool fast = dec_mult != 0u && dec_mult <= 127u;
    if (fast) {
        uint32_t big = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) big |= (((__float_as_uint(f[e]) >> 23) & 0xffu) >= 150u) ? 1u : 0u;
        fast = !__any_sync(0xffffffffu, big != 0u);
    }
    if (fast) {
        uint32_t mag[8];
        uint32_t mx32 = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            mag[e] = decimal_round_mag32(__float_as_uint(f[e]), dec_mult);
            mx32 = mag[e] > mx32 ? mag[e] : mx32;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const uint32_t o = __shfl_xor_sync(0xffffffffu, mx32, off);
            mx32 = o > mx32 ? o : mx32;
        }
        int shift = (mx32 ? 32 - __clz(static_cast<int>(mx32)) : 0) - (bits - 1);
        shift = shift < 0 ? 0 : shift;
        if (lane == 0) {
            if (scales != nullptr) scales[unit] = static_cast<float>(1u << shift);
            if (shifts != nullptr) shifts[unit] = shift;
        }
        const int qmax = (1 << (bits - 1)) - 1;
        const int qmin = -(1 << (bits - 1));
        const uint32_t round_add = shift > 0 ? (1u << (shift - 1)) : 0u;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int q = static_cast<int>((mag[e] + round_add) >> shift);
            q = (__float_as_uint(f[e]) >> 31) ? -q : q;
            q = q > qmax ? qmax : q;
            q = q < qmin ? qmin : q;                      // a negative value may use the extra level -2^(b-1)
            const uint32_t byte = static_cast<uint32_t>(q) & 0xffu;
            if (e < 4) lo |= byte << (8 * e); else hi |= byte << (8 * (e - 4));
        }
        store_packed(static_cast<u64>(lo) | (static_cast<u64>(hi) << 32), bits, lane, chunk, W, words_row, q8_row);
        return;
    }

    long long v[8];
    u64 mx = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        v[e] = decimal_round(f[e], dec_scale, dec_mult);
        const u64 a = uabs(v[e]);
        mx = a > mx ? a : mx;
    }
    mx = warp_max_u64(mx);
    const int shift = shift_for(mx, bits);
    if (lane == 0) {
        if (scales != nullptr) scales[unit] = static_cast<float>(1ull << shift);
        if (shifts != nullptr) shifts[unit] = shift;
    }
    emit_chunk(v, shift, bits, lane, chunk, W, words_row, q8_row);
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_pack_row_kernel(
    const T* __restrict__ x, int64_t rows, int64_t D, int64_t ldx, double dec_scale, uint32_t dec_mult, int bits,
    int64_t chunks, int64_t W, u64* __restrict__ words, float* __restrict__ scales,
    int32_t* __restrict__ shifts, int8_t* __restrict__ q8, int64_t ld8, int vec_ok) {
    __shared__ u64 warp_max[8];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t row = blockIdx.x;
    const T* xr = x + row * ldx;

    u64 mx = 0;
    for (int64_t chunk = warp; chunk < chunks; chunk += 8) {
        float f[8];
        load8<T>(xr, chunk * 256 + lane * 8, D, vec_ok != 0, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const u64 a = uabs(decimal_round(f[e], dec_scale, dec_mult));
            mx = a > mx ? a : mx;
        }
    }
    mx = warp_max_u64(mx);
    if (lane == 0) warp_max[warp] = mx;
    __syncthreads();
    mx = warp_max[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = warp_max[i] > mx ? warp_max[i] : mx;
    const int shift = shift_for(mx, bits);
    if (threadIdx.x == 0) {
        if (scales != nullptr) scales[row] = static_cast<float>(1ull << shift);
        if (shifts != nullptr) shifts[row] = shift;
    }
    for (int64_t chunk = warp; chunk < chunks; chunk += 8) {
        float f[8];
        load8<T>(xr, chunk * 256 + lane * 8, D, vec_ok != 0, f);
        long long v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = decimal_round(f[e], dec_scale, dec_mult);
        emit_chunk(v, shift, bits, lane, chunk, W,
                   words != nullptr ? words + row * bits * W : nullptr,
                   q8 != nullptr ? q8 + row * ld8 : nullptr);
    }
}

__global__ void __launch_bounds__(256) recombine_i8_kernel(
    const u64* __restrict__ words, int64_t rows, int bits, int64_t W, int64_t chunks,
    int8_t* __restrict__ q8, int64_t ld8) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (unit >= rows * chunks) return;
    const int64_t row = unit / chunks;
    const int64_t chunk = unit - row * chunks;
    const int64_t word = chunk * 4 + (lane >> 3);
    u64 t = 0;
    if (word < W) {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(words + row * bits * W + word) + (lane & 7);
        for (int s = 0; s < bits; ++s) {
            t |= static_cast<u64>(src[static_cast<size_t>(s) * static_cast<size_t>(W) * 8u]) << (8 * s);
        }
    }
    u64 vals = transpose8x8(t);  // byte e = the `bits`-bit two's-complement value of element e
    // Sign-extend each byte from `bits` bits: where bit (bits-1) is set, set the bits above it.
    // sign holds 0 or 1 per byte and fill < 256, so the product never carries across bytes.
    const u64 sign = (vals >> (bits - 1)) & 0x0101010101010101ull;
    const u64 fill = (0xffull << bits) & 0xffull;
    vals |= sign * fill;
    *reinterpret_cast<u64*>(q8 + row * ld8 + chunk * 256 + lane * 8) = vals;
}

template <typename Y>
__device__ __forceinline__ Y from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// y = cast(out) + cast(bias), the add evaluated in float on the two already-narrowed values and
// narrowed again, which is what the reference's `scores.to(dtype) + bias.to(dtype)` does.
template <typename Y>
__global__ void __launch_bounds__(256) cast_bias_kernel(const float* __restrict__ out, int64_t ldo,
                                                        const float* __restrict__ bias, int64_t Q,
                                                        int64_t R, Y* __restrict__ y, int64_t ldy) {
    const int64_t per_row = (R + 3) / 4;
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= Q * per_row) return;
    const int64_t q = idx / per_row;
    const int64_t r0 = (idx - q * per_row) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int64_t r = r0 + e;
        if (r < R) {
            const Y narrowed = from_float<Y>(out[q * ldo + r]);
            if (bias != nullptr) {
                const Y b = from_float<Y>(bias[r]);
                y[q * ldy + r] = from_float<Y>(to_float(narrowed) + to_float(b));
            } else {
                y[q * ldy + r] = narrowed;
            }
        }
    }
}

}  // namespace
}  // namespace bsi

extern "C" int bsi_b200_quantize_pack(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx,
                                      int decimal_places, int bits, int chunk_mode,
                                      uint64_t* words, float* scales, int32_t* shifts,
                                      int8_t* q8, int64_t ld8, bsi_stream_t stream_) {
    using namespace bsi;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (rows < 0 || D < 0 || ldx < D) return fail(BSI_ERR_INVALID, "quantize_pack: bad rows/D/ldx");
    if (bits < 2 || bits > 8) return fail(BSI_ERR_UNSUPPORTED, "quantize_pack: bits must be in [2, 8]");
    if (dtype != BSI_DTYPE_F32 && dtype != BSI_DTYPE_F16 && dtype != BSI_DTYPE_BF16)
        return fail(BSI_ERR_INVALID, "quantize_pack: unknown dtype");
    if (rows == 0 || D == 0) return BSI_OK;
    if (x == nullptr) return fail(BSI_ERR_INVALID, "quantize_pack: x is null");
    const int64_t chunks = (D + 255) / 256;
    const int64_t W = (D + 63) / 64;
    if (q8 != nullptr) {
        if (ld8 < chunks * 256 || (ld8 & 15) != 0 || (reinterpret_cast<uintptr_t>(q8) & 15) != 0)
            return fail(BSI_ERR_INVALID, "quantize_pack: q8 needs ld8 >= 256*ceil(D/256), ld8 % 16 == 0, 16-byte base");
    }
    if (int rc = require_sm100()) return rc;
    const int esz = dtype == BSI_DTYPE_F32 ? 4 : 2;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0 && ((ldx * esz) & 15) == 0) ? 1 : 0;
    const double dec_scale = pow(10.0, static_cast<double>(decimal_places));
    uint32_t dec_mult = 0;  // 10^dp when it is a small integer; 0 = use the float64 expression
    if (decimal_places >= 0 && decimal_places <= 8) {
        dec_mult = 1;
        for (int i = 0; i < decimal_places; ++i) dec_mult *= 10u;
    }
    u64* w = reinterpret_cast<u64*>(words);

#define BSI_LAUNCH_PACK(T)                                                                        \
    do {                                                                                          \
        if (chunk_mode) {                                                                         \
            const int64_t blocks = (rows * chunks + 7) / 8;                                       \
            quantize_pack_chunk_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(     \
                static_cast<const T*>(x), rows, D, ldx, dec_scale, dec_mult, bits, chunks, W, w, scales,    \
                shifts, q8, ld8, vec_ok);                                                         \
        } else {                                                                                  \
            quantize_pack_row_kernel<T><<<static_cast<unsigned>(rows), 256, 0, stream>>>(         \
                static_cast<const T*>(x), rows, D, ldx, dec_scale, dec_mult, bits, chunks, W, w, scales,    \
                shifts, q8, ld8, vec_ok);                                                         \
        }                                                                                         \
    } while (0)

    if ((chunk_mode ? (rows * chunks + 7) / 8 : rows) > 0x7fffffffll)
        return fail(BSI_ERR_UNSUPPORTED, "quantize_pack: too many rows for one launch");
    if (dtype == BSI_DTYPE_F32) BSI_LAUNCH_PACK(float);
    else if (dtype == BSI_DTYPE_F16) BSI_LAUNCH_PACK(__half);
    else BSI_LAUNCH_PACK(__nv_bfloat16);
#undef BSI_LAUNCH_PACK
    return check_launch("quantize_pack launch");
}

extern "C" int bsi_b200_recombine_i8(const uint64_t* words, int64_t rows, int bits, int64_t W,
                                     int8_t* q8, int64_t ld8, bsi_stream_t stream_) {
    using namespace bsi;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (rows < 0 || W <= 0) return fail(BSI_ERR_INVALID, "recombine_i8: bad rows/W");
    if (bits < 2 || bits > 8) return fail(BSI_ERR_UNSUPPORTED, "recombine_i8: bits must be in [2, 8]");
    if (rows == 0) return BSI_OK;
    if (words == nullptr || q8 == nullptr) return fail(BSI_ERR_INVALID, "recombine_i8: null pointer");
    const int64_t chunks = (W + 3) / 4;
    if (ld8 < chunks * 256 || (ld8 & 15) != 0 || (reinterpret_cast<uintptr_t>(q8) & 15) != 0)
        return fail(BSI_ERR_INVALID, "recombine_i8: q8 needs ld8 >= 256*ceil(W/4), ld8 % 16 == 0, 16-byte base");
    if (int rc = require_sm100()) return rc;
    const int64_t blocks = (rows * chunks + 7) / 8;
    if (blocks > 0x7fffffffll) return fail(BSI_ERR_UNSUPPORTED, "recombine_i8: too many rows for one launch");
    recombine_i8_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const u64*>(words), rows, bits, W, chunks, q8, ld8);
    return check_launch("recombine_i8 launch");
}

extern "C" int bsi_b200_cast_bias(const float* out, int64_t ldo, const float* bias, int64_t Q, int64_t R,
                                  void* y, int64_t ldy, int y_dtype, bsi_stream_t stream_) {
    using namespace bsi;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (Q < 0 || R < 0 || ldo < R || ldy < R) return fail(BSI_ERR_INVALID, "cast_bias: bad Q/R/ld");
    if (Q == 0 || R == 0) return BSI_OK;
    if (out == nullptr || y == nullptr) return fail(BSI_ERR_INVALID, "cast_bias: null pointer");
    if (int rc = require_sm100()) return rc;
    const int64_t n = Q * ((R + 3) / 4);
    const int64_t blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffll) return fail(BSI_ERR_UNSUPPORTED, "cast_bias: too large for one launch");
    const unsigned g = static_cast<unsigned>(blocks);
    if (y_dtype == BSI_DTYPE_F32)
        cast_bias_kernel<float><<<g, 256, 0, stream>>>(out, ldo, bias, Q, R, static_cast<float*>(y), ldy);
    else if (y_dtype == BSI_DTYPE_F16)
        cast_bias_kernel<__half><<<g, 256, 0, stream>>>(out, ldo, bias, Q, R, static_cast<__half*>(y), ldy);
    else if (y_dtype == BSI_DTYPE_BF16)
        cast_bias_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(out, ldo, bias, Q, R,
                                                              static_cast<__nv_bfloat16*>(y), ldy);
    else
        return fail(BSI_ERR_INVALID, "cast_bias: unknown y_dtype");
    return check_launch("cast_bias launch");
}
