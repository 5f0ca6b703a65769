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
#include "quant_bytes.cuh"

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

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Shift selection with outlier clipping (bsi_cuda_kernels_quant.cuh:82-108, BSI_FIXED_CLIP_K > 0): the width comes
// from min(max |v|, clip_k * mean |v|) instead of max |v|, so a few extreme values no longer push the whole group
// to a coarse shift; they saturate at the clamp instead. `sum_abs` is the sum of the group's |v| (integers, so any
// summation order gives the same double below 2^53), `count` its number of elements.
__device__ __forceinline__ int shift_for_clipped(u64 max_abs, double sum_abs, int count, int bits, float clip_k) {
    int width = 0;
    if (count > 0) {
        double effective = static_cast<double>(max_abs);
        const double clip_max = (sum_abs / static_cast<double>(count)) * static_cast<double>(clip_k);
        if (clip_max < effective) effective = clip_max;
        if (effective > 0.0) (void)frexp(effective, &width);
    } else {
        width = max_abs ? (64 - __clzll(static_cast<long long>(max_abs))) : 0;
    }
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

// The same transposition on the two 32-bit halves (lo = rows 0..3, hi = rows 4..7): the first two exchange steps
// stay inside a half, the third swaps the high nibbles of lo with the low nibbles of hi.
__device__ __forceinline__ void transpose8x8_halves(uint32_t& lo, uint32_t& hi) {
    uint32_t t;
    t = (lo ^ (lo >> 7)) & 0x00AA00AAu;  lo = lo ^ t ^ (t << 7);
    t = (hi ^ (hi >> 7)) & 0x00AA00AAu;  hi = hi ^ t ^ (t << 7);
    t = (lo ^ (lo >> 14)) & 0x0000CCCCu; lo = lo ^ t ^ (t << 14);
    t = (hi ^ (hi >> 14)) & 0x0000CCCCu; hi = hi ^ t ^ (t << 14);
    t = (lo ^ (hi << 4)) & 0xF0F0F0F0u;
    lo ^= t;
    hi ^= t >> 4;
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
            const uint32_t tl = static_cast<uint32_t>(t), th = static_cast<uint32_t>(t >> 32);
            const size_t step = static_cast<size_t>(W) * 8u;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                if (s < bits) dst[s * step] = static_cast<uint8_t>((s < 4 ? tl : th) >> (8 * (s & 3)));
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

// Byte-wise tail of the fast paths: u[e] carries the unsigned quantised magnitude of element e in its
// low byte (0 .. 2^(bits-1)), f[e] the sign; returns the 8 two's-complement bytes.
__device__ __forceinline__ u64 sign_clamp_bytes(const uint32_t (&u)[8], const float (&f)[8], int bits) {
    const uint32_t lo = sign_clamp4(u[0], u[1], u[2], u[3], __float_as_uint(f[0]), __float_as_uint(f[1]),
                                    __float_as_uint(f[2]), __float_as_uint(f[3]), bits);
    const uint32_t hi = sign_clamp4(u[4], u[5], u[6], u[7], __float_as_uint(f[4]), __float_as_uint(f[5]),
                                    __float_as_uint(f[6]), __float_as_uint(f[7]), bits);
    return static_cast<u64>(lo) | (static_cast<u64>(hi) << 32);
}

// One (row, chunk) unit on the generic path (any decimal_places, any magnitude, NaN/inf, any layout):
// 64-bit integers and 64-bit offsets throughout.
template <typename T>
__device__ __forceinline__ void generic_unit(const T* __restrict__ x, int64_t unit, int64_t D, int64_t ldx,
                                             double dec_scale, uint32_t dec_mult, int bits, int64_t chunks, int64_t W,
                                             u64* __restrict__ words, float* __restrict__ scales,
                                             int32_t* __restrict__ shifts, int8_t* __restrict__ q8, int64_t ld8,
                                             bool vec, int lane, float clip_k = 0.0f,
                                             float* __restrict__ sq_norms = nullptr) {
    // no sum of squares from this path: infinity makes a dot's exactness test that reads it fail safely
    if (sq_norms != nullptr && lane == 0) sq_norms[unit] = __int_as_float(0x7f800000);
    const int64_t row = unit / chunks;
    const int64_t chunk = unit - row * chunks;
    float f[8];
    load8<T>(x + row * ldx, chunk * 256 + lane * 8, D, vec, f);
    long long v[8];
    u64 mx = 0;
    double sum = 0.0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        v[e] = decimal_round(f[e], dec_scale, dec_mult);
        const u64 a = uabs(v[e]);
        mx = a > mx ? a : mx;
        sum += static_cast<double>(a);     // elements beyond D were loaded as 0
    }
    mx = warp_max_u64(mx);
    int shift;
    if (clip_k > 0.0f) {
        const int64_t left = D - chunk * 256;
        shift = shift_for_clipped(mx, warp_sum_f64(sum), static_cast<int>(left < 256 ? left : 256), bits, clip_k);
    } else {
        shift = shift_for(mx, bits);
    }
    if (lane == 0) {
        if (scales != nullptr) scales[unit] = static_cast<float>(1ull << shift);
        if (shifts != nullptr) shifts[unit] = shift;
    }
    emit_chunk(v, shift, bits, lane, chunk, W, words != nullptr ? words + row * bits * W : nullptr,
               q8 != nullptr ? q8 + row * ld8 : nullptr);
}

// Chunk mode without preconditions: one warp per unit, grid-stride.
template <typename T>
__global__ void __launch_bounds__(256) quantize_pack_chunk_generic_kernel(
    const T* __restrict__ x, int64_t rows, int64_t D, int64_t ldx, double dec_scale, uint32_t dec_mult, int bits,
    int64_t chunks, int64_t W, u64* __restrict__ words, float* __restrict__ scales,
    int32_t* __restrict__ shifts, int8_t* __restrict__ q8, int64_t ld8, int vec_ok, float clip_k,
    float* __restrict__ sq_norms) {
    const int lane = threadIdx.x & 31;
    const int64_t total = rows * chunks;
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * 8)
        generic_unit<T>(x, unit, D, ldx, dec_scale, dec_mult, bits, chunks, W, words, scales, shifts, q8, ld8,
                        vec_ok != 0, lane, clip_k, sq_norms);
}

// Fast path of one chunk: true when the chunk was quantised and stored, false when it needs the generic
// path (some |x * 10^dp| >= 2^23, NaN or inf). Same integers as the generic path, far fewer instructions.
//
//  * 16-bit inputs, 10^dp <= 1000: an 11-bit (8-bit for bfloat16) significand times a 10-bit constant
//    has at most 21 bits, so y = |x| * 10^dp and y + 0.5 are exact in float32. Adding 2^23 with
//    round-toward-zero leaves 2^23 + floor(y + 0.5) = 2^23 + |v| (floats in [2^23, 2^24) are the
//    integers). The second rounding (|v| + 2^(s-1)) >> s = floor(|v| * 2^-s + 0.5) is the same step
//    again: u = fma(r1, 2^-s, 0.5 - 2^(23-s)) is exact and its 2^23-truncation carries the result in the
//    low mantissa byte. All of this runs on the FMA pipe.
//  * float32 inputs, 10^dp <= 127: 32-bit integer arithmetic on the float's bit pattern.
template <typename T>
__device__ __forceinline__ bool fast_quantise(const float (&f)[8], uint32_t dec_mult, int bits, int& shift, u64& packed) {
    uint32_t amax_bits = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax_bits = max(amax_bits, __float_as_uint(f[e]) & 0x7fffffffu);
    amax_bits = __reduce_max_sync(0xffffffffu, amax_bits);   // NaN and inf order above every finite value

    uint32_t u[8];
    if constexpr (sizeof(T) == 2) {
        const float fmult = static_cast<float>(dec_mult);
        const float ymax = __uint_as_float(amax_bits) * fmult;
        if (!(amax_bits < 0x7f800000u && ymax < 8388608.0f)) return false;
        shift = fast_shift(ymax, bits);   // rounding is monotonic: half_away(ymax) is the largest |v|
        float inv, c;
        fast_round_consts(shift, inv, c);
#pragma unroll
        for (int e = 0; e < 8; ++e) u[e] = fast_magnitude(f[e], fmult, inv, c);
    } else {
        if (!(amax_bits < (150u << 23))) return false;
        const uint32_t mx = decimal_round_mag32(amax_bits, dec_mult);
        shift = (32 - __clz(static_cast<int>(mx))) - (bits - 1);
        shift = shift < 0 ? 0 : shift;
        const uint32_t round_add = shift > 0 ? (1u << (shift - 1)) : 0u;
#pragma unroll
        for (int e = 0; e < 8; ++e)
            u[e] = (decimal_round_mag32(__float_as_uint(f[e]), dec_mult) + round_add) >> shift;
    }
    packed = sign_clamp_bytes(u, f, bits);
    return true;
}

// Fast path of one chunk including its stores: true when the chunk was quantised and stored.
template <typename T, bool kWords, bool kQ8>
__device__ __forceinline__ bool fast_chunk(const float (&f)[8], uint32_t unit, uint32_t q8_off, uint32_t word_off,
                                           bool word_ok, int lane, uint32_t dec_mult, int bits, uint32_t slice_bytes,
                                           u64* __restrict__ words, float* __restrict__ scales,
                                           int32_t* __restrict__ shifts, int8_t* __restrict__ q8,
                                           float* __restrict__ sq_norms) {
    int shift;
    u64 packed;
    if (!fast_quantise<T>(f, dec_mult, bits, shift, packed)) return false;
    if (sq_norms != nullptr) {
        // sum of squares of the chunk's de-shifted integers, (2^shift)^2 * sum a^2: an exact float (the integer
        // sum is at most 256 * 128^2 = 2^22), which a dot's exactness test turns into a Cauchy-Schwarz bound
        int n2 = __dp4a(static_cast<int>(static_cast<uint32_t>(packed)), static_cast<int>(static_cast<uint32_t>(packed)), 0);
        n2 = __dp4a(static_cast<int>(static_cast<uint32_t>(packed >> 32)), static_cast<int>(static_cast<uint32_t>(packed >> 32)), n2);
        n2 = __reduce_add_sync(0xffffffffu, n2);
        if (lane == 0) sq_norms[unit] = static_cast<float>(n2) * __uint_as_float(static_cast<uint32_t>(127 + 2 * shift) << 23);
    }
    if (lane == 0) {
        scales[unit] = __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);   // 2^shift
        if (shifts != nullptr) shifts[unit] = shift;
    }
    if constexpr (kQ8) *reinterpret_cast<u64*>(q8 + q8_off) = packed;
    if constexpr (kWords) {
        // After the 8x8 bit transposition a lane holds one byte of each slice. Four neighbouring lanes (half a
        // 64-bit word) trade bytes in two shuffle steps so that each ends up with the four bytes of two slices:
        // two 4-byte stores per lane instead of seven 1-byte stores.
        uint32_t tl = static_cast<uint32_t>(packed), th = static_cast<uint32_t>(packed >> 32);
        transpose8x8_halves(tl, th);
        const bool upper = (lane & 2) != 0;     // lanes 2, 3 of the group collect slices 4..7, lanes 0, 1 slices 0..3
        const bool odd = (lane & 1) != 0;       // odd lanes keep the second slice pair of their group
        const uint32_t got = __shfl_xor_sync(0xffffffffu, upper ? tl : th, 2);
        const uint32_t x = upper ? got : tl;    // the slice group's bytes of group lane (lane & 1)
        const uint32_t y = upper ? th : got;    // ... and of group lane (lane & 1) + 2
        const uint32_t keep = __byte_perm(x, y, odd ? 0x7632 : 0x5410);
        const uint32_t other = __shfl_xor_sync(0xffffffffu, __byte_perm(x, y, odd ? 0x5410 : 0x7632), 1);
        const uint32_t w0 = __byte_perm(keep, other, odd ? 0x2604 : 0x6240);   // bytes of group lanes 0, 1, 2, 3
        const uint32_t w1 = __byte_perm(keep, other, odd ? 0x3715 : 0x7351);
        if (word_ok) {
            const int s0 = ((lane & 2) << 1) + ((lane & 1) << 1);              // first of the lane's two slices
            uint8_t* out = reinterpret_cast<uint8_t*>(words);
            // word_off addresses the lane's own byte (word lane / 8, byte lane % 8); the 4-byte store goes to
            // the start of its half word
            const uint32_t off = word_off - (lane & 3) + static_cast<uint32_t>(s0) * slice_bytes;
            if (s0 < bits) *reinterpret_cast<uint32_t*>(out + off) = w0;
            if (s0 + 1 < bits) *reinterpret_cast<uint32_t*>(out + off + slice_bytes) = w1;
        }
    }
    return true;
}

// Raw 16-byte vectors holding a lane's 8 elements (one for 16-bit types, two for float32). Keeping
// the next unit's data in this form lets its load stay in flight while the current unit is processed.
template <typename T>
struct RawLane {
    static constexpr int kVecs = sizeof(T) == 2 ? 1 : 2;
    uint4 v[kVecs];
    __device__ __forceinline__ void load(const T* __restrict__ p) {
#pragma unroll
        for (int i = 0; i < kVecs; ++i) v[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
    }
    __device__ __forceinline__ void to_floats(float (&f)[8]) const {
        if constexpr (sizeof(T) == 2) {
            const T* h = reinterpret_cast<const T*>(&v[0]);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = to_float(h[e]);
        } else {
            const float* g = reinterpret_cast<const float*>(&v[0]);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = g[e];
        }
    }
};

#ifndef BSI_PACK_MIN_BLOCKS
#define BSI_PACK_MIN_BLOCKS 4
#endif

// Geometry of a fast chunk-mode launch; the host checks that every offset fits 32 bits.
struct FastGeom {
    uint32_t total, chunks, D, ldx, ld8, W;
    uint32_t row_bytes;     // bits * W * 8: bytes of one row's slices
    uint32_t slice_bytes;   // W * 8
};

constexpr int kSlowQueue = 8;   // units per warp that may wait for the generic path

// Persistent fast chunk kernel. The grid is sized to what is resident at once and every warp walks the
// (row, chunk) units with stride gridDim.x * 8, loading its next unit before it processes the current one
// (the loop is written out twice so that the two register buffers swap roles without copies). Units the
// fast path cannot take are queued and redone on the generic path after the loop, which keeps the 64-bit
// code out of the loop's register budget; a warp whose queue overflows redoes all of its units.
// kDense: x and q8 are contiguous (ldx == ld8 == D), D is a multiple of 256 and x is 16-byte aligned, so
// a unit's element offset is unit * 256 and no lane ever needs the scalar tail loads.
template <typename T, bool kDense, bool kWords, bool kQ8>
__global__ void __launch_bounds__(256, BSI_PACK_MIN_BLOCKS) quantize_pack_chunk_fast_kernel(
    const T* __restrict__ x, FastGeom g, double dec_scale, uint32_t dec_mult, int bits,
    u64* __restrict__ words, float* __restrict__ scales, int32_t* __restrict__ shifts, int8_t* __restrict__ q8,
    int vec_ok, float* __restrict__ sq_norms) {
    __shared__ uint32_t slow_queue[8][kSlowQueue];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t stride = gridDim.x * 8u;
    const uint32_t first = blockIdx.x * 8u + warp;
    if (first >= g.total) return;
    constexpr bool kRows = !kDense || kWords;   // row / chunk are needed, not just the unit number
    const uint32_t stride_rows = kRows ? stride / g.chunks : 0u;
    const uint32_t stride_chunks = kRows ? stride - stride_rows * g.chunks : 0u;
    const bool vec = kDense || vec_ok != 0;
    const uint32_t lane_col = lane * 8u;
    const uint32_t lane_word = (lane >> 3) * 8u + (lane & 7u);   // byte within the chunk's 4 words
    int nslow = 0;

    struct Pos { uint32_t unit, row, chunk; };
    auto advance = [&](Pos p) {
        p.unit += stride;
        if constexpr (kRows) {
            p.row += stride_rows; p.chunk += stride_chunks;
            if (p.chunk >= g.chunks) { p.chunk -= g.chunks; ++p.row; }
        }
        return p;
    };
    auto lane_vec = [&](const Pos& p) { return kDense || (vec && p.chunk * 256u + lane_col + 8u <= g.D); };
    auto fetch = [&](RawLane<T>& r, const Pos& p) {
        if constexpr (kDense) r.load(x + (p.unit * 256u + lane_col));
        else if (lane_vec(p)) r.load(x + (p.row * g.ldx + p.chunk * 256u + lane_col));
    };
    auto process = [&](const RawLane<T>& r, const Pos& p) {
        float f[8];
        if (lane_vec(p)) r.to_floats(f);
        else load8<T>(x + static_cast<int64_t>(p.row) * g.ldx, static_cast<int64_t>(p.chunk) * 256 + lane_col,
                      static_cast<int64_t>(g.D), false, f);
        const uint32_t q8_off = kDense ? p.unit * 256u + lane_col : p.row * g.ld8 + p.chunk * 256u + lane_col;
        const uint32_t word_off = kWords ? p.row * g.row_bytes + p.chunk * 32u + lane_word : 0u;
        const bool word_ok = kDense || p.chunk * 4u + (lane >> 3) < g.W;
        if (!fast_chunk<T, kWords, kQ8>(f, p.unit, q8_off, word_off, word_ok, lane, dec_mult, bits, g.slice_bytes,
                                        words, scales, shifts, q8, sq_norms)) {
            if (nslow < kSlowQueue && lane == 0) slow_queue[warp][nslow] = p.unit;
            ++nslow;
        }
    };

    Pos cur;
    cur.unit = first;
    cur.row = kRows ? first / g.chunks : 0u;
    cur.chunk = kRows ? first - cur.row * g.chunks : 0u;
    RawLane<T> a, b;
    fetch(a, cur);
    for (;;) {
        Pos nxt = advance(cur);
        bool more = nxt.unit < g.total;
        if (more) fetch(b, nxt);
        process(a, cur);
        if (!more) break;
        cur = nxt;
        nxt = advance(cur);
        more = nxt.unit < g.total;
        if (more) fetch(a, nxt);
        process(b, cur);
        if (!more) break;
        cur = nxt;
    }
    if (nslow == 0) return;
    __syncwarp();
    const int64_t ld8 = kDense ? g.D : g.ld8;
    if (nslow <= kSlowQueue) {
        for (int i = 0; i < nslow; ++i)
            generic_unit<T>(x, slow_queue[warp][i], g.D, g.ldx, dec_scale, dec_mult, bits, g.chunks, g.W, words, scales,
                            shifts, q8, ld8, vec, lane, 0.0f, sq_norms);
    } else {
        for (uint32_t unit = first; unit < g.total; unit += stride)
            generic_unit<T>(x, unit, g.D, g.ldx, dec_scale, dec_mult, bits, g.chunks, g.W, words, scales, shifts, q8,
                            ld8, vec, lane, 0.0f, sq_norms);
    }
}

// Destinations of the multi-destination pack: the same int8 image / chunk scales go to each of them.
struct MultiDst {
    int n_q8, n_scales;
    int8_t* q8[BSI_B200_MAX_PEERS];
    float* scales[BSI_B200_MAX_PEERS];
};

// Generic quantiser of one chunk without the stores (the multi-destination kernel's fallback).
__device__ __noinline__ void generic_quantise(float f0, float f1, float f2, float f3, float f4, float f5, float f6,
                                              float f7, double dec_scale, uint32_t dec_mult, int bits, int* shift_out,
                                              u64* packed_out) {
    const float f[8] = {f0, f1, f2, f3, f4, f5, f6, f7};
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
    *shift_out = shift;
    *packed_out = packed;
}

// Chunk-mode pack whose int8 image and chunk scales are stored to several destinations at once (own
// memory and peer mappings alike): element (row, col) at q8[i] + row * ld8 + col, the scale of
// (row, chunk) at scales[i] + row * scale_ld + chunk. Persistent warps with next-unit prefetch as in
// the fast kernel; D is a multiple of 256 and x is 16-byte aligned, so every lane loads vectors.
template <typename T>
__global__ void __launch_bounds__(256, BSI_PACK_MIN_BLOCKS) quantize_pack_multi_kernel(
    const T* __restrict__ x, uint32_t total, uint32_t chunks, uint32_t ldx, uint32_t ld8, uint32_t scale_ld,
    double dec_scale, uint32_t dec_mult, uint32_t fast_limit, int bits, const MultiDst dst) {
    const int lane = threadIdx.x & 31;
    const uint32_t stride = gridDim.x * 8u;
    const uint32_t first = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (first >= total) return;
    const uint32_t stride_rows = stride / chunks;
    const uint32_t stride_chunks = stride - stride_rows * chunks;
    const uint32_t lane_col = lane * 8u;
    const bool try_fast = dec_mult != 0u && dec_mult <= fast_limit;

    struct Pos { uint32_t unit, row, chunk; };
    auto advance = [&](Pos p) {
        p.unit += stride; p.row += stride_rows; p.chunk += stride_chunks;
        if (p.chunk >= chunks) { p.chunk -= chunks; ++p.row; }
        return p;
    };
    auto fetch = [&](RawLane<T>& r, const Pos& p) { r.load(x + (p.row * ldx + p.chunk * 256u + lane_col)); };
    auto process = [&](const RawLane<T>& r, const Pos& p) {
        float f[8];
        r.to_floats(f);
        int shift;
        u64 packed;
        if (!(try_fast && fast_quantise<T>(f, dec_mult, bits, shift, packed)))
            generic_quantise(f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7], dec_scale, dec_mult, bits, &shift, &packed);
        const uint32_t q8_off = p.row * ld8 + p.chunk * 256u + lane_col;
        const uint32_t sc_off = p.row * scale_ld + p.chunk;
        const float scale = __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);   // 2^shift, shift <= 62
#pragma unroll
        for (int i = 0; i < BSI_B200_MAX_PEERS; ++i) {
            if (i < dst.n_q8) *reinterpret_cast<u64*>(dst.q8[i] + q8_off) = packed;
            if (i < dst.n_scales && lane == 0) dst.scales[i][sc_off] = scale;
        }
    };

    Pos cur;
    cur.unit = first;
    cur.row = first / chunks;
    cur.chunk = first - cur.row * chunks;
    RawLane<T> a, b;
    fetch(a, cur);
    for (;;) {
        Pos nxt = advance(cur);
        bool more = nxt.unit < total;
        if (more) fetch(b, nxt);
        process(a, cur);
        if (!more) break;
        cur = nxt;
        nxt = advance(cur);
        more = nxt.unit < total;
        if (more) fetch(a, nxt);
        process(b, cur);
        if (!more) break;
        cur = nxt;
    }
}

// Residual add + LayerNorm + activation pack of one token row per block, for 16-bit layer types:
//   x_out = T(x + delta)                      (delta may be null: x_out = x)
//   y     = T((x_out - mean) * rstd * gamma + beta), float32 statistics over the row (two passes over registers)
//   y is quantised per 256-element chunk exactly as the chunk-mode packer would quantise it and the int8
//   image / chunk scales go to the destinations (own buffer or peer mappings), as in the multi-destination pack.
// Warp w owns chunks w, w + 8, ...; lane L the 8 consecutive elements 8L..8L+7 of each (the packer's mapping), so the
// row stays in registers between the add, the statistics and the quantisation. CPW = chunks per warp (H <= 2048*CPW).
template <typename T, int CPW>
__global__ void __launch_bounds__(256) add_layernorm_pack_kernel(
    const T* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ gamma, const T* __restrict__ beta,
    float eps, int rows, int H, int chunks, T* __restrict__ x_out, double dec_scale, uint32_t dec_mult,
    uint32_t fast_limit, int bits, int64_t ld8, int64_t scale_ld, const MultiDst dst) {
    __shared__ float red[2][8];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const bool try_fast = dec_mult != 0u && dec_mult <= fast_limit;
    const float inv_h = 1.0f / static_cast<float>(H);
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int64_t base = static_cast<int64_t>(row) * H;
        float v[CPW][8];
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < CPW; ++i) {
            const int c = warp + i * 8;
            if (c < chunks) {
                const int64_t off = base + c * 256 + lane * 8;
                uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + off));
                const T* xv = reinterpret_cast<const T*>(&raw);
                if (delta != nullptr) {
                    const uint4 draw = __ldg(reinterpret_cast<const uint4*>(delta + off));
                    const T* dv = reinterpret_cast<const T*>(&draw);
                    T ov[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        ov[e] = static_cast<T>(to_float(xv[e]) + to_float(dv[e]));
                        v[i][e] = to_float(ov[e]);
                    }
                    *reinterpret_cast<uint4*>(x_out + off) = *reinterpret_cast<const uint4*>(ov);
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[i][e] = to_float(xv[e]);
                    if (x_out != x) *reinterpret_cast<uint4*>(x_out + off) = raw;
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) sum += v[i][e];
            }
        }
        // mean
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) red[0][warp] = sum;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += red[0][w];
        const float mean = tot * inv_h;
        // variance around the mean
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < CPW; ++i) {
            if (warp + i * 8 < chunks) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float d = v[i][e] - mean;
                    sq = fmaf(d, d, sq);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) red[1][warp] = sq;
        __syncthreads();
        float tsq = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tsq += red[1][w];
        const float rstd = rsqrtf(tsq * inv_h + eps);
        // normalise, round to the layer type, quantise the chunk, store everywhere
#pragma unroll
        for (int i = 0; i < CPW; ++i) {
            const int c = warp + i * 8;
            if (c < chunks) {
                const int col = c * 256 + lane * 8;
                const uint4 graw = __ldg(reinterpret_cast<const uint4*>(gamma + col));
                const uint4 braw = __ldg(reinterpret_cast<const uint4*>(beta + col));
                const T* gv = reinterpret_cast<const T*>(&graw);
                const T* bv = reinterpret_cast<const T*>(&braw);
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    f[e] = to_float(static_cast<T>(fmaf((v[i][e] - mean) * rstd, to_float(gv[e]), to_float(bv[e]))));
                int shift;
                u64 packed;
                if (!(try_fast && fast_quantise<T>(f, dec_mult, bits, shift, packed)))
                    generic_quantise(f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7], dec_scale, dec_mult, bits, &shift,
                                     &packed);
                const int64_t q8_off = static_cast<int64_t>(row) * ld8 + col;
                const int64_t sc_off = static_cast<int64_t>(row) * scale_ld + c;
                const float scale = __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);
#pragma unroll
                for (int d = 0; d < BSI_B200_MAX_PEERS; ++d) {
                    if (d < dst.n_q8) *reinterpret_cast<u64*>(dst.q8[d] + q8_off) = packed;
                    if (d < dst.n_scales && lane == 0) dst.scales[d][sc_off] = scale;
                }
            }
        }
        __syncthreads();   // red[] is rewritten by the next row
    }
}

// ---- variable-slice mode (no shift: the decimal integers themselves are sliced) ---------------------------------
// Pass 1: largest |v| and "has a negative" per row, v = half_away(double(float(x)) * 10^dp). The reference takes
// them with torch reductions over the int64 tensor (bsi_vector_cuda.cpp:1089-1099, 1156-1159).
template <typename T>
__global__ void __launch_bounds__(256) decimal_absmax_kernel(const T* __restrict__ x, int64_t rows, int64_t D, int64_t ldx,
                                                             double dec_scale, uint32_t dec_mult, int64_t chunks, int vec_ok,
                                                             u64* __restrict__ row_absmax, int32_t* __restrict__ row_negative) {
    __shared__ u64 wmax[8];
    __shared__ int wneg[8];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t row = blockIdx.x;
    const T* xr = x + row * ldx;
    u64 mx = 0;
    int neg = 0;
    for (int64_t chunk = warp; chunk < chunks; chunk += 8) {
        float f[8];
        load8<T>(xr, chunk * 256 + lane * 8, D, vec_ok != 0, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const long long v = decimal_round(f[e], dec_scale, dec_mult);
            const u64 a = uabs(v);
            mx = a > mx ? a : mx;
            neg |= v < 0 ? 1 : 0;
        }
    }
    mx = warp_max_u64(mx);
    neg = __any_sync(0xffffffffu, neg) ? 1 : 0;
    if (lane == 0) {
        wmax[warp] = mx;
        wneg[warp] = neg;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 m = 0;
        int n = 0;
        for (int w = 0; w < 8; ++w) {
            m = wmax[w] > m ? wmax[w] : m;
            n |= wneg[w];
        }
        row_absmax[row] = m;
        row_negative[row] = n;
    }
}

// Pass 2: the low `slices` bits of the two's-complement integers as bit slices (what launch_pack_bits_all_ballot_batch
// writes, bsi_cuda_kernels_pack.cuh:129-174, 204-230), plus, for the tensor-core dot, the integers as two signed
// 8-bit digits: v = 128 * hi + lo with lo in [0, 127] (hi8 may be NULL when every |v| <= 127: lo8 then holds v itself).
// One warp per 256-element chunk, lane = 8 elements, byte (lane % 8) of word (lane / 8) of each slice.
template <typename T>
__global__ void __launch_bounds__(256) pack_plain_kernel(const T* __restrict__ x, int64_t rows, int64_t D, int64_t ldx,
                                                         double dec_scale, uint32_t dec_mult, int slices, int64_t chunks,
                                                         int64_t W, int vec_ok, u64* __restrict__ words,
                                                         int8_t* __restrict__ lo8, int8_t* __restrict__ hi8, int64_t ld8) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (unit >= rows * chunks) return;
    const int64_t row = unit / chunks;
    const int64_t chunk = unit - row * chunks;
    float f[8];
    load8<T>(x + row * ldx, chunk * 256 + lane * 8, D, vec_ok != 0, f);
    long long v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = decimal_round(f[e], dec_scale, dec_mult);
    if (lo8 != nullptr) {
        u64 lo = 0, hi = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (hi8 != nullptr) {
                lo |= static_cast<u64>(v[e] & 127) << (8 * e);
                hi |= static_cast<u64>((v[e] >> 7) & 255) << (8 * e);
            } else {
                lo |= static_cast<u64>(v[e] & 255) << (8 * e);
            }
        }
        *reinterpret_cast<u64*>(lo8 + row * ld8 + chunk * 256 + lane * 8) = lo;
        if (hi8 != nullptr) *reinterpret_cast<u64*>(hi8 + row * ld8 + chunk * 256 + lane * 8) = hi;
    }
    if (words != nullptr) {
        const int64_t word = chunk * 4 + (lane >> 3);
        if (word < W) {
            uint8_t* base = reinterpret_cast<uint8_t*>(words + (row * slices) * W + word) + (lane & 7);
            for (int s = 0; s < slices; ++s) {
                uint32_t byte = 0;
#pragma unroll
                for (int e = 0; e < 8; ++e) byte |= static_cast<uint32_t>((v[e] >> s) & 1ll) << e;
                base[static_cast<int64_t>(s) * W * 8] = static_cast<uint8_t>(byte);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_pack_row_kernel(
    const T* __restrict__ x, int64_t rows, int64_t D, int64_t ldx, double dec_scale, uint32_t dec_mult, int bits,
    int64_t chunks, int64_t W, u64* __restrict__ words, float* __restrict__ scales,
    int32_t* __restrict__ shifts, int8_t* __restrict__ q8, int64_t ld8, int vec_ok, float clip_k) {
    __shared__ u64 warp_max[8];
    __shared__ double warp_sum[8];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t row = blockIdx.x;
    const T* xr = x + row * ldx;

    u64 mx = 0;
    double sum = 0.0;
    for (int64_t chunk = warp; chunk < chunks; chunk += 8) {
        float f[8];
        load8<T>(xr, chunk * 256 + lane * 8, D, vec_ok != 0, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const u64 a = uabs(decimal_round(f[e], dec_scale, dec_mult));
            mx = a > mx ? a : mx;
            if (clip_k > 0.0f) sum += static_cast<double>(a);
        }
    }
    mx = warp_max_u64(mx);
    if (clip_k > 0.0f) sum = warp_sum_f64(sum);
    if (lane == 0) {
        warp_max[warp] = mx;
        warp_sum[warp] = sum;
    }
    __syncthreads();
    mx = warp_max[0];
    sum = warp_sum[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) {
        mx = warp_max[i] > mx ? warp_max[i] : mx;
        sum += warp_sum[i];
    }
    const int shift = clip_k > 0.0f ? shift_for_clipped(mx, sum, static_cast<int>(D), bits, clip_k) : shift_for(mx, bits);
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

namespace bsi {
namespace {
// Blocks of 256 threads of `kernel` that fit the current device at once (cached per kernel).
template <typename K>
int64_t resident_blocks(K kernel) {
    static thread_local int cached_dev = -1;
    static thread_local K cached_fn = nullptr;
    static thread_local int cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { set_error("quantize_pack: cudaGetDevice failed"); return -1; }
    if (dev != cached_dev || kernel != cached_fn) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0) != cudaSuccess || per_sm <= 0) {
            set_error("quantize_pack: occupancy query failed");
            return -1;
        }
        cached = per_sm * sm_count();
        cached_dev = dev;
        cached_fn = kernel;
    }
    return cached;
}
struct ChunkArgs {
    int64_t rows, D, ldx, ld8, chunks, W;
    double dec_scale;
    uint32_t dec_mult;
    int bits;
    u64* words;
    float* scales;
    int32_t* shifts;
    int8_t* q8;
    int vec_ok;
    cudaStream_t stream;
    float clip_k;
    float* sq_norms;
};

template <typename T, bool kDense, bool kWords, bool kQ8>
int launch_chunk_fast(const T* x, const ChunkArgs& a) {
    const int64_t resident = resident_blocks(quantize_pack_chunk_fast_kernel<T, kDense, kWords, kQ8>);
    if (resident <= 0) return BSI_ERR_CUDA;
    int64_t blocks = (a.rows * a.chunks + 7) / 8;
    blocks = blocks < resident ? blocks : resident;
    FastGeom g;
    g.total = static_cast<uint32_t>(a.rows * a.chunks);
    g.chunks = static_cast<uint32_t>(a.chunks);
    g.D = static_cast<uint32_t>(a.D);
    g.ldx = static_cast<uint32_t>(a.ldx);
    g.ld8 = static_cast<uint32_t>(kQ8 ? a.ld8 : 0);
    g.W = static_cast<uint32_t>(a.W);
    g.row_bytes = static_cast<uint32_t>(a.bits * a.W * 8);
    g.slice_bytes = static_cast<uint32_t>(a.W * 8);
    quantize_pack_chunk_fast_kernel<T, kDense, kWords, kQ8><<<static_cast<unsigned>(blocks), 256, 0, a.stream>>>(
        x, g, a.dec_scale, a.dec_mult, a.bits, a.words, a.scales, a.shifts, a.q8, a.vec_ok, a.sq_norms);
    return BSI_OK;
}

// Chunk mode: the fast kernel when its preconditions hold (10^dp small enough for the input type, scales
// wanted, every offset below 2^31, no outlier clipping), else the generic kernel.
template <typename T>
int launch_chunk(const T* x, const ChunkArgs& a) {
    int64_t widest = a.chunks * 256;
    if (a.ldx > widest) widest = a.ldx;
    if (a.q8 != nullptr && a.ld8 > widest) widest = a.ld8;
    const uint32_t mult_limit = sizeof(T) == 2 ? 1000u : 127u;
    const bool fast = a.dec_mult != 0u && a.dec_mult <= mult_limit && a.scales != nullptr && !(a.clip_k > 0.0f) &&
                      a.rows * widest < (1ll << 31) && (a.words != nullptr || a.q8 != nullptr);
    if (!fast) {
        int64_t blocks = (a.rows * a.chunks + 7) / 8;
        const int64_t cap = static_cast<int64_t>(sm_count()) * 64;
        blocks = blocks < cap ? blocks : cap;
        quantize_pack_chunk_generic_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, a.stream>>>(
            x, a.rows, a.D, a.ldx, a.dec_scale, a.dec_mult, a.bits, a.chunks, a.W, a.words, a.scales, a.shifts, a.q8,
            a.ld8, a.vec_ok, a.clip_k, a.sq_norms);
        return BSI_OK;
    }
    const bool dense = a.vec_ok && a.ldx == a.D && (a.D & 255) == 0 && (a.q8 == nullptr || a.ld8 == a.D);
    const bool w = a.words != nullptr, q = a.q8 != nullptr;
    if (dense) {
        if (w && q) return launch_chunk_fast<T, true, true, true>(x, a);
        if (q) return launch_chunk_fast<T, true, false, true>(x, a);
        return launch_chunk_fast<T, true, true, false>(x, a);
    }
    if (w && q) return launch_chunk_fast<T, false, true, true>(x, a);
    if (q) return launch_chunk_fast<T, false, false, true>(x, a);
    return launch_chunk_fast<T, false, true, false>(x, a);
}
}  // namespace
}  // namespace bsi

extern "C" int bsi_b200_quantize_pack(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx,
                                      int decimal_places, int bits, int chunk_mode,
                                      uint64_t* words, float* scales, int32_t* shifts,
                                      int8_t* q8, int64_t ld8, bsi_stream_t stream_) {
    return bsi_b200_quantize_pack_clip(x, dtype, rows, D, ldx, decimal_places, bits, chunk_mode, 0.0f, words, scales,
                                       shifts, q8, ld8, stream_);
}

extern "C" int bsi_b200_quantize_pack_clip(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx,
                                           int decimal_places, int bits, int chunk_mode, float clip_k,
                                           uint64_t* words, float* scales, int32_t* shifts,
                                           int8_t* q8, int64_t ld8, bsi_stream_t stream_) {
    return bsi_b200_quantize_pack_norms(x, dtype, rows, D, ldx, decimal_places, bits, chunk_mode, clip_k, words, scales,
                                        shifts, q8, ld8, nullptr, stream_);
}

extern "C" int bsi_b200_quantize_pack_norms(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx,
                                            int decimal_places, int bits, int chunk_mode, float clip_k,
                                            uint64_t* words, float* scales, int32_t* shifts,
                                            int8_t* q8, int64_t ld8, float* sq_norms, bsi_stream_t stream_) {
    using namespace bsi;
    if (sq_norms != nullptr && !chunk_mode)
        return fail(BSI_ERR_UNSUPPORTED, "quantize_pack: sums of squares are per (row, chunk): chunk mode only");
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

    if (chunk_mode) {
        ChunkArgs a{rows, D, ldx, ld8, chunks, W, dec_scale, dec_mult, bits, w, scales, shifts, q8, vec_ok, stream, clip_k,
                    sq_norms};
        int rc;
        if (dtype == BSI_DTYPE_F32) rc = launch_chunk<float>(static_cast<const float*>(x), a);
        else if (dtype == BSI_DTYPE_F16) rc = launch_chunk<__half>(static_cast<const __half*>(x), a);
        else rc = launch_chunk<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(x), a);
        if (rc != BSI_OK) return rc;
    } else {
        if (rows > 0x7fffffffll) return fail(BSI_ERR_UNSUPPORTED, "quantize_pack: too many rows for one launch");
#define BSI_LAUNCH_ROW(T)                                                                              \
    quantize_pack_row_kernel<T><<<static_cast<unsigned>(rows), 256, 0, stream>>>(                      \
        static_cast<const T*>(x), rows, D, ldx, dec_scale, dec_mult, bits, chunks, W, w, scales, shifts, q8, ld8, vec_ok, clip_k)
        if (dtype == BSI_DTYPE_F32) BSI_LAUNCH_ROW(float);
        else if (dtype == BSI_DTYPE_F16) BSI_LAUNCH_ROW(__half);
        else BSI_LAUNCH_ROW(__nv_bfloat16);
#undef BSI_LAUNCH_ROW
    }
    return check_launch("quantize_pack launch");
}

extern "C" int bsi_b200_quantize_pack_multi(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx,
                                            int decimal_places, int bits, int n_q8_dst, int8_t* const* q8_dst,
                                            int64_t ld8, int n_scale_dst, float* const* scale_dst, int64_t scale_ld,
                                            bsi_stream_t stream_) {
    using namespace bsi;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (rows < 0 || D < 0 || ldx < D) return fail(BSI_ERR_INVALID, "quantize_pack_multi: bad rows/D/ldx");
    if (bits < 2 || bits > 8) return fail(BSI_ERR_UNSUPPORTED, "quantize_pack_multi: bits must be in [2, 8]");
    if (dtype != BSI_DTYPE_F32 && dtype != BSI_DTYPE_F16 && dtype != BSI_DTYPE_BF16)
        return fail(BSI_ERR_INVALID, "quantize_pack_multi: unknown dtype");
    if (n_q8_dst < 1 || n_q8_dst > BSI_B200_MAX_PEERS || n_scale_dst < 1 || n_scale_dst > BSI_B200_MAX_PEERS ||
        q8_dst == nullptr || scale_dst == nullptr)
        return fail(BSI_ERR_INVALID, "quantize_pack_multi: bad destinations");
    if (rows == 0 || D == 0) return BSI_OK;
    if (x == nullptr) return fail(BSI_ERR_INVALID, "quantize_pack_multi: x is null");
    if ((D & 255) != 0) return fail(BSI_ERR_UNSUPPORTED, "quantize_pack_multi: D must be a multiple of 256");
    const int64_t chunks = D / 256;
    const int esz = dtype == BSI_DTYPE_F32 ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || ((ldx * esz) & 15) != 0)
        return fail(BSI_ERR_INVALID, "quantize_pack_multi: x needs 16-byte aligned rows");
    if (ld8 < D || (ld8 & 7) != 0 || scale_ld < chunks)
        return fail(BSI_ERR_INVALID, "quantize_pack_multi: ld8 >= D, ld8 % 8 == 0 and scale_ld >= D/256 are required");
    int64_t widest = ldx > ld8 ? ldx : ld8;
    if (rows * widest >= (1ll << 31)) return fail(BSI_ERR_UNSUPPORTED, "quantize_pack_multi: matrix too large for one launch");
    MultiDst dst = {};
    dst.n_q8 = n_q8_dst;
    dst.n_scales = n_scale_dst;
    for (int i = 0; i < n_q8_dst; ++i) {
        if (q8_dst[i] == nullptr || (reinterpret_cast<uintptr_t>(q8_dst[i]) & 7) != 0)
            return fail(BSI_ERR_INVALID, "quantize_pack_multi: q8 destinations must be non-null and 8-byte aligned");
        dst.q8[i] = q8_dst[i];
    }
    for (int i = 0; i < n_scale_dst; ++i) {
        if (scale_dst[i] == nullptr) return fail(BSI_ERR_INVALID, "quantize_pack_multi: null scale destination");
        dst.scales[i] = scale_dst[i];
    }
    if (int rc = require_sm100()) return rc;
    const double dec_scale = pow(10.0, static_cast<double>(decimal_places));
    uint32_t dec_mult = 0;
    if (decimal_places >= 0 && decimal_places <= 8) {
        dec_mult = 1;
        for (int i = 0; i < decimal_places; ++i) dec_mult *= 10u;
    }
#define BSI_LAUNCH_MULTI(T, LIMIT)                                                                          \
    do {                                                                                                    \
        const int64_t resident = resident_blocks(quantize_pack_multi_kernel<T>);                            \
        if (resident <= 0) return BSI_ERR_CUDA;                                                             \
        int64_t blocks = (rows * chunks + 7) / 8;                                                           \
        blocks = blocks < resident ? blocks : resident;                                                     \
        quantize_pack_multi_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(                   \
            static_cast<const T*>(x), static_cast<uint32_t>(rows * chunks), static_cast<uint32_t>(chunks),  \
            static_cast<uint32_t>(ldx), static_cast<uint32_t>(ld8), static_cast<uint32_t>(scale_ld), dec_scale, \
            dec_mult, LIMIT, bits, dst);                                                                    \
    } while (0)
    if (dtype == BSI_DTYPE_F32) BSI_LAUNCH_MULTI(float, 127u);
    else if (dtype == BSI_DTYPE_F16) BSI_LAUNCH_MULTI(__half, 1000u);
    else BSI_LAUNCH_MULTI(__nv_bfloat16, 1000u);
#undef BSI_LAUNCH_MULTI
    return check_launch("quantize_pack_multi launch");
}

extern "C" int bsi_b200_add_layernorm_pack(const void* x, const void* delta, const void* gamma, const void* beta,
                                           float eps, int dtype, int64_t rows, int64_t H, void* x_out,
                                           int decimal_places, int bits, int n_q8_dst, int8_t* const* q8_dst,
                                           int64_t ld8, int n_scale_dst, float* const* scale_dst, int64_t scale_ld,
                                           bsi_stream_t stream_) {
    using namespace bsi;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (rows < 0 || H <= 0) return fail(BSI_ERR_INVALID, "add_layernorm_pack: bad rows/H");
    if (dtype != BSI_DTYPE_F16 && dtype != BSI_DTYPE_BF16)
        return fail(BSI_ERR_UNSUPPORTED, "add_layernorm_pack: the layer type must be float16 or bfloat16");
    if ((H & 255) != 0 || H > 16384) return fail(BSI_ERR_UNSUPPORTED, "add_layernorm_pack: H must be a multiple of 256, at most 16384");
    if (bits < 2 || bits > 8) return fail(BSI_ERR_UNSUPPORTED, "add_layernorm_pack: bits must be in [2, 8]");
    if (rows == 0) return BSI_OK;
    if (rows > 0x7fffffffll) return fail(BSI_ERR_UNSUPPORTED, "add_layernorm_pack: too many rows");
    if (x == nullptr || gamma == nullptr || beta == nullptr || x_out == nullptr || q8_dst == nullptr || scale_dst == nullptr)
        return fail(BSI_ERR_INVALID, "add_layernorm_pack: null pointer");
    auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (misaligned(x) || misaligned(x_out) || misaligned(gamma) || misaligned(beta) || (delta != nullptr && misaligned(delta)))
        return fail(BSI_ERR_INVALID, "add_layernorm_pack: pointers must be 16-byte aligned");
    const int64_t chunks = H / 256;
    if (n_q8_dst < 1 || n_q8_dst > BSI_B200_MAX_PEERS || n_scale_dst < 1 || n_scale_dst > BSI_B200_MAX_PEERS ||
        ld8 < H || (ld8 & 7) != 0 || scale_ld < chunks)
        return fail(BSI_ERR_INVALID, "add_layernorm_pack: bad destinations (ld8 >= H, ld8 % 8 == 0, scale_ld >= H/256)");
    MultiDst dst = {};
    dst.n_q8 = n_q8_dst;
    dst.n_scales = n_scale_dst;
    for (int i = 0; i < n_q8_dst; ++i) {
        if (q8_dst[i] == nullptr || (reinterpret_cast<uintptr_t>(q8_dst[i]) & 7) != 0)
            return fail(BSI_ERR_INVALID, "add_layernorm_pack: q8 destinations must be non-null and 8-byte aligned");
        dst.q8[i] = q8_dst[i];
    }
    for (int i = 0; i < n_scale_dst; ++i) {
        if (scale_dst[i] == nullptr) return fail(BSI_ERR_INVALID, "add_layernorm_pack: null scale destination");
        dst.scales[i] = scale_dst[i];
    }
    if (int rc = require_sm100()) return rc;
    const double dec_scale = pow(10.0, static_cast<double>(decimal_places));
    uint32_t dec_mult = 0;
    if (decimal_places >= 0 && decimal_places <= 8) {
        dec_mult = 1;
        for (int i = 0; i < decimal_places; ++i) dec_mult *= 10u;
    }
    const int cpw = static_cast<int>((chunks + 7) / 8);   // chunks per warp, 8 warps
    int64_t blocks = rows;   // one block per row; the kernel's row loop only matters under a block cap
#define BSI_LAUNCH_ALP(T, CPW_)                                                                                   \
    add_layernorm_pack_kernel<T, CPW_><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(                       \
        static_cast<const T*>(x), static_cast<const T*>(delta), static_cast<const T*>(gamma),                    \
        static_cast<const T*>(beta), eps, static_cast<int>(rows), static_cast<int>(H), static_cast<int>(chunks), \
        static_cast<T*>(x_out), dec_scale, dec_mult, 1000u, bits, ld8, scale_ld, dst)
#define BSI_LAUNCH_ALP_T(T)                       \
    do {                                          \
        if (cpw <= 1) BSI_LAUNCH_ALP(T, 1);       \
        else if (cpw <= 2) BSI_LAUNCH_ALP(T, 2);  \
        else if (cpw <= 4) BSI_LAUNCH_ALP(T, 4);  \
        else BSI_LAUNCH_ALP(T, 8);                \
    } while (0)
    if (dtype == BSI_DTYPE_F16) BSI_LAUNCH_ALP_T(__half);
    else BSI_LAUNCH_ALP_T(__nv_bfloat16);
#undef BSI_LAUNCH_ALP_T
#undef BSI_LAUNCH_ALP
    return check_launch("add_layernorm_pack launch");
}

extern "C" int bsi_b200_decimal_absmax(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx, int decimal_places,
                                       uint64_t* row_absmax, int32_t* row_negative, bsi_stream_t stream_) {
    using namespace bsi;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (rows < 0 || D < 0 || ldx < D) return fail(BSI_ERR_INVALID, "decimal_absmax: bad rows / D / ldx");
    if (rows == 0) return BSI_OK;
    if (x == nullptr || row_absmax == nullptr || row_negative == nullptr) return fail(BSI_ERR_INVALID, "decimal_absmax: null pointer");
    if (dtype != BSI_DTYPE_F32 && dtype != BSI_DTYPE_F16 && dtype != BSI_DTYPE_BF16)
        return fail(BSI_ERR_INVALID, "decimal_absmax: unknown dtype");
    if (rows > 0x7fffffffll) return fail(BSI_ERR_UNSUPPORTED, "decimal_absmax: too many rows for one launch");
    if (int rc = require_sm100()) return rc;
    const double dec_scale = pow(10.0, static_cast<double>(decimal_places));
    const uint32_t dec_mult = (decimal_places >= 0 && decimal_places <= 8) ? static_cast<uint32_t>(dec_scale + 0.5) : 0u;
    const int64_t chunks = (D + 255) / 256;
    const int esz = dtype == BSI_DTYPE_F32 ? 4 : 2;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0 && ((ldx * esz) & 15) == 0) ? 1 : 0;
    const unsigned g = static_cast<unsigned>(rows);
#define BSI_ABSMAX(T) decimal_absmax_kernel<T><<<g, 256, 0, stream>>>(static_cast<const T*>(x), rows, D, ldx, dec_scale, \
                                                                      dec_mult, chunks, vec_ok, reinterpret_cast<u64*>(row_absmax), row_negative)
    if (dtype == BSI_DTYPE_F32) BSI_ABSMAX(float);
    else if (dtype == BSI_DTYPE_F16) BSI_ABSMAX(__half);
    else BSI_ABSMAX(__nv_bfloat16);
#undef BSI_ABSMAX
    return check_launch("decimal_absmax launch");
}

extern "C" int bsi_b200_pack_plain(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx, int decimal_places,
                                   int slices, uint64_t* words, int8_t* lo8, int8_t* hi8, int64_t ld8, bsi_stream_t stream_) {
    using namespace bsi;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (rows < 0 || D < 0 || ldx < D) return fail(BSI_ERR_INVALID, "pack_plain: bad rows / D / ldx");
    if (slices < 1 || slices > 64) return fail(BSI_ERR_INVALID, "pack_plain: slices must be in [1, 64]");
    if (rows == 0 || D == 0) return BSI_OK;
    if (x == nullptr) return fail(BSI_ERR_INVALID, "pack_plain: null pointer");
    if (dtype != BSI_DTYPE_F32 && dtype != BSI_DTYPE_F16 && dtype != BSI_DTYPE_BF16)
        return fail(BSI_ERR_INVALID, "pack_plain: unknown dtype");
    const int64_t chunks = (D + 255) / 256;
    if (lo8 == nullptr && hi8 != nullptr) return fail(BSI_ERR_INVALID, "pack_plain: hi8 without lo8");
    if (lo8 != nullptr && (ld8 < chunks * 256 || (ld8 & 15) != 0 || (reinterpret_cast<uintptr_t>(lo8) & 15) != 0 ||
                           (reinterpret_cast<uintptr_t>(hi8) & 15) != 0))
        return fail(BSI_ERR_INVALID, "pack_plain: int8 images need ld8 >= 256*ceil(D/256), ld8 % 16 == 0, 16-byte bases");
    if (int rc = require_sm100()) return rc;
    const double dec_scale = pow(10.0, static_cast<double>(decimal_places));
    const uint32_t dec_mult = (decimal_places >= 0 && decimal_places <= 8) ? static_cast<uint32_t>(dec_scale + 0.5) : 0u;
    const int64_t W = (D + 63) / 64;
    const int esz = dtype == BSI_DTYPE_F32 ? 4 : 2;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0 && ((ldx * esz) & 15) == 0) ? 1 : 0;
    const int64_t blocks = (rows * chunks + 7) / 8;
    if (blocks > 0x7fffffffll) return fail(BSI_ERR_UNSUPPORTED, "pack_plain: too many rows for one launch");
    const unsigned g = static_cast<unsigned>(blocks);
#define BSI_PLAIN(T) pack_plain_kernel<T><<<g, 256, 0, stream>>>(static_cast<const T*>(x), rows, D, ldx, dec_scale, dec_mult, \
                                                                  slices, chunks, W, vec_ok, reinterpret_cast<u64*>(words), lo8, hi8, ld8)
    if (dtype == BSI_DTYPE_F32) BSI_PLAIN(float);
    else if (dtype == BSI_DTYPE_F16) BSI_PLAIN(__half);
    else BSI_PLAIN(__nv_bfloat16);
#undef BSI_PLAIN
    return check_launch("pack_plain launch");
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
