// Device helpers shared by the pack kernels and the re-quantising linear epilogue: the exact
// float32 form of the reference's two roundings and the byte-wise sign / clamp.
#pragma once

#include <stdint.h>

namespace bsi {

// prmt.b32 with the full 4-bit selectors (values 8..15 replicate the sign bit of the chosen byte over the
// result byte; the __byte_perm intrinsic only honours 3 bits per selector).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// u0..u3 carry the unsigned quantised magnitudes of four elements in their low bytes (0 .. 2^(bits-1)),
// s0..s3 the sign bits (bit 31, e.g. the float bit patterns). Clamps positives to 2^(bits-1)-1, negates
// the negatives and returns the four two's-complement bytes.
__device__ __forceinline__ uint32_t sign_clamp4(uint32_t u0, uint32_t u1, uint32_t u2, uint32_t u3, uint32_t s0,
                                                uint32_t s1, uint32_t s2, uint32_t s3, int bits) {
    const uint32_t top = 0x01010101u << (bits - 1);
    uint32_t w = __byte_perm(__byte_perm(u0, u1, 0x0040), __byte_perm(u2, u3, 0x0040), 0x5410);   // the low bytes
    const uint32_t m = prmt(prmt(s0, s1, 0x00fbu), prmt(s2, s3, 0x00fbu), 0x5410u);               // 0xff per negative
    // positive 2^(bits-1) -> 2^(bits-1) - 1 (the byte is exactly `top` there, so the borrow stays inside it)
    const uint32_t over = w & ~m & top;
    w -= over >> (bits - 1);
    // negate the bytes under m: (~b + 1) per byte, the carry kept inside the byte by adding in 7 bits
    const uint32_t x = w ^ m;
    const uint32_t t = (x & 0x7f7f7f7fu) + (m & 0x01010101u);
    return t ^ (x & 0x80808080u);
}

// Shift of a chunk whose largest |x * 10^dp| is ymax (exact in float32, below 2^23): the reference's
// bits(max|v|) - (b - 1), clamped at 0, with max|v| = half_away(ymax).
__device__ __forceinline__ int fast_shift(float ymax, int bits) {
    const uint32_t mx = __float2uint_rz(ymax + 0.5f);
    const int shift = (32 - __clz(static_cast<int>(mx))) - (bits - 1);
    return shift < 0 ? 0 : shift;
}

// Constants of the second rounding for a given shift: u = fma(r1, inv, c) with r1 = 2^23 + |v|.
__device__ __forceinline__ void fast_round_consts(int shift, float& inv, float& c) {
    inv = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);   // 2^-shift
    c = (shift > 0 ? 0.5f : 0.0f) - 8388608.0f * inv;
}

// Quantised magnitude of x (low mantissa byte of the result) for 16-bit-precision x with |x * mult| < 2^23:
// |v| = floor(|x| * mult + 0.5) and then floor(|v| * 2^-shift + 0.5 * [shift > 0]), each as an exact
// float32 sum whose round-toward-zero addition of 2^23 leaves the integer in the mantissa.
__device__ __forceinline__ uint32_t fast_magnitude(float x, float mult, float inv, float c) {
    const float r1 = __fadd_rz(fmaf(fabsf(x), mult, 0.5f), 8388608.0f);
    return __float_as_uint(__fadd_rz(fmaf(r1, inv, c), 8388608.0f));
}

}  // namespace bsi
