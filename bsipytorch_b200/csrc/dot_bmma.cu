// Dot core directly on the slice words with the legacy binary tensor-core path
// (mma.sync m16n8k256 b1 AND+POPC). This is the second engine the library evaluates next to the
// tcgen05 int8 engine; it needs Sa*Sb binary MMAs per 256 of depth where the int8 engine needs
// one contraction, and it is what a caller that only holds bit slices can run without building
// an int8 image.
//
// Tile: 64 query rows x 64 key rows per CTA, 8 warps as 4 (query) x 2 (key); a warp owns
// 16 x 32 outputs = four m16n8 sub-tiles. Per 256-bit chunk the slices of the tile are staged in
// shared memory with cp.async (double buffered), 12 words per 8-word row so that the fragment
// loads of the 8 row groups fall in distinct banks.
//
// Slice pairs with the same weight 2^(i+j) and the same sign share one MMA accumulator chain, so
// the shift-and-add work is per (shift, sign) group, not per pair.
#include "common.cuh"

namespace bsi {
namespace {

typedef unsigned long long u64;

constexpr int kTQ = 64;
constexpr int kTR = 64;
constexpr int kRowWords = 12;  // 8 data words + 4 pad

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void bmma(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.and.popc "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Stages one chunk: rows beyond the matrix edge are zero-filled.
__device__ __forceinline__ void stage_chunk(uint32_t* dst, const u64* __restrict__ src, int slices, int64_t W,
                                            int row0, int rows_total, int tile_rows, int64_t chunk) {
    // Each (slice, row) contributes 32 bytes = two 16-byte copies.
    const int items = slices * tile_rows * 2;
    for (int idx = threadIdx.x; idx < items; idx += blockDim.x) {
        const int part = idx & 1;
        const int row = (idx >> 1) % tile_rows;
        const int s = (idx >> 1) / tile_rows;
        uint32_t* d = dst + (s * tile_rows + row) * kRowWords + part * 4;
        const int g = row0 + row;
        if (g < rows_total) {
            cp_async16(d, src + (static_cast<int64_t>(g) * slices + s) * W + chunk * 4 + part * 2);
        } else {
            d[0] = 0u; d[1] = 0u; d[2] = 0u; d[3] = 0u;
        }
    }
}

template <int SA, int SB>
__global__ void __launch_bounds__(256) dot_words_bmma_kernel(
    const u64* __restrict__ A, const float* __restrict__ qs, int64_t qs_stride, int64_t W,
    const u64* __restrict__ B, const float* __restrict__ Bw, int R, int Q, float scale_inv,
    int64_t ldo, float* __restrict__ out, int32_t* __restrict__ dbg_iacc) {
    extern __shared__ __align__(16) uint32_t smem_words[];
    constexpr int kAWords = SA * kTQ * kRowWords;
    constexpr int kBWords = SB * kTR * kRowWords;
    uint32_t* As[2] = {smem_words, smem_words + kAWords + kBWords};
    uint32_t* Bs[2] = {smem_words + kAWords, smem_words + 2 * kAWords + kBWords};

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int wq = warp >> 1;  // 0..3: which 16 query rows
    const int wr = warp & 1;   // 0..1: which 32 key rows
    const int g = lane >> 2;
    const int t = lane & 3;
    const int q0 = blockIdx.y * kTQ;
    const int r0 = blockIdx.x * kTR;
    const int chunks = static_cast<int>(W / 4);

    const int m0 = wq * 16 + g;
    const int m1 = m0 + 8;
    const int gq0 = q0 + m0;
    const int gq1 = q0 + m1;

    float acc[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.0f;

    stage_chunk(As[0], A, SA, W, q0, Q, kTQ, 0);
    stage_chunk(Bs[0], B, SB, W, r0, R, kTR, 0);
    cp_async_commit();

    for (int c = 0; c < chunks; ++c) {
        const int cur = c & 1;
        cp_async_wait_all();
        __syncthreads();
        if (c + 1 < chunks) {
            stage_chunk(As[cur ^ 1], A, SA, W, q0, Q, kTQ, c + 1);
            stage_chunk(Bs[cur ^ 1], B, SB, W, r0, R, kTR, c + 1);
            cp_async_commit();
        }
        const uint32_t* a_s = As[cur];
        const uint32_t* b_s = Bs[cur];

        uint32_t afrag[SA][4];
#pragma unroll
        for (int i = 0; i < SA; ++i) {
            const uint32_t* ai = a_s + i * kTQ * kRowWords;
            afrag[i][0] = ai[m0 * kRowWords + t];
            afrag[i][1] = ai[m1 * kRowWords + t];
            afrag[i][2] = ai[m0 * kRowWords + t + 4];
            afrag[i][3] = ai[m1 * kRowWords + t + 4];
        }
        const float qs0 = gq0 < Q ? (qs_stride ? qs[static_cast<int64_t>(gq0) * qs_stride + c] : qs[gq0]) : 0.0f;
        const float qs1 = gq1 < Q ? (qs_stride ? qs[static_cast<int64_t>(gq1) * qs_stride + c] : qs[gq1]) : 0.0f;

#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const int col = wr * 32 + n * 8 + g;  // key row within the tile feeding this lane's B fragment
            uint32_t b0[SB], b1[SB];
#pragma unroll
            for (int j = 0; j < SB; ++j) {
                const uint32_t* bj = b_s + (j * kTR + col) * kRowWords;
                b0[j] = bj[t];
                b1[j] = bj[t + 4];
            }
            int I[4] = {0, 0, 0, 0};
            // Positive pairs: both or neither of (i == SA-1), (j == SB-1); grouped by s = i + j.
#pragma unroll
            for (int s = 0; s <= SA + SB - 2; ++s) {
                int pos[4] = {0, 0, 0, 0};
                int neg[4] = {0, 0, 0, 0};
                bool any_pos = false, any_neg = false;
#pragma unroll
                for (int i = 0; i < SA; ++i) {
                    const int j = s - i;
                    if (j < 0 || j >= SB) continue;
                    const bool negative = (i == SA - 1) != (j == SB - 1);
                    if (negative) {
                        bmma(neg, afrag[i], b0[j], b1[j]);
                        any_neg = true;
                    } else {
                        bmma(pos, afrag[i], b0[j], b1[j]);
                        any_pos = true;
                    }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (any_pos) I[e] += pos[e] << s;
                    if (any_neg) I[e] -= neg[e] << s;
                }
            }
            acc[n][0] = __fmaf_rn(static_cast<float>(I[0]), qs0, acc[n][0]);
            acc[n][1] = __fmaf_rn(static_cast<float>(I[1]), qs0, acc[n][1]);
            acc[n][2] = __fmaf_rn(static_cast<float>(I[2]), qs1, acc[n][2]);
            acc[n][3] = __fmaf_rn(static_cast<float>(I[3]), qs1, acc[n][3]);
            if (dbg_iacc != nullptr) {
                const int rc = r0 + wr * 32 + n * 8 + t * 2;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int q = (e < 2) ? gq0 : gq1;
                    const int r = rc + (e & 1);
                    if (q < Q && r < R) dbg_iacc[(static_cast<int64_t>(q) * R + r) * chunks + c] = I[e];
                }
            }
        }
    }

#pragma unroll
    for (int n = 0; n < 4; ++n) {
        const int rc = r0 + wr * 32 + n * 8 + t * 2;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int q = (e < 2) ? gq0 : gq1;
            const int r = rc + (e & 1);
            if (q < Q && r < R) {
                const float bw0 = Bw[static_cast<int64_t>(r) * SB];
                out[static_cast<int64_t>(q) * ldo + r] = (acc[n][e] * bw0) * scale_inv;
            }
        }
    }
}

template <int SA, int SB>
int launch(const u64* A, const float* qs, int64_t qs_stride, int64_t W, const u64* B, const float* Bw,
           int64_t R, int64_t Q, float scale_inv, int64_t ldo, float* out, int32_t* dbg, cudaStream_t stream) {
    constexpr int smem = 2 * (SA * kTQ + SB * kTR) * kRowWords * 4;
    static bool attr_set[64] = {false};
    int dev = 0;
    BSI_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        BSI_CUDA_TRY(cudaFuncSetAttribute(dot_words_bmma_kernel<SA, SB>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    dim3 grid(static_cast<unsigned>((R + kTR - 1) / kTR), static_cast<unsigned>((Q + kTQ - 1) / kTQ), 1);
    if (grid.y > 65535u) return fail(BSI_ERR_UNSUPPORTED, "dot_words: too many query rows");
    dot_words_bmma_kernel<SA, SB><<<grid, 256, smem, stream>>>(A, qs, qs_stride, W, B, Bw, static_cast<int>(R),
                                                                 static_cast<int>(Q), scale_inv, ldo, out, dbg);
    return check_launch("dot_words bmma launch");
}

}  // namespace

int dot_words_bmma(const uint64_t* A_, const float* qs, int64_t qs_stride, int Sa, int64_t W,
                   const uint64_t* B_, const float* Bw, int Sb, int64_t R, int64_t Q, float scale_inv,
                   int64_t ldo, float* out, int32_t* dbg, cudaStream_t stream) {
    const u64* A = reinterpret_cast<const u64*>(A_);
    const u64* B = reinterpret_cast<const u64*>(B_);
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
        return fail(BSI_ERR_INVALID, "dot_words: slice words must be 16-byte aligned");
    if (Q > 0x7fffff00ll || R > 0x7fffff00ll) return fail(BSI_ERR_UNSUPPORTED, "dot_words: Q or R too large");
#define BSI_CASE(SA_, SB_) \
    if (Sa == SA_ && Sb == SB_) return launch<SA_, SB_>(A, qs, qs_stride, W, B, Bw, R, Q, scale_inv, ldo, out, dbg, stream)
    BSI_CASE(7, 6);
    BSI_CASE(8, 8);
    BSI_CASE(7, 7);
    BSI_CASE(6, 6);
    BSI_CASE(8, 6);
    BSI_CASE(4, 4);
#undef BSI_CASE
    return fail(BSI_ERR_UNSUPPORTED, "dot_words: slice counts (Sa, Sb) must be one of (7,6) (8,8) (7,7) (6,6) (8,6) (4,4)");
}

}  // namespace bsi
