// Dot entry points and the CUDA-core (dp4a) cross-check engine.
//
// All engines evaluate the same recurrence, in the reference's order
// (bsi_cuda_kernels_dot.cuh:1519-1526, 1539):
//     acc_0 = 0;  acc_{c+1} = fmaf(float(I_c), qs[q][c], acc_c);  out = (acc * bw0[r]) * scale_inv
// bw0[r] is a power of two, so applying it after the loop leaves every bit unchanged.
#include "common.cuh"

namespace bsi {

int dot_i8_tcgen05(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride, const int8_t* k8,
                   int64_t ldk, const float* bw0, int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                   float* out, int64_t ldo, int32_t* dbg_iacc, int force_bn, cudaStream_t stream);

int dot_i8_pair(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride, const int8_t* k8, int64_t ldk,
                const float* bw0, const float* bias, int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                void* out, int64_t ldo, int y_dtype, int32_t* dbg_iacc, int force_bn, int relu,
                const ScatterDst* scatter, const RequantDst* requant, cudaStream_t stream);

int dot_words_bmma(const uint64_t* A, const float* qs, int64_t qs_stride, int Sa, int64_t W,
                   const uint64_t* B, const float* Bw, int Sb, int64_t R, int64_t Q, float scale_inv,
                   int64_t ldo, float* out, int32_t* dbg_iacc, cudaStream_t stream);

namespace {

// 64 x 64 outputs per block, 4 x 4 per thread, one 256-deep chunk staged in smem per step.
constexpr int kT = 64;
constexpr int kPad = 65;  // row stride in 32-bit words; odd, so a column walk hits 32 banks

__global__ void __launch_bounds__(256) dot_i8_simt_kernel(
    const int8_t* __restrict__ a8, int64_t lda, const float* __restrict__ qs, int64_t qs_stride,
    const int8_t* __restrict__ k8, int64_t ldk, const float* __restrict__ bw0, int Q, int R, int chunks,
    float scale_inv, float* __restrict__ out, int64_t ldo, int32_t* __restrict__ dbg_iacc) {
    __shared__ int As[kT * kPad];
    __shared__ int Bs[kT * kPad];
    const int tx = threadIdx.x & 15;
    const int ty = threadIdx.x >> 4;
    const int q0 = blockIdx.y * kT;
    const int r0 = blockIdx.x * kT;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int c = 0; c < chunks; ++c) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < kT * 64; idx += 256) {
            const int row = idx >> 6;
            const int k4 = idx & 63;
            const int q = q0 + row;
            const int r = r0 + row;
            As[row * kPad + k4] =
                q < Q ? *reinterpret_cast<const int*>(a8 + static_cast<int64_t>(q) * lda + c * 256 + k4 * 4) : 0;
            Bs[row * kPad + k4] =
                r < R ? *reinterpret_cast<const int*>(k8 + static_cast<int64_t>(r) * ldk + c * 256 + k4 * 4) : 0;
        }
        __syncthreads();
        int I[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) I[i][j] = 0;
#pragma unroll 4
        for (int k4 = 0; k4 < 64; ++k4) {
            int a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[(ty + 16 * i) * kPad + k4];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[(tx + 16 * j) * kPad + k4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) I[i][j] = __dp4a(a[i], b[j], I[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int q = q0 + ty + 16 * i;
            if (q >= Q) continue;
            const float qscale = qs_stride ? qs[static_cast<int64_t>(q) * qs_stride + c] : qs[q];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[i][j] = __fmaf_rn(static_cast<float>(I[i][j]), qscale, acc[i][j]);
                const int r = r0 + tx + 16 * j;
                if (dbg_iacc != nullptr && r < R)
                    dbg_iacc[(static_cast<int64_t>(q) * R + r) * chunks + c] = I[i][j];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int q = q0 + ty + 16 * i;
        if (q >= Q) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = r0 + tx + 16 * j;
            if (r < R) out[static_cast<int64_t>(q) * ldo + r] = (acc[i][j] * bw0[r]) * scale_inv;
        }
    }
}

}  // namespace
}  // namespace bsi

extern "C" int bsi_b200_dot_i8(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride,
                               const int8_t* k8, int64_t ldk, const float* bw0,
                               int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                               float* out, int64_t ldo, int32_t* dbg_iacc, int engine,
                               bsi_stream_t stream_) {
    using namespace bsi;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (Q < 0 || R < 0 || chunks < 0) return fail(BSI_ERR_INVALID, "dot_i8: negative size");
    if (Q == 0 || R == 0) return BSI_OK;
    if (a8 == nullptr || k8 == nullptr || qs == nullptr || bw0 == nullptr || out == nullptr)
        return fail(BSI_ERR_INVALID, "dot_i8: null pointer");
    if (chunks == 0) return fail(BSI_ERR_INVALID, "dot_i8: chunks must be positive");
    if (lda < chunks * 256 || ldk < chunks * 256 || (lda & 15) || (ldk & 15) ||
        (reinterpret_cast<uintptr_t>(a8) & 15) || (reinterpret_cast<uintptr_t>(k8) & 15))
        return fail(BSI_ERR_INVALID, "dot_i8: a8/k8 need 16-byte aligned rows of at least 256*chunks bytes");
    if (ldo < R) return fail(BSI_ERR_INVALID, "dot_i8: ldo < R");
    if (qs_stride != 0 && qs_stride < chunks) return fail(BSI_ERR_INVALID, "dot_i8: qs_stride < chunks");
    if (int rc = require_sm100()) return rc;

    int force_bn = 0;
    if (engine >= 1000) {  // 1000 + tile width: test hook to pin the tcgen05 tile shape
        force_bn = engine - 1000;
        engine = BSI_ENGINE_TCGEN05;
    }
    if (engine == BSI_ENGINE_AUTO) engine = BSI_ENGINE_TCGEN05;
    if (engine == BSI_ENGINE_TCGEN05) {
        return dot_i8_tcgen05(a8, lda, qs, qs_stride, k8, ldk, bw0, Q, R, chunks, scale_inv, out, ldo,
                              dbg_iacc, force_bn, stream);
    }
    if (engine == BSI_ENGINE_SIMT) {
        if (Q > 0x7fffff00ll || R > 0x7fffff00ll || chunks > 0x400000)
            return fail(BSI_ERR_UNSUPPORTED, "dot_i8: Q, R or chunks too large");
        dim3 grid(static_cast<unsigned>((R + kT - 1) / kT), static_cast<unsigned>((Q + kT - 1) / kT), 1);
        if (grid.y > 65535u) return fail(BSI_ERR_UNSUPPORTED, "dot_i8 simt: too many query rows");
        dot_i8_simt_kernel<<<grid, 256, 0, stream>>>(a8, lda, qs, qs_stride, k8, ldk, bw0,
                                                     static_cast<int>(Q), static_cast<int>(R),
                                                     static_cast<int>(chunks), scale_inv, out, ldo, dbg_iacc);
        return check_launch("dot_i8 simt launch");
    }
    return fail(BSI_ERR_INVALID, "dot_i8: engine must be AUTO, TCGEN05 or SIMT (BMMA takes slice words: bsi_b200_dot_words)");
}

extern "C" int bsi_b200_linear_i8_act(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride,
                                  const int8_t* k8, int64_t ldk, const float* bw0, const float* bias,
                                  int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                                  void* y, int64_t ldy, int y_dtype, int activation, bsi_stream_t stream_) {
    using namespace bsi;
    if (Q < 0 || R < 0 || chunks < 0) return fail(BSI_ERR_INVALID, "linear_i8: negative size");
    if (Q == 0 || R == 0) return BSI_OK;
    if (a8 == nullptr || k8 == nullptr || qs == nullptr || bw0 == nullptr || y == nullptr)
        return fail(BSI_ERR_INVALID, "linear_i8: null pointer");
    if (chunks == 0) return fail(BSI_ERR_INVALID, "linear_i8: chunks must be positive");
    if (lda < chunks * 256 || ldk < chunks * 256 || (lda & 15) || (ldk & 15) ||
        (reinterpret_cast<uintptr_t>(a8) & 15) || (reinterpret_cast<uintptr_t>(k8) & 15))
        return fail(BSI_ERR_INVALID, "linear_i8: a8/k8 need 16-byte aligned rows of at least 256*chunks bytes");
    if (ldy < R) return fail(BSI_ERR_INVALID, "linear_i8: ldy < R");
    if (qs_stride != 0 && qs_stride < chunks) return fail(BSI_ERR_INVALID, "linear_i8: qs_stride < chunks");
    if (activation != BSI_ACT_NONE && activation != BSI_ACT_RELU)
        return fail(BSI_ERR_INVALID, "linear_i8: unknown activation");
    if (y_dtype != BSI_DTYPE_F32 && y_dtype != BSI_DTYPE_F16 && y_dtype != BSI_DTYPE_BF16)
        return fail(BSI_ERR_INVALID, "linear_i8: unknown y_dtype");
    if (int rc = require_sm100()) return rc;
    return dot_i8_pair(a8, lda, qs, qs_stride, k8, ldk, bw0, bias, Q, R, chunks, scale_inv, y, ldy, y_dtype,
                       nullptr, 0, activation == BSI_ACT_RELU ? 1 : 0, nullptr, nullptr, static_cast<cudaStream_t>(stream_));
}

extern "C" int bsi_b200_linear_i8_scatter(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride,
                                          const int8_t* k8, int64_t ldk, const float* bw0, const float* bias,
                                          int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                                          int n_dst, void* const* y_dst, int64_t rows_per_dst, int64_t ldy,
                                          int y_dtype, int activation, bsi_stream_t stream_) {
    using namespace bsi;
    if (Q < 0 || R < 0 || chunks < 0) return fail(BSI_ERR_INVALID, "linear_i8_scatter: negative size");
    if (Q == 0 || R == 0) return BSI_OK;
    if (a8 == nullptr || k8 == nullptr || qs == nullptr || bw0 == nullptr || y_dst == nullptr)
        return fail(BSI_ERR_INVALID, "linear_i8_scatter: null pointer");
    if (chunks == 0) return fail(BSI_ERR_INVALID, "linear_i8_scatter: chunks must be positive");
    if (lda < chunks * 256 || ldk < chunks * 256 || (lda & 15) || (ldk & 15) ||
        (reinterpret_cast<uintptr_t>(a8) & 15) || (reinterpret_cast<uintptr_t>(k8) & 15))
        return fail(BSI_ERR_INVALID, "linear_i8_scatter: a8/k8 need 16-byte aligned rows of at least 256*chunks bytes");
    if (ldy < R) return fail(BSI_ERR_INVALID, "linear_i8_scatter: ldy < R");
    if (qs_stride != 0 && qs_stride < chunks) return fail(BSI_ERR_INVALID, "linear_i8_scatter: qs_stride < chunks");
    if (activation != BSI_ACT_NONE && activation != BSI_ACT_RELU)
        return fail(BSI_ERR_INVALID, "linear_i8_scatter: unknown activation");
    if (y_dtype != BSI_DTYPE_F32 && y_dtype != BSI_DTYPE_F16 && y_dtype != BSI_DTYPE_BF16)
        return fail(BSI_ERR_INVALID, "linear_i8_scatter: unknown y_dtype");
    if (n_dst < 1 || n_dst > BSI_B200_MAX_PEERS || rows_per_dst <= 0 || rows_per_dst > 0x7fffffe0ll)
        return fail(BSI_ERR_INVALID, "linear_i8_scatter: bad n_dst / rows_per_dst");
    ScatterDst sc = {};
    sc.n = n_dst;
    sc.rows_per_dst = static_cast<int>(rows_per_dst);
    // the kernel chooses 16-byte or scalar stores from destination 0: all must be aligned alike
    const uintptr_t align0 = reinterpret_cast<uintptr_t>(y_dst[0]) & 15;
    for (int i = 0; i < n_dst; ++i) {
        if (y_dst[i] == nullptr) return fail(BSI_ERR_INVALID, "linear_i8_scatter: null destination");
        if ((reinterpret_cast<uintptr_t>(y_dst[i]) & 15) != align0)
            return fail(BSI_ERR_INVALID, "linear_i8_scatter: destinations must share their 16-byte alignment");
        sc.y[i] = y_dst[i];
    }
    if (int rc = require_sm100()) return rc;
    return dot_i8_pair(a8, lda, qs, qs_stride, k8, ldk, bw0, bias, Q, R, chunks, scale_inv, nullptr, ldy, y_dtype,
                       nullptr, 0, activation == BSI_ACT_RELU ? 1 : 0, &sc, nullptr, static_cast<cudaStream_t>(stream_));
}

extern "C" int bsi_b200_linear_i8_requant(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride,
                                          const int8_t* k8, int64_t ldk, const float* bw0, const float* bias,
                                          int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                                          int layer_dtype, int activation, int decimal_places, int bits,
                                          int n_dst, int8_t* const* q8_dst, int64_t ld8,
                                          float* const* scale_dst, int64_t scale_ld, bsi_stream_t stream_) {
    using namespace bsi;
    if (Q < 0 || R < 0 || chunks < 0) return fail(BSI_ERR_INVALID, "linear_i8_requant: negative size");
    if (Q == 0 || R == 0) return BSI_OK;
    if (a8 == nullptr || k8 == nullptr || qs == nullptr || bw0 == nullptr || q8_dst == nullptr || scale_dst == nullptr)
        return fail(BSI_ERR_INVALID, "linear_i8_requant: null pointer");
    if (chunks == 0) return fail(BSI_ERR_INVALID, "linear_i8_requant: chunks must be positive");
    if (lda < chunks * 256 || ldk < chunks * 256 || (lda & 15) || (ldk & 15) ||
        (reinterpret_cast<uintptr_t>(a8) & 15) || (reinterpret_cast<uintptr_t>(k8) & 15))
        return fail(BSI_ERR_INVALID, "linear_i8_requant: a8/k8 need 16-byte aligned rows of at least 256*chunks bytes");
    if (qs_stride != 0 && qs_stride < chunks) return fail(BSI_ERR_INVALID, "linear_i8_requant: qs_stride < chunks");
    if (activation != BSI_ACT_NONE && activation != BSI_ACT_RELU)
        return fail(BSI_ERR_INVALID, "linear_i8_requant: unknown activation");
    if (layer_dtype != BSI_DTYPE_F16 && layer_dtype != BSI_DTYPE_BF16)
        return fail(BSI_ERR_UNSUPPORTED, "linear_i8_requant: the layer type must be float16 or bfloat16");
    if ((R & 255) != 0) return fail(BSI_ERR_UNSUPPORTED, "linear_i8_requant: R must be a multiple of 256");
    if (bits < 2 || bits > 8) return fail(BSI_ERR_UNSUPPORTED, "linear_i8_requant: bits must be in [2, 8]");
    if (decimal_places < 0 || decimal_places > 3)
        return fail(BSI_ERR_UNSUPPORTED, "linear_i8_requant: decimal_places must be in [0, 3]");
    if (n_dst < 1 || n_dst > BSI_B200_MAX_PEERS || ld8 < R || (ld8 & 15) != 0 || scale_ld < R / 256)
        return fail(BSI_ERR_INVALID, "linear_i8_requant: bad destinations (ld8 >= R, ld8 % 16 == 0, scale_ld >= R/256)");
    RequantDst rq = {};
    rq.n = n_dst;
    rq.bits = bits;
    rq.mult = 1.0f;
    for (int i = 0; i < decimal_places; ++i) rq.mult *= 10.0f;
    rq.ld8 = ld8;
    rq.scale_ld = scale_ld;
    for (int i = 0; i < n_dst; ++i) {
        if (q8_dst[i] == nullptr || scale_dst[i] == nullptr || (reinterpret_cast<uintptr_t>(q8_dst[i]) & 15) != 0)
            return fail(BSI_ERR_INVALID, "linear_i8_requant: destinations must be non-null, q8 16-byte aligned");
        rq.q8[i] = q8_dst[i];
        rq.scales[i] = scale_dst[i];
    }
    if (int rc = require_sm100()) return rc;
    return dot_i8_pair(a8, lda, qs, qs_stride, k8, ldk, bw0, bias, Q, R, chunks, scale_inv, q8_dst[0], R, layer_dtype,
                       nullptr, 0, activation == BSI_ACT_RELU ? 1 : 0, nullptr, &rq, static_cast<cudaStream_t>(stream_));
}

extern "C" int bsi_b200_linear_i8(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride,
                                  const int8_t* k8, int64_t ldk, const float* bw0, const float* bias,
                                  int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                                  void* y, int64_t ldy, int y_dtype, bsi_stream_t stream_) {
    return bsi_b200_linear_i8_act(a8, lda, qs, qs_stride, k8, ldk, bw0, bias, Q, R, chunks, scale_inv, y, ldy, y_dtype,
                                  BSI_ACT_NONE, stream_);
}

extern "C" int bsi_b200_dot_words(const uint64_t* A, const float* qs, int64_t qs_stride, int Sa, int64_t W,
                                  const uint64_t* B, const float* Bw, int Sb, int64_t R, int64_t Q,
                                  float scale_inv, int64_t ldo, float* out, int32_t* dbg_iacc,
                                  bsi_stream_t stream_) {
    using namespace bsi;
    if (Q < 0 || R < 0 || W <= 0) return fail(BSI_ERR_INVALID, "dot_words: bad size");
    if (Q == 0 || R == 0) return BSI_OK;
    if (A == nullptr || B == nullptr || qs == nullptr || Bw == nullptr || out == nullptr)
        return fail(BSI_ERR_INVALID, "dot_words: null pointer");
    if (W % 4 != 0) return fail(BSI_ERR_UNSUPPORTED, "dot_words: W must be a multiple of 4 (256-bit chunks)");
    if (Sa < 2 || Sa > 8 || Sb < 2 || Sb > 8) return fail(BSI_ERR_UNSUPPORTED, "dot_words: slices must be in [2, 8]");
    if (ldo < R) return fail(BSI_ERR_INVALID, "dot_words: ldo < R");
    if (qs_stride != 0 && qs_stride < W / 4) return fail(BSI_ERR_INVALID, "dot_words: qs_stride < chunks");
    if (int rc = require_sm100()) return rc;
    return dot_words_bmma(A, qs, qs_stride, Sa, W, B, Bw, Sb, R, Q, scale_inv, ldo, out, dbg_iacc,
                          static_cast<cudaStream_t>(stream_));
}
