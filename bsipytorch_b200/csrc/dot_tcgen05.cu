// Dot core on the 5th-generation tensor cores.
//
// The 7 query slices and 6 key slices are recombined into signed 8-bit operands, so that the
// per-chunk integer accumulator
//     I[q][r][c] = sum_{d in chunk c} a8[q][d] * k8[r][d]
// (identical to sum_{i,j} +-2^(i+j) popc(A_i & B_j), the reference's weighted popcount,
// bsi_cuda_kernels_dot.cuh:1447-1517) is ONE int8 contraction of depth 256 instead of 42
// binary MMAs. Per output tile of 128 query rows x BN key rows:
//
//   warp 0   TMA producer: per 128-byte k-block, one box of A (128 x 128 B) and one of B
//            (BN x 128 B), 128-byte swizzled, into a ring of smem stages (mbarrier full/empty)
//   warp 1   MMA issuer: per chunk 2 k-blocks x 4 tcgen05.mma.kind::i8 (M=128, N=BN, K=32) into one
//            of two TMEM accumulators (int32, BN columns each); tcgen05.commit frees the stage
//            and, after the 8th MMA, publishes the accumulator
//   warps 2+ epilogue: tcgen05.ld the finished accumulator, acc = fmaf(float(I), qs[q][c], acc)
//            in registers, in chunk order (the reference's order, :1519-1526), hand the TMEM
//            buffer back; at the end out = acc * bw0[r] * scale_inv.
//
// The chunk scale cannot ride inside the integer contraction (each chunk has its own power of
// two per row), which is why the accumulator is drained every 256 of depth; the two TMEM buffers
// let the drain of chunk c overlap the MMAs of chunk c+1.
//
// Every wait is bounded: on a timeout the waiting role records a site code in a device status
// word, raises a CTA-wide abort flag, every role leaves its loop, outstanding copies and MMAs
// are waited for (bounded again), TMEM is freed and the kernel returns.
#include <cuda.h>
#include <stdlib.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "quant_bytes.cuh"

namespace bsi {

// Device-side status word: 0 = clean; otherwise the site code of the first wait that gave up.
__device__ int g_device_status = 0;
// warp-tiles of the paired kernel that took the integer accumulation (a test hook: bsi_b200_debug_exact_int_tiles)
__device__ unsigned long long g_exact_int_tiles = 0ull;

namespace {

constexpr int BM = 128;     // query rows per tile = TMEM lanes
constexpr int BK = 128;     // int8 per k-block = one 128-byte swizzle row
constexpr int UMMA_K = 32;  // depth of one kind::i8 instruction
constexpr int kEpiWarps = 8;
constexpr int kThreads = (2 + kEpiWarps) * 32;
constexpr long long kWaitCycles = 4000000000ll;  // ~2 s at B200 clocks; real waits are microseconds

enum Site { kSiteProducer = 1, kSiteMmaFull = 2, kSiteMmaTmem = 3, kSiteEpilogue = 4, kSiteDrain = 5 };

template <int BN>
struct Cfg {
    static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = BN * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;  // two accumulators; 128, 256 or 512: powers of two
    static constexpr int kBarriers = 2 * kStages + 5;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarriers * 8 + 16 + 1024;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// try_wait that lets the hardware park the thread for up to `hint_ns` before it reports "not yet":
// a parked thread issues nothing, so waiting warps do not steal issue slots from the MMA issuer.
__device__ __forceinline__ bool mbar_try_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Bounded wait. Returns false when the CTA is aborting (this wait or another one timed out).
// The abort flag and the clock are looked at only every 16th unsuccessful (parked) try.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int site) {
    if (mbar_try(bar, parity)) return true;
    long long t0 = 0;
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try_parked(bar, parity, 20000u)) return true;
        if ((spins & 15u) == 0u) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            if (now - t0 > kWaitCycles) {
                *abort_flag = 1;
                atomicCAS(&g_device_status, 0, site);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// K-major, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart (SBO), descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1024u >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// kind::i8: D = S32 (2 at bit 4), A and B signed 8-bit (1 at bits 7 and 10), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// 16 columns into r[0..15] (the tail piece of tiles whose column count per warp is not a multiple of 32).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

template <int BN, bool DBG>
__global__ void __launch_bounds__(kThreads, 1) dot_i8_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
    const float* __restrict__ qs, int64_t qs_stride, const float* __restrict__ bw0,
    int Q, int R, int chunks, float scale_inv, float* __restrict__ out, int64_t ldo,
    int32_t* __restrict__ dbg_iacc) {
    using C = Cfg<BN>;
    constexpr int kStages = C::kStages;
    constexpr int kCols = BN / 2;  // accumulator columns per epilogue warp

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * C::kStageBytes);
    // bars: full[kStages], empty[kStages], tfull[2], tempty[2], drain
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kBarriers);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN;
    const int m0 = blockIdx.y * BM;
    const int num_kb = chunks * 2;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), kEpiWarps * 32);
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(static_cast<uint32_t>(C::kTmemCols)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % kStages;
                const uint32_t ph = static_cast<uint32_t>(kb / kStages) & 1u;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, kSiteProducer)) break;
                mbar_expect_tx(full_bar(s), C::kStageBytes);
                const uint32_t a_dst = smem_base + s * C::kStageBytes;
                tma_load_2d(a_dst, &map_a, kb * BK, m0, full_bar(s));
                tma_load_2d(a_dst + C::kABytes, &map_b, kb * BK, n0, full_bar(s));
                issued = kb + 1;
            }
            if (*abort_flag) {
                // Let every copy that was issued land before the CTA gives its smem back.
                const int first = issued > kStages ? issued - kStages : 0;
                for (int kb = first; kb < issued; ++kb) {
                    const int s = kb % kStages;
                    const uint32_t ph = static_cast<uint32_t>(kb / kStages) & 1u;
                    const long long t0 = clock64();
                    while (!mbar_try(full_bar(s), ph) && clock64() - t0 < kWaitCycles / 64) {}
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BN);
            bool ok = true;
            for (int c = 0; c < chunks && ok; ++c) {
                const int b = c & 1;
                const uint32_t tph = static_cast<uint32_t>(c >> 1) & 1u;
                if (!mbar_wait(tempty_bar(b), tph ^ 1u, abort_flag, kSiteMmaTmem)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(b * BN);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int kb = 2 * c + half;
                    const int s = kb % kStages;
                    const uint32_t ph = static_cast<uint32_t>(kb / kStages) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_flag, kSiteMmaFull)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + s * C::kStageBytes;
                    const uint64_t adesc = umma_desc(a_addr);
                    const uint64_t bdesc = umma_desc(a_addr + C::kABytes);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // +32 bytes of K inside the swizzle row = +2 in the 16-byte address field
                        umma_i8(tmem_d, adesc + 2u * k, bdesc + 2u * k, idesc, (half | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));
                }
                if (ok) umma_commit(tfull_bar(b));
            }
            if (!ok) {
                // Wait (bounded) for whatever MMAs are still in flight before TMEM is freed.
                umma_commit(drain_bar);
                const long long t0 = clock64();
                while (!mbar_try(drain_bar, 0) && clock64() - t0 < kWaitCycles / 64) {}
            }
        }
    } else {
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
        const int half = (warp - 2) >> 2;          // which half of the BN columns
        const int row = m0 + quad * 32 + lane;     // query row of this thread
        const int col0 = half * kCols;
        const bool row_ok = row < Q;
        const float* qs_row = qs + static_cast<int64_t>(row_ok ? row : 0) * (qs_stride ? qs_stride : 1);
        float acc[kCols];
#pragma unroll
        for (int j = 0; j < kCols; ++j) acc[j] = 0.0f;

        bool ok = true;
        for (int c = 0; c < chunks && ok; ++c) {
            const int b = c & 1;
            const uint32_t tph = static_cast<uint32_t>(c >> 1) & 1u;
            const float qscale = qs_stride ? __ldg(qs_row + c) : __ldg(qs_row);
            if (!mbar_wait(tfull_bar(b), tph, abort_flag, kSiteEpilogue)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                                   static_cast<uint32_t>(b * BN + col0);
#pragma unroll
            for (int j = 0; j < kCols / 32; ++j) {
                int32_t v[32];
                tmem_ld32(taddr + j * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    acc[j * 32 + e] = __fmaf_rn(static_cast<float>(v[e]), qscale, acc[j * 32 + e]);
                }
                if (DBG) {
                    if (row_ok) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const int col = n0 + col0 + j * 32 + e;
                            if (col < R)
                                dbg_iacc[(static_cast<int64_t>(row) * R + col) * chunks + c] = v[e];
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(tempty_bar(b));
        }
        if (ok && row_ok) {
            float* orow = out + static_cast<int64_t>(row) * ldo;
            const bool vec = ((reinterpret_cast<uintptr_t>(orow) & 15) == 0) &&
                             ((reinterpret_cast<uintptr_t>(bw0) & 15) == 0) && (n0 + col0 + kCols <= R);
            if (vec) {
#pragma unroll
                for (int j = 0; j < kCols; j += 4) {
                    const int col = n0 + col0 + j;
                    const float4 w = __ldg(reinterpret_cast<const float4*>(bw0 + col));
                    float4 o;
                    o.x = (acc[j + 0] * w.x) * scale_inv;
                    o.y = (acc[j + 1] * w.y) * scale_inv;
                    o.z = (acc[j + 2] * w.z) * scale_inv;
                    o.w = (acc[j + 3] * w.w) * scale_inv;
                    *reinterpret_cast<float4*>(orow + col) = o;
                }
            } else {
#pragma unroll
                for (int j = 0; j < kCols; ++j) {
                    const int col = n0 + col0 + j;
                    if (col < R) orow[col] = (acc[j] * __ldg(bw0 + col)) * scale_inv;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(static_cast<uint32_t>(C::kTmemCols)) : "memory");
    }
}

#include "dot_tcgen05_pair.cuh"

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &qres) ==
                cudaSuccess && qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    }
    return fn;
}

// [rows, depth] int8, row stride ld bytes; box = 128 bytes of depth x box_rows rows, 128-byte
// swizzle; rows beyond `rows` read as zero.
int make_map(CUtensorMap* map, const int8_t* base, int64_t rows, int64_t depth, int64_t ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(BSI_ERR_CUDA, "dot_i8: cuTensorMapEncodeTiled entry point not found");
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(depth), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(base), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("dot_i8: cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
        return BSI_ERR_CUDA;
    }
    return BSI_OK;
}

template <int BN, bool DBG>
int launch_tile(const CUtensorMap& ma, const CUtensorMap& mb, const float* qs, int64_t qs_stride,
                const float* bw0, int Q, int R, int chunks, float scale_inv, float* out, int64_t ldo,
                int32_t* dbg, cudaStream_t stream) {
    using C = Cfg<BN>;
    static bool attr_set[64] = {false};
    int dev = 0;
    BSI_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        BSI_CUDA_TRY(cudaFuncSetAttribute(dot_i8_tcgen05_kernel<BN, DBG>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    dim3 grid((R + BN - 1) / BN, (Q + BM - 1) / BM, 1);
    dot_i8_tcgen05_kernel<BN, DBG><<<grid, kThreads, C::kSmemBytes, stream>>>(
        ma, mb, qs, qs_stride, bw0, Q, R, chunks, scale_inv, out, ldo, dbg);
    return check_launch("dot_i8 tcgen05 launch");
}

template <int BN, bool DBG, typename OutT, bool REQ = false>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, int vector_store,
                const float* qs, int64_t qs_stride, const float* bw0, const float* bias, int Q, int R, int chunks,
                float scale_inv, void* out, int64_t ldo, int32_t* dbg, const ScatterDst& scatter,
                const RequantDst& requant, const float* k_abs_sum, float q_abs_max, const float* q_sq, int64_t q_sq_stride,
                cudaStream_t stream) {
    using C = pair::Cfg<BN>;
    static int max_clusters[64] = {0};   // per instantiation
    int dev = 0;
    BSI_CUDA_TRY(cudaGetDevice(&dev));
    const int tiles_m = (Q + 255) / 256;
    const int tiles_n = (R + BN - 1) / BN;
    const int tiles_total = tiles_m * tiles_n;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: this kernel's set-up may overlap the tail of the kernel before it
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.blockDim = dim3(pair::kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    int resident = 0;
    if (dev >= 0 && dev < 64) resident = max_clusters[dev];
    if (resident == 0) {
        BSI_CUDA_TRY(cudaFuncSetAttribute(pair::dot_i8_tcgen05_pair_kernel<BN, DBG, OutT, REQ>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        cfg.gridDim = dim3(2 * (sm_count() / 2), 1, 1);
        BSI_CUDA_TRY(cudaOccupancyMaxActiveClusters(&resident, pair::dot_i8_tcgen05_pair_kernel<BN, DBG, OutT, REQ>, &cfg));
        if (resident <= 0) return fail(BSI_ERR_CUDA, "dot_i8: no cluster of 2 CTAs fits on this device");
        if (dev >= 0 && dev < 64) max_clusters[dev] = resident;
    }
    int pairs = tiles_total < resident ? tiles_total : resident;
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    BSI_CUDA_TRY(cudaLaunchKernelEx(&cfg, pair::dot_i8_tcgen05_pair_kernel<BN, DBG, OutT, REQ>, ma, mb, vector_store, qs,
                                    qs_stride, bw0, bias, Q, R, chunks, tiles_m, tiles_total, scale_inv, out, ldo, dbg, scatter, requant,
                                    k_abs_sum, q_abs_max, q_sq, q_sq_stride));
    return check_launch("dot_i8 tcgen05 pair launch");
}

// Pair kernel tile width. Measured on the 512 x 8192 x 2048 shape, a pair spends about 650 + 3.1 * BN cycles per
// 256-deep chunk of a tile (the epilogue's per-column work plus a fixed hand-off cost), and walks through
// ceil(tiles / pairs) tiles. The widest tile wins unless a narrower one is clearly cheaper (more than 8 %: at equal
// rounds the wider tile also has the shorter fill and store phases). float32 output may use any multiple of 32,
// the 16-bit layer epilogues (whole 64-column store rounds) the powers of two.
int pick_bn_pair(int64_t Q, int64_t R, bool any_width) {
    const int pairs = sm_count() / 2;
    const int64_t mt = (Q + 255) / 256;
    int best = 256;
    double best_cost = 1e300;
    for (int bn = 256; bn >= 64; bn -= 32) {
        if (!any_width && bn != 256 && bn != 128 && bn != 64) continue;
        const int64_t tiles = mt * ((R + bn - 1) / bn);
        const int64_t waves = (tiles + pairs - 1) / pairs;
        const double cost = static_cast<double>(waves) * (650.0 + 3.1 * bn);
        if (cost < best_cost * 0.92) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

// Picks the key-tile width: the widest tile wins unless a narrower one fills more SMs.
int pick_bn(int64_t Q, int64_t R) {
    const int sms = sm_count();
    const int64_t mt = (Q + BM - 1) / BM;
    const int cand[3] = {256, 128, 64};
    const double eff[3] = {1.0, 0.9, 0.67};  // narrower tiles re-read A more often per MMA
    int best = 256;
    double best_cost = 1e300;
    for (int i = 0; i < 3; ++i) {
        const int64_t tiles = mt * ((R + cand[i] - 1) / cand[i]);
        const int64_t waves = (tiles + sms - 1) / sms;
        const double cost = static_cast<double>(waves) * cand[i] / eff[i];
        if (cost < best_cost * 0.999) {
            best_cost = cost;
            best = cand[i];
        }
    }
    return best;
}

}  // namespace

// Paired-CTA engine with the output type and the bias chosen at run time (y_dtype: BSI_DTYPE_*).
int dot_i8_pair(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride, const int8_t* k8, int64_t ldk,
                const float* bw0, const float* bias, int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                void* out, int64_t ldo, int y_dtype, int32_t* dbg_iacc, int force_bn, int relu,
                const ScatterDst* scatter_in, const RequantDst* requant_in, cudaStream_t stream) {
    RequantDst requant = {};
    if (requant_in != nullptr) {
        requant = *requant_in;
        if (requant.n < 1 || requant.n > BSI_B200_MAX_PEERS || (R & 255) != 0 ||
            (y_dtype != BSI_DTYPE_F16 && y_dtype != BSI_DTYPE_BF16) || dbg_iacc != nullptr || scatter_in != nullptr)
            return fail(BSI_ERR_INVALID, "dot_i8: re-quantised output needs R % 256 == 0 and a 16-bit layer type");
        force_bn = 256;   // one tile row = one 256-column chunk
    }
    ScatterDst scatter = {};
    if (scatter_in != nullptr) {
        scatter = *scatter_in;
        if (scatter.n < 1 || scatter.n > BSI_B200_MAX_PEERS || scatter.rows_per_dst <= 0 || (scatter.rows_per_dst & 31) != 0 ||
            static_cast<int64_t>(scatter.n) * scatter.rows_per_dst < Q)
            return fail(BSI_ERR_INVALID, "dot_i8: scatter needs 1..16 destinations of a multiple of 32 rows covering Q");
        out = scatter.y[0];
    }
    if (Q > 0x7fffff00ll || R > 0x7fffff00ll || chunks > 0x400000)
        return fail(BSI_ERR_UNSUPPORTED, "dot_i8: Q, R or chunks too large");
    const bool any_width = y_dtype == BSI_DTYPE_F32;
    // bounds registered for this key image switch on the integer accumulation where it is provably exact
    KeyBounds kb = {};
    const float* kabs = nullptr;
    float qabs = 0.0f;
    const float* qsq = nullptr;
    int64_t qsq_stride = 0;
    if (lookup_key_bounds(k8, &kb) && kb.rows == R) {
        kabs = kb.abs_sum;
        qabs = kb.query_abs_max;
        QueryBounds qb = {};
        if (qs_stride != 0 && lookup_query_bounds(a8, &qb) && qb.stride >= chunks) {
            qsq = qb.sq_norms;
            qsq_stride = qb.stride;
        }
    }
    int bn = force_bn ? force_bn : pick_bn_pair(Q, R, any_width);
    if (!force_bn && any_width && bn == 256 && kabs != nullptr && qsq != nullptr) {
        // Both sides carry their bounds, so the integer route is likely, and with its cheaper epilogue a single
        // wave of 256 x 224 tiles on more pairs beats one of 256 x 256 tiles (measured on 512 x 8192 x 2048:
        // 13.64 against 13.82 us; with the float32 chain the two are even).
        const int64_t pairs = sm_count() / 2, mt = (Q + 255) / 256;
        const int64_t t256 = mt * ((R + 255) / 256), t224 = mt * ((R + 223) / 224);
        if (t256 <= pairs && t224 <= pairs && t224 > t256) bn = 224;
    }
    if (bn < 64 || bn > 256 || (bn & 31) != 0 || (!any_width && (bn & (bn - 1)) != 0))
        return fail(BSI_ERR_INVALID, "dot_i8: tile width must be a multiple of 32 in [64, 256] (64, 128 or 256 for 16-bit outputs)");
    if (dbg_iacc != nullptr && y_dtype != BSI_DTYPE_F32)
        return fail(BSI_ERR_INVALID, "dot_i8: the accumulator dump is only available with float32 output");
    CUtensorMap ma, mb;
    if (int rc = make_map(&ma, a8, Q, chunks * 256, lda, BM)) return rc;
    if (int rc = make_map(&mb, k8, R, chunks * 256, ldk, bn / 2)) return rc;
    // 16-byte stores need an aligned base, a row pitch that is a multiple of 16 bytes and R a multiple
    // of the values per 16 bytes; anything else takes the scalar store path
    const int esz = y_dtype == BSI_DTYPE_F32 ? 4 : 2;
    const int per16 = 16 / esz;
    const int vector_store =
        (((reinterpret_cast<uintptr_t>(out) & 15) == 0 && (ldo % per16) == 0 && (R % per16) == 0) ? 1 : 0) |
        (relu ? 2 : 0);   // the kernel's store_flags
    const int q = static_cast<int>(Q), r = static_cast<int>(R), c = static_cast<int>(chunks);
#define BSI_PAIR_T(BN_, DBG_, T_)                                                                              \
    launch_pair<BN_, DBG_, T_>(ma, mb, vector_store, qs, qs_stride, bw0, bias, q, r, c, scale_inv, out, ldo,  \
                               dbg_iacc, scatter, requant, kabs, qabs, qsq, qsq_stride, stream)
#define BSI_PAIR(BN_)                                                                   \
    (y_dtype == BSI_DTYPE_F16    ? BSI_PAIR_T(BN_, false, __half)                       \
     : y_dtype == BSI_DTYPE_BF16 ? BSI_PAIR_T(BN_, false, __nv_bfloat16)                \
     : dbg_iacc                  ? BSI_PAIR_T(BN_, true, float)                         \
                                 : BSI_PAIR_T(BN_, false, float))
    if (requant.n > 0) {
        if (y_dtype == BSI_DTYPE_F16)
            return launch_pair<256, false, __half, true>(ma, mb, vector_store, qs, qs_stride, bw0, bias, q, r, c, scale_inv,
                                                         out, ldo, nullptr, scatter, requant, kabs, qabs, qsq, qsq_stride, stream);
        return launch_pair<256, false, __nv_bfloat16, true>(ma, mb, vector_store, qs, qs_stride, bw0, bias, q, r, c,
                                                            scale_inv, out, ldo, nullptr, scatter, requant, kabs, qabs, qsq,
                                                            qsq_stride, stream);
    }
#define BSI_PAIR_F32(BN_) (dbg_iacc ? BSI_PAIR_T(BN_, true, float) : BSI_PAIR_T(BN_, false, float))
    switch (bn) {
        case 256: return BSI_PAIR(256);
        case 224: return BSI_PAIR_F32(224);
        case 192: return BSI_PAIR_F32(192);
        case 160: return BSI_PAIR_F32(160);
        case 96: return BSI_PAIR_F32(96);
        case 128: return BSI_PAIR(128);
        default: return BSI_PAIR(64);
    }
#undef BSI_PAIR_F32
#undef BSI_PAIR
#undef BSI_PAIR_T
}

int dot_i8_tcgen05(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride, const int8_t* k8,
                   int64_t ldk, const float* bw0, int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                   float* out, int64_t ldo, int32_t* dbg_iacc, int force_bn, cudaStream_t stream) {
    if (Q > 0x7fffff00ll || R > 0x7fffff00ll || chunks > 0x400000)
        return fail(BSI_ERR_UNSUPPORTED, "dot_i8: Q, R or chunks too large");
    // force_bn: 0 = automatic; 64/128/256 = single-CTA tiles; 2064/2128/2256 = paired-CTA tiles.
    const bool want_pair = force_bn ? (force_bn >= 2000) : (Q > 128);
    if (want_pair) {
        return dot_i8_pair(a8, lda, qs, qs_stride, k8, ldk, bw0, nullptr, Q, R, chunks, scale_inv, out, ldo,
                           BSI_DTYPE_F32, dbg_iacc, force_bn ? force_bn - 2000 : 0, /*relu=*/0, nullptr, nullptr, stream);
    }
    const int bn = force_bn ? force_bn : pick_bn(Q, R);
    CUtensorMap ma, mb;
    if (int rc = make_map(&ma, a8, Q, chunks * 256, lda, BM)) return rc;
    if (int rc = make_map(&mb, k8, R, chunks * 256, ldk, bn)) return rc;
    const int q = static_cast<int>(Q), r = static_cast<int>(R), c = static_cast<int>(chunks);
#define BSI_DISPATCH(BN_)                                                                              \
    (dbg_iacc ? launch_tile<BN_, true>(ma, mb, qs, qs_stride, bw0, q, r, c, scale_inv, out, ldo,      \
                                       dbg_iacc, stream)                                               \
              : launch_tile<BN_, false>(ma, mb, qs, qs_stride, bw0, q, r, c, scale_inv, out, ldo,     \
                                        nullptr, stream))
    switch (bn) {
        case 256: return BSI_DISPATCH(256);
        case 128: return BSI_DISPATCH(128);
        case 64: return BSI_DISPATCH(64);
        default: return fail(BSI_ERR_INVALID, "dot_i8: tile width must be 64, 128 or 256");
    }
#undef BSI_DISPATCH
}

}  // namespace bsi

extern "C" int bsi_b200_device_status(int* status_out) {
    using namespace bsi;
    if (status_out == nullptr) return fail(BSI_ERR_INVALID, "device_status: null pointer");
    BSI_CUDA_TRY(cudaDeviceSynchronize());
    int v = 0;
    BSI_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        BSI_CUDA_TRY(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    }
    int pv = 0;
    if (int rc = take_peer_status(&pv)) return rc;
    if (v == 0) v = pv;
    *status_out = v;
    return BSI_OK;
}

extern "C" int bsi_b200_debug_exact_int_tiles(unsigned long long* count_out) {
    using namespace bsi;
    if (count_out == nullptr) return fail(BSI_ERR_INVALID, "debug_exact_int_tiles: null pointer");
    BSI_CUDA_TRY(cudaDeviceSynchronize());
    unsigned long long v = 0;
    BSI_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_exact_int_tiles, sizeof(v)));
    const unsigned long long zero = 0;
    BSI_CUDA_TRY(cudaMemcpyToSymbol(g_exact_int_tiles, &zero, sizeof(zero)));
    *count_out = v;
    return BSI_OK;
}
