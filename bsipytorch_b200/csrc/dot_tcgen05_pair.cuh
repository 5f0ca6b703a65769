// Paired-CTA, persistent variant of the int8 tcgen05 dot engine. Included by dot_tcgen05.cu (same
// translation unit: it shares the PTX wrappers and the device status word).
//
// Why pairs: with one CTA per 128 x 256 tile every SM has to pull 48 KB of operands through L2 for
// every 512 cycles of MMA work (96 B/clk/SM), and the L2->SM fabric delivers about half of that.
// Two CTAs of a cluster work on one 256 x BN tile with tcgen05.mma.cta_group::2: each CTA loads its
// own 128 query rows (A) and only HALF of the key rows (B); the pair's tensor cores read B from
// both shared memories. Operand traffic per SM drops to 32 KB per k-block (64 B/clk/SM at full rate).
//
// Why persistent: a pair walks over tiles t = pair, pair + P, ... . Barrier/TMEM set-up happens once,
// the TMA producer runs ahead into the next tile while the epilogue of the current one drains, and
// the fp32 result leaves through shared memory as coalesced stores that overlap the next tile's MMAs.
//
// Tile = 256 query rows x BN key rows, BN any multiple of 32 up to 256 (float32 output; the 16-bit layer
// epilogues use 64, 128 or 256): tcgen05.mma with M = 256 takes every N that is a multiple of 16.
//
// Roles per CTA (12 warps; register budget moved with setmaxnreg):
//   warps 0, 2, 3 TMA producers, k-blocks round robin (both CTAs; every load signals the LEADER's
//                 full barrier)
//   warp 1        MMA issuer (leader CTA only), TMEM alloc/dealloc (both CTAs)
//   warps 4..11   epilogue: TMEM -> registers, acc = fmaf(float(I), qs[q][c], acc) per chunk in order;
//                 at the end of a tile: scale, transpose through smem, coalesced st.global.v4
//
// Barriers (same smem offsets in both CTAs):
//   full[s]    leader's copy used: 1 arrival (leader producer, expect_tx of BOTH CTAs' bytes)
//   empty[s]   local in each CTA: tcgen05.commit (multicast to both CTAs) after the stage's MMAs
//   tfull[b]   local in each CTA: multicast commit after a chunk's 8 MMAs
//   tempty[b]  leader's copy used: one arrival per epilogue warp of BOTH CTAs (16)
// The accumulator ring holds 2, 4 or 8 buffers (BN > 128, > 64, = 64): with narrow tiles the MMA issuer runs
// several chunks ahead of the epilogue, which takes the barrier round trip off the critical path.
// What bounds a chunk on wide tiles is the epilogue, not the 8 MMAs (1024 cycles at BN = 256): three
// instructions per accumulator value (integer add, float add, FMA; see int_to_float_exact) at one warp
// instruction per clock and SM sub-partition, next to TMEM loads that slow down while the tensor pipe
// reads and writes its accumulators; measured about 1450 cycles per chunk at BN = 256.
// All waits are bounded; a timeout raises the abort flag of both CTAs and every role drains out.
#pragma once

namespace pair {

constexpr int kThreads = 384;
constexpr int kEpiWarps = 8;
constexpr int kFirstEpiWarp = 4;
constexpr int kRegsLow = 40;
constexpr int kRegsHigh = 232;
// setmaxnreg.inc draws only on what setmaxnreg.dec returned to the CTA's own pool (threads x registers per thread at
// launch, the latter being 65536 / threads rounded down to a multiple of 8); an increase beyond the pool never returns.
static_assert(kFirstEpiWarp * 32 * kRegsLow + kEpiWarps * 32 * kRegsHigh <= kThreads * ((65536 / kThreads) / 8 * 8),
              "register budget of the warp groups exceeds the CTA's pool");
constexpr long long kWait = 500000000ll;  // ~0.25 s; real waits are microseconds

constexpr int kSmemLimit = 232448;   // 227 KB: the most dynamic shared memory one CTA can opt in to

template <int BN>
struct Cfg {
    static_assert(BN % 32 == 0 && BN >= 64 && BN <= 256, "tile width: a multiple of 32 in [64, 256]");
    static constexpr int kHalfN = BN / 2;                 // key rows each CTA loads
    static constexpr int kABytes = BM * BK;               // 16 KB
    static constexpr int kBBytes = kHalfN * BK;           // 4 .. 16 KB, a multiple of 1 KB (swizzle atom)
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStoreBytes = kEpiWarps * 4096;  // one 32x32 fp32 block per epilogue warp
    static constexpr int kTmemCols = 512;                 // all of TMEM: 1 CTA per SM anyway
    // accumulator ring: buffers start at multiples of the next power of two >= BN (2, 4 or 8 buffers)
    static constexpr int kAccStride = BN > 128 ? 256 : (BN > 64 ? 128 : 64);
    static constexpr int kAccBufs = 512 / kAccStride;
    // chunk-maximum exchange of the re-quantising epilogue: 2 parities x 8 warps x 32 lanes x 2 bytes + 8 counters
    static constexpr int kXchgBytes = 2 * kEpiWarps * 32 * 2 + kEpiWarps * 4;
    static constexpr int kFixedBytes = kStoreBytes + (2 * 9 + 2 * kAccBufs + 1) * 8 + 16 + kXchgBytes + 1024;
    static constexpr int kFit = (kSmemLimit - kFixedBytes) / kStageBytes;
    static constexpr int kStages = kFit > 9 ? 9 : kFit;   // 6 (BN >= 192), 7, 8, 8, 9 (BN = 64)
    static constexpr int kBarriers = 2 * kStages + 2 * kAccBufs + 1;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + kBarriers * 8 + 16 + kXchgBytes + 1024;
    static_assert(kStages >= 4 && kSmemBytes <= kSmemLimit, "operand ring does not fit");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n.reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    // Plain (CTA-scope release) arrive: the ordering that matters here -- TMEM reads done before the
    // accumulator is overwritten -- comes from tcgen05.wait::ld + tcgen05.fence::before_thread_sync.
    // A cluster-scope release would put a full memory barrier into every chunk of the epilogue.
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void store_flag_cluster(uint32_t cluster_addr, int v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(leader_bar)
        : "memory");
}

__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives on the barrier at this smem offset in BOTH CTAs of the pair once all earlier MMAs are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(mask)
        : "memory");
}

// M = 256 across the pair.
__host__ __device__ constexpr uint32_t umma_idesc_pair(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(256 >> 4) << 24);
}

struct AbortCtx {
    volatile int* flag;    // this CTA's abort flag
    uint32_t peer_flag;    // cluster address of the peer's
};

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, const AbortCtx& a, int site) {
    if (mbar_try(bar, parity)) return true;
    long long t0 = 0;
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try_parked(bar, parity, 20000u)) return true;
        if ((spins & 15u) == 0u) {
            if (*a.flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            if (now - t0 > kWait) {
                *a.flag = 1;
                store_flag_cluster(a.peer_flag, 1);
                atomicCAS(&g_device_status, 0, 16 + site);
                return false;
            }
        }
    }
}

// float(v) for |v| <= 2^22 without a conversion instruction: adding v to the bit pattern of 1.5 * 2^23 gives the
// float 1.5 * 2^23 + v exactly, and subtracting the constant again is exact too. (A chunk accumulator of 8-bit
// operands is at most 256 * 128 * 128 = 2^22 in magnitude.) An integer add and a float add on the full-rate
// pipes instead of one conversion on the slow one.
__device__ __forceinline__ float int_to_float_exact(int32_t v) {
    return __int_as_float(v + 0x4B400000) - 12582912.0f;
}

// Last step of one output element. float: the raw dot value (the microbenchmark entry point).
// half / bfloat16: the layer epilogue of the reference, `scores.to(dtype) + bias.to(dtype)`
// (verify_accuracy_bsi.py:193-195): both terms are narrowed first, added, and narrowed again.
template <typename OutT>
__device__ __forceinline__ OutT finish(float v, float bias, bool has_bias);
template <>
__device__ __forceinline__ float finish<float>(float v, float bias, bool has_bias) {
    return has_bias ? v + bias : v;
}
template <>
__device__ __forceinline__ __half finish<__half>(float v, float bias, bool has_bias) {
    const __half h = __float2half_rn(v);
    return has_bias ? __float2half_rn(__half2float(h) + __half2float(__float2half_rn(bias))) : h;
}
template <>
__device__ __forceinline__ __nv_bfloat16 finish<__nv_bfloat16>(float v, float bias, bool has_bias) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    return has_bias ? __float2bfloat16_rn(__bfloat162float(h) + __bfloat162float(__float2bfloat16_rn(bias))) : h;
}

// max(v, 0) on the finished output value when the layer's activation is fused (NaN stays NaN).
template <typename OutT>
__device__ __forceinline__ OutT relu_if(OutT v, bool relu) {
    return (relu && static_cast<float>(v) < 0.0f) ? static_cast<OutT>(0.0f) : v;
}

template <int BN, bool DBG, typename OutT, bool REQ = false>
__global__ void __launch_bounds__(kThreads, 1) dot_i8_tcgen05_pair_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
    int store_flags,   // bit 0: 16-byte vector stores are possible; bit 1: ReLU on the finished value
    const float* __restrict__ qs, int64_t qs_stride, const float* __restrict__ bw0,
    const float* __restrict__ bias, int Q, int R, int chunks, int tiles_m, int tiles_total, float scale_inv,
    void* __restrict__ out, int64_t ldo, int32_t* __restrict__ dbg_iacc, const ScatterDst scatter,
    const RequantDst requant, const float* __restrict__ k_abs_sum, float q_abs_max,
    const float* __restrict__ q_sq, int64_t q_sq_stride) {
    using C = Cfg<BN>;
    constexpr int kStages = C::kStages;
    constexpr int kCols = BN / 2;              // accumulator columns per epilogue warp: a multiple of 16

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* store_area = smem + kStages * C::kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(store_area + C::kStoreBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kBarriers);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint16_t* xchg_vals = reinterpret_cast<uint16_t*>(tmem_slot + 4);                       // [2][kEpiWarps][32]
    volatile uint32_t* xchg_count = reinterpret_cast<volatile uint32_t*>(xchg_vals + 2 * kEpiWarps * 32);   // [kEpiWarps]

    // let the next kernel of the stream start its own set-up as soon as every CTA of this grid is running
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    constexpr int kAccBufs = C::kAccBufs;
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + kAccBufs + b); };
    const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 2 * kAccBufs);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const int num_kb = chunks * 2;
    const bool has_bias = bias != nullptr;
    const bool relu = (store_flags & 2) != 0;

    const uint32_t leader_full0 = map_to_cta(full_bar(0), 0);
    AbortCtx actx;
    actx.flag = abort_flag;
    actx.peer_flag = map_to_cta(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u);

    if (warp == 0) {
        // one barrier per lane: full[s], empty[s], tfull[b] and drain count 1 arrival, tempty[b] one per epilogue
        // warp of both CTAs
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
            *abort_flag = 0;
        }
        if (lane < kEpiWarps) xchg_count[lane] = 0u;
        for (int i = lane; i < C::kBarriers; i += 32) {
            const bool is_tempty = i >= 2 * kStages + kAccBufs && i < 2 * kStages + 2 * kAccBufs;
            mbar_init(bar_base + 8u * i, is_tempty ? 2 * kEpiWarps : 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // Cluster barrier split around the TMEM allocation: arrive now (thread 0's barrier inits are
    // released by its own arrive), wait after the allocation, so the two latencies overlap.
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    const bool is_producer = warp < kFirstEpiWarp && warp != 1;
    uint32_t tmem_base = 0;
    if (is_producer) {
        // The producers need the barriers of both CTAs, not the accumulator memory: they go on to their
        // first copies while warp 1 is still allocating TMEM.
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    } else {
        if (warp == 1) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(tmem_slot)), "r"(static_cast<uint32_t>(C::kTmemCols)) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        }
        tc_fence_before();
        // warp 1 and the eight epilogue warps: the TMEM address is in shared memory from here on
        asm volatile("bar.sync 1, %0;" ::"n"((1 + kEpiWarps) * 32) : "memory");
        // both CTAs' barriers are initialised before anyone touches the peer's
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        tc_fence_after();
        tmem_base = *tmem_slot;
    }

    // Programmatic dependent launch: everything above (barriers, TMEM, tensor-map prefetch) touched no global
    // memory of an earlier kernel and may run while that kernel drains; from here on its results are needed.
    // Without the launch attribute both instructions do nothing.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp < kFirstEpiWarp) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLow));
        if (warp != 1 && lane == 0) {
            // ---------------- TMA producers ----------------
            // One thread needs ~450 cycles per k-block (empty wait, expect_tx, two tensor copies), which
            // is slower than the MMAs consume narrow tiles; warps 0, 2 and 3 therefore take the k-blocks
            // round robin. Stage s = it % kStages is always filled by the producer that owns `it`.
            constexpr int kProducers = 3;
            const int me = warp == 0 ? 0 : warp - 1;
            int it = 0;
            bool ok = true;
            for (int tile = pair_id; tile < tiles_total && ok; tile += num_pairs) {
                const int tm = tile % tiles_m;
                const int tn = tile / tiles_m;
                const int row_a = tm * 256 + static_cast<int>(rank) * BM;
                const int row_b = tn * BN + static_cast<int>(rank) * C::kHalfN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    if (it % kProducers != me) continue;
                    const int s = it % kStages;
                    const uint32_t ph = static_cast<uint32_t>(it / kStages) & 1u;
                    if (!wait_or_abort(empty_bar(s), ph ^ 1u, actx, 1)) { ok = false; break; }
                    if (leader) mbar_expect_tx(full_bar(s), 2u * C::kStageBytes);
                    const uint32_t a_dst = smem_base + s * C::kStageBytes;
                    tma_load_2d_pair(a_dst, &map_a, kb * BK, row_a, leader_full0 + 8u * s);
                    tma_load_2d_pair(a_dst + C::kABytes, &map_b, kb * BK, row_b, leader_full0 + 8u * s);
                }
            }
        } else if (warp == 1 && leader) {
            // ---------------- MMA issuer (leader CTA) ----------------
            // The whole warp walks the loop (so that addresses and descriptors stay in the uniform
            // datapath) and one elected lane issues the tensor-core instructions.
            constexpr uint32_t idesc = umma_idesc_pair(BN);
            int it = 0, cc = 0;
            bool ok = true;
            for (int tile = pair_id; tile < tiles_total && ok; tile += num_pairs) {
                for (int c = 0; c < chunks && ok; ++c, ++cc) {
                    const int b = cc % kAccBufs;
                    const uint32_t tph = static_cast<uint32_t>(cc / kAccBufs) & 1u;
                    if (!wait_or_abort(tempty_bar(b), tph ^ 1u, actx, 3)) { ok = false; break; }
                    const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(b * C::kAccStride);
#pragma unroll
                    for (int half = 0; half < 2; ++half, ++it) {
                        const int s = it % kStages;
                        const uint32_t ph = static_cast<uint32_t>(it / kStages) & 1u;
                        if (!wait_or_abort(full_bar(s), ph, actx, 2)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a_addr = smem_base + s * C::kStageBytes;
                        const uint64_t adesc = umma_desc(a_addr);
                        const uint64_t bdesc = umma_desc(a_addr + C::kABytes);
                        if (elect_one()) {
#pragma unroll
                            for (int k = 0; k < BK / UMMA_K; ++k) {
                                umma_i8_pair(tmem_d, adesc + 2u * k, bdesc + 2u * k, idesc,
                                             (half | k) != 0 ? 1u : 0u);
                            }
                            umma_commit_pair(empty_bar(s));
                            if (half == 1) umma_commit_pair(tfull_bar(b));
                        }
                        __syncwarp();
                    }
                }
            }
            if (!ok && lane == 0) {
                umma_commit(drain_bar);
                const long long t0 = clock64();
                while (!mbar_try(drain_bar, 0) && clock64() - t0 < kWait / 64) {}
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsHigh));
        // ---------------- epilogue ----------------
        const int ew = warp - kFirstEpiWarp;   // 0..7
        const int quad = warp & 3;             // TMEM lane quadrant this warp may read
        const int half = ew >> 2;              // which half of the BN columns
        const int col0 = half * kCols;
        uint8_t* my_store = store_area + ew * 4096;
        const uint32_t leader_tempty0 = map_to_cta(tempty_bar(0), 0);

        float acc[kCols];
        int cc = 0;
        bool ok = true;
        uint32_t tiles_done = 0;   // tiles this warp has re-quantised (the chunk-maximum exchange counts them)
        for (int tile = pair_id; tile < tiles_total && ok; tile += num_pairs) {
            const int tm = tile % tiles_m;
            const int tn = tile / tiles_m;
            const int row = tm * 256 + static_cast<int>(rank) * BM + quad * 32 + lane;
            const int n0 = tn * BN;
            const bool row_ok = row < Q;
            const float* qs_row = qs + static_cast<int64_t>(row_ok ? row : 0) * (qs_stride ? qs_stride : 1);
#pragma unroll
            for (int j = 0; j < kCols; ++j) acc[j] = 0.0f;
            // Key scales of this warp's columns: lane L keeps columns 4L..4L+3 (of the warp's kCols) in
            // registers; the load's latency hides behind the mainloop and the store phase fetches them
            // with shuffles.
            float bwreg[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            float biasreg[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (lane * 4 < kCols) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = n0 + col0 + lane * 4 + e;
                    if (col < R) {
                        bwreg[e] = __ldg(bw0 + col);
                        if (has_bias) biasreg[e] = __ldg(bias + col);
                    }
                }
            }

            // Integer accumulation where it provably equals the float32 chain: the chunk terms I_c * 2^shift are
            // integers, so while every prefix sum stays below 2^24 in magnitude no float32 addition rounds and
            // acc += I_c << shift in int32 gives the same bits. With A the largest query magnitude, a prefix is at
            // most A x (largest 2^shift of the row) x (sum of |k| over the key row), and also at most
            // A x (sum of the row's 2^shift) x (largest sum of |k| over one chunk of the key row); the key sums come
            // from the caller (k_abs_sum: R row sums, then R chunk maxima, then R sums of squares; null: not
            // available). Where both fail and the query image carries its chunk sums of squares (q_sq), the
            // Cauchy-Schwarz product of the two rows' L2 norms is tried. The test is made for the warp's 32 rows x
            // kCols columns at once, so the branch is uniform; a warp whose bounds all fail runs the float32 chain.
            bool exact = false;
            if (k_abs_sum != nullptr) {
                // largest and summed 2^shift of the row
                float smax = 0.0f, ssum = 0.0f;
                if (row_ok) {
                    if (qs_stride) {
                        // the row's chunk scales, 16 bytes at a time and four loads in flight where the row allows
                        int c = 0;
                        float m0 = 0.0f, m1 = 0.0f, m2 = 0.0f, m3 = 0.0f, t0 = 0.0f, t1 = 0.0f, t2 = 0.0f, t3 = 0.0f;
                        if ((reinterpret_cast<uintptr_t>(qs_row) & 15) == 0) {
                            const float4* q4 = reinterpret_cast<const float4*>(qs_row);
                            for (; c + 16 <= chunks; c += 16) {
                                const float4 a = __ldg(q4 + (c >> 2)), b4 = __ldg(q4 + (c >> 2) + 1);
                                const float4 d = __ldg(q4 + (c >> 2) + 2), e4 = __ldg(q4 + (c >> 2) + 3);
                                m0 = fmaxf(m0, fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)));
                                m1 = fmaxf(m1, fmaxf(fmaxf(b4.x, b4.y), fmaxf(b4.z, b4.w)));
                                m2 = fmaxf(m2, fmaxf(fmaxf(d.x, d.y), fmaxf(d.z, d.w)));
                                m3 = fmaxf(m3, fmaxf(fmaxf(e4.x, e4.y), fmaxf(e4.z, e4.w)));
                                t0 += (a.x + a.y) + (a.z + a.w);
                                t1 += (b4.x + b4.y) + (b4.z + b4.w);
                                t2 += (d.x + d.y) + (d.z + d.w);
                                t3 += (e4.x + e4.y) + (e4.z + e4.w);
                            }
                            for (; c + 4 <= chunks; c += 4) {
                                const float4 a = __ldg(q4 + (c >> 2));
                                m0 = fmaxf(m0, fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)));
                                t0 += (a.x + a.y) + (a.z + a.w);
                            }
                        }
                        for (; c < chunks; ++c) {
                            const float v1 = __ldg(qs_row + c);
                            m0 = fmaxf(m0, v1);
                            t0 += v1;
                        }
                        smax = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                        ssum = (t0 + t1) + (t2 + t3);
                    } else {
                        smax = __ldg(qs_row);
                        ssum = smax * static_cast<float>(chunks);
                    }
                }
                // of the warp's key rows: the largest sum of |k| over a row and over one 256-element chunk
                float ktot = 0.0f, kchk = 0.0f;
                if (lane * 4 < kCols) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int col = n0 + col0 + lane * 4 + e;
                        if (col < R) {
                            ktot = fmaxf(ktot, __ldg(k_abs_sum + col));
                            kchk = fmaxf(kchk, __ldg(k_abs_sum + R + col));
                        }
                    }
                }
                // non-negative floats order like their bit patterns; an infinity anywhere fails the test
                const float su = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(smax)));
                const float tu = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(ssum)));
                const float ku = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(ktot)));
                const float cu = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(kchk)));
                // the sums above round (relative 2^-24 per addition, at most a few hundred additions): 0.999 covers it
                exact = fminf(su * ku, tu * cu) * q_abs_max < 16777216.0f * 0.999f;
                if (!exact && q_sq != nullptr) {
                    // Cauchy-Schwarz: |prefix|^2 <= (sum of squares of the de-shifted query row) x (sum of k^2)
                    float u2 = 0.0f;
                    if (row_ok) {
                        const float* nrow = q_sq + static_cast<int64_t>(row) * q_sq_stride;
                        float a0 = 0.0f, a1 = 0.0f;
                        int c = 0;
                        for (; c + 2 <= chunks; c += 2) {
                            a0 += __ldg(nrow + c);
                            a1 += __ldg(nrow + c + 1);
                        }
                        if (c < chunks) a0 += __ldg(nrow + c);
                        u2 = a0 + a1;
                    }
                    float k2 = 0.0f;
                    if (lane * 4 < kCols) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int col = n0 + col0 + lane * 4 + e;
                            if (col < R) k2 = fmaxf(k2, __ldg(k_abs_sum + 2 * static_cast<int64_t>(R) + col));
                        }
                    }
                    const float u2w = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(u2)));
                    const float k2w = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(k2)));
                    exact = u2w * k2w < 281474976710656.0f * 0.999f;      // 2^48
                }
            }

            for (int c = 0; c < chunks && ok; ++c, ++cc) {
                const int b = cc % kAccBufs;
                const uint32_t tph = static_cast<uint32_t>(cc / kAccBufs) & 1u;
                const float qscale = qs_stride ? __ldg(qs_row + c) : __ldg(qs_row);
                const int qmul = exact ? __float2int_rn(qscale) : 0;
                if (!wait_or_abort(tfull_bar(b), tph, actx, 4)) { ok = false; break; }
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                                       static_cast<uint32_t>(b * C::kAccStride + col0);
                // The warp's kCols columns come in pieces of up to 64 (two loads issued back to back, one wait):
                // under the tensor pipe's own accumulator traffic a TMEM load takes a few hundred cycles, and the
                // fewer round trips a chunk needs, the sooner its buffer goes back to the MMA issuer. While this
                // warp waits, the other epilogue warp of the SM sub-partition folds its piece.
                int32_t v[2][32];
                constexpr int kSuper = (kCols + 63) / 64;
#pragma unroll
                for (int sp = 0; sp < kSuper; ++sp) {
                    const int c0 = sp * 64;
                    const int wsp = (kCols - c0) < 64 ? (kCols - c0) : 64;   // 64, 48, 32 or 16
                    if (wsp >= 32) tmem_ld32(taddr + c0, v[0]); else tmem_ld16(taddr + c0, v[0]);
                    if (wsp == 64) tmem_ld32(taddr + c0 + 32, v[1]);
                    else if (wsp == 48) tmem_ld16(taddr + c0 + 32, v[1]);
                    tmem_ld_wait();
                    if (sp + 1 == kSuper) {
                        // every column of the buffer is in registers: hand it back before the last piece is folded in
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(leader_tempty0 + 8u * b);
                    }
                    if (exact) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                if (h * 32 + e < wsp)
                                    acc[c0 + h * 32 + e] =
                                        __int_as_float(v[h][e] * qmul + __float_as_int(acc[c0 + h * 32 + e]));
                            }
                        }
                    } else {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                if (h * 32 + e < wsp)
                                    acc[c0 + h * 32 + e] = __fmaf_rn(int_to_float_exact(v[h][e]), qscale, acc[c0 + h * 32 + e]);
                            }
                        }
                    }
                    if (DBG) {
                        if (row_ok) {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
#pragma unroll
                                for (int e = 0; e < 32; ++e) {
                                    const int col = n0 + col0 + c0 + h * 32 + e;
                                    if (h * 32 + e < wsp && col < R)
                                        dbg_iacc[(static_cast<int64_t>(row) * R + col) * chunks + c] = v[h][e];
                                }
                            }
                        }
                    }
                }
            }
            if (!ok) break;
            if (exact) {
                // the int32 sums (below 2^24 in magnitude) as floats: what the float32 chain would hold
#pragma unroll
                for (int j = 0; j < kCols; ++j) acc[j] = static_cast<float>(__float_as_int(acc[j]));
                if (lane == 0) atomicAdd(&g_exact_int_tiles, 1ull);
            }

            // ---- tile result: out = (acc * bw0[r]) * scale_inv ----
            // A lane owns a row; 32 x 32 blocks go through this warp's 4 KB of smem (16-byte chunks
            // XOR-swizzled by row so that both directions are conflict free) and leave as
            // st.global.v4 with 8 lanes per 128-byte row segment: every store instruction writes
            // four full 128-byte lines. Plain stores are fire-and-forget, so the warp moves on to
            // the next tile (or exits) while they drain.
            const int row_base = tm * 256 + static_cast<int>(rank) * BM + quad * 32;
            constexpr int E = static_cast<int>(sizeof(OutT));
            constexpr int kPerChunk = 16 / E;                                   // values per 16-byte chunk
            constexpr int kRoundCols = (kCols * E >= 128) ? 128 / E : kCols;    // columns staged per round
            constexpr int kChunks = kRoundCols * E / 16;                        // 8, or 4 for 64-byte rows
            constexpr int kRounds = kCols / kRoundCols;
            constexpr int kRowBytes = kChunks * 16;
            if constexpr (REQ) {
                static_assert(BN == 256 && !DBG && sizeof(OutT) == 2, "re-quantisation: 256-wide tiles, 16-bit layer type");
                {
                    // ---- fused re-quantisation: the finished value in the layer's type (cast + bias, ReLU) is
                    // what the next linear's packer would read; with BN = 256 a tile row is exactly one chunk,
                    // split between this warp and the warp of the other column half. Same integers as the pack
                    // kernel's fast path (the values have 16-bit precision, so the float32 rounding is exact).
                    uint32_t amax_bits = 0;
#pragma unroll
                    for (int j = 0; j < kCols; ++j) {
                        const float w = __shfl_sync(0xffffffffu, bwreg[j & 3], j >> 2);
                        const float bv = __shfl_sync(0xffffffffu, biasreg[j & 3], j >> 2);
                        // cast, then add the bias rounded to the layer type (0 without bias: the sum is then the
                        // value itself), round again: what finish<OutT> computes, without its branch on has_bias
                        float v = static_cast<float>(static_cast<OutT>((acc[j] * w) * scale_inv));
                        v = static_cast<float>(static_cast<OutT>(v + static_cast<float>(static_cast<OutT>(bv))));
                        if (relu && v < 0.0f) v = 0.0f;
                        acc[j] = v;
                        amax_bits = max(amax_bits, __float_as_uint(v) & 0x7fffffffu);
                        if ((j & 15) == 15) asm volatile("" ::: "memory");   // keeps the 128 steps from being interleaved
                    }
                    // Largest magnitude of the whole chunk: swap with the partner warp (same rows, other column
                    // half). The value is one of the OutT values, so its 16-bit pattern carries it exactly. Each
                    // warp publishes into its slot of parity (tiles_done & 1) and bumps its counter; a slot is
                    // rewritten two tiles later, after the partner's next publication, which follows its read.
                    // The wait is bounded like every other wait of the kernel.
                    {
                        const uint32_t par = tiles_done & 1u;
                        const OutT amax_t = static_cast<OutT>(__uint_as_float(amax_bits));
                        xchg_vals[(par * kEpiWarps + ew) * 32 + lane] = *reinterpret_cast<const uint16_t*>(&amax_t);
                        __syncwarp();
                        if (lane == 0) {
                            __threadfence_block();
                            xchg_count[ew] = tiles_done + 1u;
                        }
                        const long long t0 = clock64();
                        while (static_cast<int32_t>(xchg_count[ew ^ 4] - (tiles_done + 1u)) < 0) {
                            if (*actx.flag || clock64() - t0 > kWait) {
                                *actx.flag = 1;
                                store_flag_cluster(actx.peer_flag, 1);
                                atomicCAS(&g_device_status, 0, 16 + 7);
                                ok = false;
                                break;
                            }
                        }
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        __threadfence_block();
                        const uint16_t other = xchg_vals[(par * kEpiWarps + (ew ^ 4)) * 32 + lane];
                        const OutT other_t = *reinterpret_cast<const OutT*>(&other);
                        amax_bits = max(amax_bits, __float_as_uint(static_cast<float>(other_t)) & 0x7fffffffu);
                        ++tiles_done;
                    }
                    float ymax = __uint_as_float(amax_bits) * requant.mult;
                    if (!(amax_bits < 0x7f800000u && ymax < 8388608.0f)) {
                        // NaN / inf / out of the exact range: not representable on this path; report, store zeros
                        atomicCAS(&g_device_status, 0, 48);
                        ymax = 0.0f;
#pragma unroll
                        for (int j = 0; j < kCols; ++j) acc[j] = 0.0f;
                    }
                    const int shift = fast_shift(ymax, requant.bits);
                    float inv, cst;
                    fast_round_consts(shift, inv, cst);
                    // stage 32 rows x 128 bytes through this warp's 4 KB (16-byte chunks XOR-swizzled by row)
                    uint8_t* dst = my_store + lane * 128;
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        uint32_t wv[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int j = ch * 16 + k * 4;
                            wv[k] = sign_clamp4(fast_magnitude(acc[j], requant.mult, inv, cst),
                                                fast_magnitude(acc[j + 1], requant.mult, inv, cst),
                                                fast_magnitude(acc[j + 2], requant.mult, inv, cst),
                                                fast_magnitude(acc[j + 3], requant.mult, inv, cst),
                                                __float_as_uint(acc[j]), __float_as_uint(acc[j + 1]),
                                                __float_as_uint(acc[j + 2]), __float_as_uint(acc[j + 3]), requant.bits);
                        }
                        *reinterpret_cast<uint4*>(dst + ((ch ^ (lane & 7)) << 4)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                    }
                    __syncwarp();
                    const int cchunk = lane & 7;
                    const int col = n0 + col0 + cchunk * 16;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = i * 4 + (lane >> 3);
                        const uint4 o = *reinterpret_cast<const uint4*>(my_store + rr * 128 + ((cchunk ^ (rr & 7)) << 4));
                        const int grow = row_base + rr;
                        if (grow < Q) {
                            const int64_t off = static_cast<int64_t>(grow) * requant.ld8 + col;
#pragma unroll
                            for (int d = 0; d < BSI_B200_MAX_PEERS; ++d)
                                if (d < requant.n) *reinterpret_cast<uint4*>(requant.q8[d] + off) = o;
                        }
                    }
                    if (half == 0 && row_ok) {
                        const float scale = __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);   // 2^shift
                        const int64_t off = static_cast<int64_t>(row) * requant.scale_ld + (n0 >> 8);
#pragma unroll
                        for (int d = 0; d < BSI_B200_MAX_PEERS; ++d)
                            if (d < requant.n) requant.scales[d][off] = scale;
                    }
                    __syncwarp();
                    continue;
                }
            }
            OutT* outp = static_cast<OutT*>(out);
            int row_shift = 0;   // first global row of the destination matrix this warp's 32 rows belong to
            if (scatter.n > 0) {
                int d = row_base / scatter.rows_per_dst;
                d = d < scatter.n ? d : scatter.n - 1;
                outp = static_cast<OutT*>(scatter.y[d]);
                row_shift = d * scatter.rows_per_dst;
            }
            if ((store_flags & 1)) {
                if constexpr (sizeof(OutT) == 4) {
                    // float32 output: the raw running sums are transposed first and scaled afterwards, when a
                    // lane holds four consecutive columns of a row: the key scales (and bias) of those columns
                    // are four loads per round instead of two shuffles per value (the warp shuffles of the
                    // other order cost as many cycles as the stores themselves). Rounds of 32 columns, then
                    // one of 16 when the warp's column count is not a multiple of 32.
                    float* outf = reinterpret_cast<float*>(outp);
                    constexpr int kFull = kCols / 32;
                    constexpr int kRoundsF = kFull + ((kCols % 32) != 0 ? 1 : 0);
#pragma unroll
                    for (int g = 0; g < kRoundsF; ++g) {
                        const bool tail = g == kFull;
                        const int nch = tail ? 4 : 8;          // 16-byte pieces per staged row
                        const int cchunk = lane & (nch - 1);
                        const int col = n0 + col0 + g * 32 + cchunk * 4;
                        float w[4], bv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const bool in = col + e < R;
                            w[e] = in ? __ldg(bw0 + col + e) : 0.0f;
                            bv[e] = (in && has_bias) ? __ldg(bias + col + e) : 0.0f;
                        }
                        uint8_t* dst = my_store + lane * (nch * 16);
#pragma unroll
                        for (int ch = 0; ch < 8; ++ch) {
                            if (ch < nch) {
                                const int swz = tail ? (ch ^ ((lane >> 1) & 3)) : (ch ^ (lane & 7));
                                const int j = g * 32 + ch * 4;
                                *reinterpret_cast<float4*>(dst + (swz << 4)) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                            }
                        }
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            if (i < nch) {
                                const int rr = i * (32 / nch) + lane / nch;
                                const int swz = tail ? (cchunk ^ ((rr >> 1) & 3)) : (cchunk ^ (rr & 7));
                                float4 o = *reinterpret_cast<const float4*>(my_store + rr * (nch * 16) + (swz << 4));
                                o.x = relu_if<float>(finish<float>((o.x * w[0]) * scale_inv, bv[0], has_bias), relu);
                                o.y = relu_if<float>(finish<float>((o.y * w[1]) * scale_inv, bv[1], has_bias), relu);
                                o.z = relu_if<float>(finish<float>((o.z * w[2]) * scale_inv, bv[2], has_bias), relu);
                                o.w = relu_if<float>(finish<float>((o.w * w[3]) * scale_inv, bv[3], has_bias), relu);
                                const int grow = row_base + rr;
                                if (grow < Q && col < R) {   // R is a multiple of 4 on this path
                                    *reinterpret_cast<float4*>(outf + static_cast<int64_t>(grow - row_shift) * ldo + col) = o;
                                }
                            }
                        }
                        __syncwarp();
                    }
                } else {
                static_assert(kCols % kRoundCols == 0, "this store order needs whole rounds");
#pragma unroll
                for (int g = 0; g < kRounds; ++g) {
                    const int colg = n0 + col0 + g * kRoundCols;
                    uint8_t* dst = my_store + lane * kRowBytes;
#pragma unroll
                    for (int ch = 0; ch < kChunks; ++ch) {
                        OutT vals[kPerChunk];
#pragma unroll
                        for (int e = 0; e < kPerChunk; ++e) {
                            const int j = g * kRoundCols + ch * kPerChunk + e;
                            const float w = __shfl_sync(0xffffffffu, bwreg[j & 3], j >> 2);
                            const float bv = __shfl_sync(0xffffffffu, biasreg[j & 3], j >> 2);
                            vals[e] = relu_if<OutT>(finish<OutT>((acc[j] * w) * scale_inv, bv, has_bias), relu);
                        }
                        const int swz = kChunks == 8 ? (ch ^ (lane & 7)) : (ch ^ ((lane >> 1) & 3));
                        *reinterpret_cast<uint4*>(dst + (swz << 4)) = *reinterpret_cast<const uint4*>(vals);
                    }
                    __syncwarp();
                    const int cchunk = lane % kChunks;
                    const int col = colg + cchunk * kPerChunk;
#pragma unroll
                    for (int i = 0; i < kChunks; ++i) {
                        const int rr = i * (32 / kChunks) + lane / kChunks;
                        const int swz = kChunks == 8 ? (cchunk ^ (rr & 7)) : (cchunk ^ ((rr >> 1) & 3));
                        const uint4 o = *reinterpret_cast<const uint4*>(my_store + rr * kRowBytes + (swz << 4));
                        const int grow = row_base + rr;
                        if (grow < Q && col < R) {   // R is a multiple of kPerChunk on this path
                            *reinterpret_cast<uint4*>(outp + static_cast<int64_t>(grow - row_shift) * ldo + col) = o;
                        }
                    }
                    __syncwarp();
                }
                }
            } else {
                OutT* orow = outp + static_cast<int64_t>(row_ok ? row - row_shift : 0) * ldo;
#pragma unroll
                for (int j = 0; j < kCols; ++j) {
                    const int col = n0 + col0 + j;
                    const float w = __shfl_sync(0xffffffffu, bwreg[j & 3], j >> 2);
                    const float bv = __shfl_sync(0xffffffffu, biasreg[j & 3], j >> 2);
                    if (row_ok && col < R) orow[col] = relu_if<OutT>(finish<OutT>((acc[j] * w) * scale_inv, bv, has_bias), relu);
                }
            }
        }
    }

    if (threadIdx.x == 0 && *abort_flag) {
        // Error path only: give copies that are still in flight time to land before the smem goes away.
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000ll) {}
    }
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();  // the peer may still be reading this CTA's smem or arriving on its barriers
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(static_cast<uint32_t>(C::kTmemCols)) : "memory");
    }
}

}  // namespace pair
