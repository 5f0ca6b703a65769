// EWAH / verbatim slice encoder and decoder.
//
// The reference encodes each slice with ONE thread walking the words in order
// (bsi_cuda_kernels_ewah.cuh:118-162 size, :178-232 emit). The same stream is produced here by
// one WARP per slice with ballots and prefix counts:
//   type(w)     = zero-fill (word == 0), one-fill (word == ~0) or literal; with the compress
//                 flag clear every word is a literal
//   start(w)    = w == 0, or word w is a fill word whose type differs from word w-1
//                 (a segment is: an optional run of one fill word, then literals up to the
//                 next fill word)
//   RLW position of the k-th segment (k from 0) = k + literals before its first word
//   literal w goes to (segments started at or before w) + (literals before w)
//   RLW = run_bit | (run_len & 0xFFFFFFFF) << 1 | literal_count << 33, written when the segment
//   closes (at the next start, or at W).
#include <string.h>

#include <atomic>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace bsi {
namespace {

typedef unsigned long long u64;

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ u64 warp_sum_u64(u64 v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ int compress_flag(u64 count, int64_t W, double threshold) {
    // Same expressions as bsi_cuda_kernels_ewah.cuh:94-101 so that pow() rounds identically.
    const double total_bits = static_cast<double>(W) * 64.0;
    double p = (total_bits > 0.0) ? (static_cast<double>(count) / total_bits) : 0.0;
    if (p < 0.0) p = 0.0;
    if (p > 1.0) p = 1.0;
    const double a = pow(1.0 - p, 128.0);
    const double b = pow(p, 128.0);
    const double M = 1.0 - a - b;
    return (M <= threshold) ? 1 : 0;
}

// Walks one slice with a warp. EMIT=false only counts; EMIT=true also writes the stream.
template <bool EMIT>
__device__ __forceinline__ u64 encode_slice(const u64* __restrict__ base, int64_t W, int compress,
                                            u64* __restrict__ out, int lane) {
    if (!compress) {
        if (EMIT) {
            if (lane == 0) out[0] = static_cast<u64>(W) << 33;
            for (int64_t w = lane; w < W; w += 32) out[1 + w] = base[w];
        }
        return 1ull + static_cast<u64>(W);
    }
    const unsigned below = (1u << lane) - 1u;
    u64 seg_base = 0;  // segments started before this tile
    u64 lit_base = 0;  // literals before this tile
    int prev_type = 2; // type of the last word of the previous tile
    // The open segment (valid once seg_base > 0): first word, literals before it, its fill bit.
    int64_t open_w0 = 0;
    u64 open_lit0 = 0;
    int open_bit = 0;
    int open_isfill = 0;

    for (int64_t tile = 0; tile < W; tile += 32) {
        const int64_t w = tile + lane;
        const bool valid = w < W;
        const u64 word = valid ? base[w] : 1ull;  // padding lanes look like literals, never counted
        const int type = (word == 0ull) ? 0 : ((word == ~0ull) ? 1 : 2);
        int left = __shfl_up_sync(0xffffffffu, type, 1);
        if (lane == 0) left = prev_type;
        const bool start = valid && (w == 0 || (type != 2 && type != left));
        const bool lit = valid && type == 2;
        const unsigned S = __ballot_sync(0xffffffffu, start);
        const unsigned L = __ballot_sync(0xffffffffu, lit);

        if (EMIT) {
            const u64 lit_here = lit_base + __popc(L & below);
            if (lit) {
                const u64 segs_incl = seg_base + __popc(S & (below | (1u << lane)));
                out[segs_incl + lit_here] = word;
            }
            // A start at w (other than the very first word) closes the segment before it.
            const unsigned prior = S & below;
            const int p = prior ? (31 - __clz(prior)) : 0;
            const int p_type = __shfl_sync(0xffffffffu, type, p);
            if (start && w != 0) {
                int64_t w0;
                u64 lit0, pos;
                int bit, isfill;
                if (prior) {
                    w0 = tile + p;
                    lit0 = lit_base + __popc(L & ((1u << p) - 1u));
                    pos = seg_base + __popc(S & ((1u << p) - 1u)) + lit0;
                    bit = (p_type == 1);
                    isfill = (p_type != 2);
                } else {
                    w0 = open_w0;
                    lit0 = open_lit0;
                    pos = (seg_base - 1) + lit0;
                    bit = open_bit;
                    isfill = open_isfill;
                }
                const u64 lit_count = lit_here - lit0;
                const u64 run_len = isfill ? (static_cast<u64>(w - w0) - lit_count) : 0ull;
                out[pos] = static_cast<u64>(bit) | ((run_len & 0xFFFFFFFFull) << 1) | (lit_count << 33);
            }
        }
        // Carry the last start of this tile forward as the open segment.
        if (S) {
            const int p = 31 - __clz(S);
            const int p_type = __shfl_sync(0xffffffffu, type, p);
            open_w0 = tile + p;
            open_lit0 = lit_base + __popc(L & ((1u << p) - 1u));
            open_bit = (p_type == 1);
            open_isfill = (p_type != 2);
        }
        seg_base += __popc(S);
        lit_base += __popc(L);
        const int last = (W - tile) >= 32 ? 31 : static_cast<int>(W - tile - 1);
        prev_type = __shfl_sync(0xffffffffu, type, last);
    }
    if (EMIT && lane == 0 && seg_base > 0) {
        const u64 lit_count = lit_base - open_lit0;
        const u64 run_len = open_isfill ? (static_cast<u64>(W - open_w0) - lit_count) : 0ull;
        out[(seg_base - 1) + open_lit0] =
            static_cast<u64>(open_bit) | ((run_len & 0xFFFFFFFFull) << 1) | (lit_count << 33);
    }
    return seg_base + lit_base;
}

// counts/flags and (optionally) sizes in one pass over the words.
template <bool WITH_SIZE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) ewah_flags_kernel(
    const u64* __restrict__ words, int64_t S, int64_t W, double threshold,
    u64* __restrict__ counts, int32_t* __restrict__ flags, u64* __restrict__ sizes) {
    const int lane = threadIdx.x & 31;
    const int64_t s = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (s >= S) return;
    const u64* base = words + s * W;
    u64 local = 0;
    for (int64_t w = lane; w < W; w += 32) local += static_cast<u64>(__popcll(base[w]));
    const u64 count = warp_sum_u64(local);
    const int flag = compress_flag(count, W, threshold);
    if (lane == 0) {
        if (counts != nullptr) counts[s] = count;
        flags[s] = flag;
    }
    if (WITH_SIZE) {
        const u64 n = encode_slice<false>(base, W, flag, nullptr, lane);
        if (lane == 0) sizes[s] = n;
    }
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32) ewah_size_kernel(
    const u64* __restrict__ words, int64_t S, int64_t W, const int32_t* __restrict__ flags,
    u64* __restrict__ sizes) {
    const int lane = threadIdx.x & 31;
    const int64_t s = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (s >= S) return;
    const u64 n = encode_slice<false>(words + s * W, W, flags[s], nullptr, lane);
    if (lane == 0) sizes[s] = n;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32) ewah_emit_kernel(
    const u64* __restrict__ words, int64_t S, int64_t W, const int32_t* __restrict__ flags,
    const u64* __restrict__ off, const u64* __restrict__ sizes, u64 capacity,
    u64* __restrict__ out, int32_t* __restrict__ out_len) {
    const int lane = threadIdx.x & 31;
    const int64_t s = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (s >= S) return;
    const u64 o = off[s];
    if (sizes != nullptr && o + sizes[s] > capacity) {
        if (lane == 0) out_len[s] = static_cast<int32_t>(sizes[s]);
        return;
    }
    const u64 n = encode_slice<true>(words + s * W, W, flags[s], out + o, lane);
    if (lane == 0) out_len[s] = static_cast<int32_t>(n);
}

// Exclusive prefix sum with one block; S is at most a few hundred thousand slices. Every thread owns
// kScanItems consecutive sizes per tile (all of its loads are in flight together, and the next tile's are
// issued before the current tile is scanned), so a tile of 8192 slices costs one round of block barriers.
constexpr int kScanItems = 8;
__device__ __forceinline__ void exclusive_scan_block(const u64* __restrict__ sizes, int64_t S,
                                                     u64* __restrict__ off, u64* __restrict__ total) {
    __shared__ u64 warp_tot[32];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    constexpr int64_t kTile = 1024 * kScanItems;
    u64 carry = 0;   // sum of all earlier tiles, kept by every thread
    u64 v[kScanItems], nxt[kScanItems];
    auto load = [&](int64_t tile, u64 (&dst)[kScanItems]) {
        const int64_t base = tile + static_cast<int64_t>(threadIdx.x) * kScanItems;
#pragma unroll
        for (int k = 0; k < kScanItems; ++k) dst[k] = (base + k < S) ? sizes[base + k] : 0ull;
    };
    load(0, v);
    for (int64_t tile = 0; tile < S; tile += kTile) {
        if (tile + kTile < S) load(tile + kTile, nxt);
        u64 local = 0;
#pragma unroll
        for (int k = 0; k < kScanItems; ++k) local += v[k];
        u64 incl = local;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const u64 t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            u64 t = warp_tot[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const u64 u = __shfl_up_sync(0xffffffffu, t, d);
                if (lane >= d) t += u;
            }
            warp_tot[lane] = t;
        }
        __syncthreads();
        u64 run = carry + (warp ? warp_tot[warp - 1] : 0ull) + (incl - local);
        const int64_t base = tile + static_cast<int64_t>(threadIdx.x) * kScanItems;
#pragma unroll
        for (int k = 0; k < kScanItems; ++k) {
            if (base + k < S) off[base + k] = run;
            run += v[k];
        }
        carry += warp_tot[31];
        __syncthreads();   // warp_tot is rewritten by the next tile
#pragma unroll
        for (int k = 0; k < kScanItems; ++k) v[k] = nxt[k];
    }
    if (threadIdx.x == 0 && total != nullptr) *total = carry;
}

__global__ void __launch_bounds__(1024) ewah_offsets_kernel(const u64* __restrict__ sizes, int64_t S,
                                                            u64* __restrict__ off,
                                                            u64* __restrict__ total) {
    exclusive_scan_block(sizes, S, off, total);
}

// The same scan as the middle kernel of the one-call encoder, launched as a programmatic dependent of the sizes
// pass: it lets the emit pass start (whose blocks first load their slices, which depend on nothing), then waits
// for the sizes pass to be complete.
__global__ void __launch_bounds__(1024) ewah_block_offsets_kernel(const u64* __restrict__ sums, int64_t n,
                                                                  u64* __restrict__ off, u64* __restrict__ total) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    exclusive_scan_block(sums, n, off, total);
}

// Decode: lane 0 parses the RLWs in order (bsi_cuda_kernels_ewah.cuh:16-32), the warp fills runs
// and copies literals together.
__global__ void __launch_bounds__(kWarpsPerBlock * 32) ewah_decode_kernel(
    const u64* __restrict__ in, const u64* __restrict__ off, const int32_t* __restrict__ len,
    int64_t S, int64_t W, u64* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t s = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (s >= S) return;
    const u64* src = in + off[s];
    const int64_t in_len = len[s];
    u64* dst = out + s * W;
    int64_t idx = 0, o = 0;
    while (idx < in_len && o < W) {
        const u64 rlw = src[idx++];
        const u64 run_val = (rlw & 1ull) ? ~0ull : 0ull;
        int64_t run_len = static_cast<int64_t>((rlw >> 1) & 0xFFFFFFFFull);
        int64_t lit = static_cast<int64_t>(rlw >> 33);
        if (run_len > W - o) run_len = W - o;
        for (int64_t k = lane; k < run_len; k += 32) dst[o + k] = run_val;
        o += run_len;
        if (lit > W - o) lit = W - o;
        if (lit > in_len - idx) lit = in_len - idx;
        for (int64_t k = lane; k < lit; k += 32) dst[o + k] = src[idx + k];
        o += lit;
        idx += lit;
    }
    for (int64_t k = o + lane; k < W; k += 32) dst[k] = 0ull;
}

// ---- the one-call encoder's own kernels -----------------------------------------------------------
// Slices of up to 256 words (8 words per lane) are held in registers: every load of a slice is in flight at once,
// the popcount and the size walk share one read, and the walk itself never waits for memory.
//
// The compress flag depends on the slice only through its popcount, and for one (W, threshold) the reference's
// float64 expression is evaluated for every possible count once (ewah_cuts_kernel, same compress_flag, hence the
// same roundings) and summarised by the host as "flag = count < first_zero or count > last_zero" when the flags
// have that shape; the per-slice kernels then compare two integers instead of calling pow() twice.
struct FlagCuts {
    long long first_zero;   // smallest count whose flag is 0 (64 W + 1 if none)
    long long last_zero;    // largest count whose flag is 0 (-1 if none)
    int regular;            // 1: every count in [first_zero, last_zero] has flag 0, so the two bounds decide
};

__global__ void __launch_bounds__(1024) ewah_cuts_kernel(int64_t W, double threshold, long long* __restrict__ result) {
    __shared__ long long s_first, s_last, s_zeros;
    if (threadIdx.x == 0) {
        s_first = 64 * W + 1;
        s_last = -1;
        s_zeros = 0;
    }
    __syncthreads();
    long long first = 64 * W + 1, last = -1, zeros = 0;
    for (long long c = threadIdx.x; c <= 64 * W; c += blockDim.x) {
        if (!compress_flag(static_cast<u64>(c), W, threshold)) {
            first = c < first ? c : first;
            last = c > last ? c : last;
            ++zeros;
        }
    }
    atomicMin(&s_first, first);
    atomicMax(&s_last, last);
    atomicAdd(reinterpret_cast<unsigned long long*>(&s_zeros), static_cast<unsigned long long>(zeros));
    __syncthreads();
    if (threadIdx.x == 0) {
        result[0] = s_first;
        result[1] = s_last;
        result[2] = (s_last < 0 || s_zeros == s_last - s_first + 1) ? 1 : 0;
    }
}

__device__ __forceinline__ int flag_from(u64 count, int64_t W, double threshold, const FlagCuts& cuts) {
    if (cuts.regular) {
        const long long c = static_cast<long long>(count);
        return (c < cuts.first_zero || c > cuts.last_zero) ? 1 : 0;
    }
    return compress_flag(count, W, threshold);
}

// encode_slice on a slice held in registers: wv[t] is this lane's word of tile t (word index 32 t + lane).
template <bool EMIT, int TILES>
__device__ __forceinline__ u64 encode_slice_regs(const u64 (&wv)[TILES], int64_t W, int compress,
                                                 u64* __restrict__ out, int lane) {
    if (!compress) {
        if (EMIT) {
            if (lane == 0) out[0] = static_cast<u64>(W) << 33;
#pragma unroll
            for (int t = 0; t < TILES; ++t) {
                const int64_t w = t * 32 + lane;
                if (w < W) out[1 + w] = wv[t];
            }
        }
        return 1ull + static_cast<u64>(W);
    }
    const unsigned below = (1u << lane) - 1u;
    u64 seg_base = 0, lit_base = 0;
    int prev_type = 2;
    int64_t open_w0 = 0;
    u64 open_lit0 = 0;
    int open_bit = 0, open_isfill = 0;
#pragma unroll
    for (int t = 0; t < TILES; ++t) {
        const int64_t tile = t * 32;
        if (tile < W) {
            const int64_t w = tile + lane;
            const bool valid = w < W;
            const u64 word = valid ? wv[t] : 1ull;
            const int type = (word == 0ull) ? 0 : ((word == ~0ull) ? 1 : 2);
            int left = __shfl_up_sync(0xffffffffu, type, 1);
            if (lane == 0) left = prev_type;
            const bool start = valid && (w == 0 || (type != 2 && type != left));
            const bool lit = valid && type == 2;
            const unsigned S = __ballot_sync(0xffffffffu, start);
            const unsigned L = __ballot_sync(0xffffffffu, lit);
            if (EMIT) {
                const u64 lit_here = lit_base + __popc(L & below);
                if (lit) {
                    const u64 segs_incl = seg_base + __popc(S & (below | (1u << lane)));
                    out[segs_incl + lit_here] = word;
                }
                const unsigned prior = S & below;
                const int p = prior ? (31 - __clz(prior)) : 0;
                const int p_type = __shfl_sync(0xffffffffu, type, p);
                if (start && w != 0) {
                    int64_t w0;
                    u64 lit0, pos;
                    int bit, isfill;
                    if (prior) {
                        w0 = tile + p;
                        lit0 = lit_base + __popc(L & ((1u << p) - 1u));
                        pos = seg_base + __popc(S & ((1u << p) - 1u)) + lit0;
                        bit = (p_type == 1);
                        isfill = (p_type != 2);
                    } else {
                        w0 = open_w0;
                        lit0 = open_lit0;
                        pos = (seg_base - 1) + lit0;
                        bit = open_bit;
                        isfill = open_isfill;
                    }
                    const u64 lit_count = lit_here - lit0;
                    const u64 run_len = isfill ? (static_cast<u64>(w - w0) - lit_count) : 0ull;
                    out[pos] = static_cast<u64>(bit) | ((run_len & 0xFFFFFFFFull) << 1) | (lit_count << 33);
                }
            }
            if (S) {
                const int p = 31 - __clz(S);
                const int p_type = __shfl_sync(0xffffffffu, type, p);
                open_w0 = tile + p;
                open_lit0 = lit_base + __popc(L & ((1u << p) - 1u));
                open_bit = (p_type == 1);
                open_isfill = (p_type != 2);
            }
            seg_base += __popc(S);
            lit_base += __popc(L);
            const int last = (W - tile) >= 32 ? 31 : static_cast<int>(W - tile - 1);
            prev_type = __shfl_sync(0xffffffffu, type, last);
        }
    }
    if (EMIT && lane == 0 && seg_base > 0) {
        const u64 lit_count = lit_base - open_lit0;
        const u64 run_len = open_isfill ? (static_cast<u64>(W - open_w0) - lit_count) : 0ull;
        out[(seg_base - 1) + open_lit0] =
            static_cast<u64>(open_bit) | ((run_len & 0xFFFFFFFFull) << 1) | (lit_count << 33);
    }
    return seg_base + lit_base;
}

template <int TILES>
__device__ __forceinline__ void load_slice(const u64* __restrict__ base, int64_t W, int lane, u64 (&wv)[TILES]) {
#pragma unroll
    for (int t = 0; t < TILES; ++t) {
        const int64_t w = t * 32 + lane;
        wv[t] = w < W ? __ldg(base + w) : 0ull;
    }
}

// Pass 1: flag and encoded size of every slice, and the sum of the sizes of each block's 8 slices.
// TILES = 0 walks the slice in memory (W > 256).
template <int TILES>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) ewah_sizes_kernel(
    const u64* __restrict__ words, int64_t S, int64_t W, double threshold, const FlagCuts cuts,
    int32_t* __restrict__ flags, u64* __restrict__ sizes, u64* __restrict__ block_sums) {
    __shared__ u64 wsize[kWarpsPerBlock];
    // the scan and the emit pass are launched as programmatic dependents: once every block of this grid runs,
    // theirs may be scheduled into SMs that fall idle (they wait for this grid's results where they need them)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t s = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
    u64 n = 0;
    if (s < S) {
        const u64* base = words + s * W;
        u64 local = 0;
        int flag;
        if constexpr (TILES > 0) {
            u64 wv[TILES];
            load_slice<TILES>(base, W, lane, wv);
#pragma unroll
            for (int t = 0; t < TILES; ++t) local += static_cast<u64>(__popcll(wv[t]));
            flag = flag_from(warp_sum_u64(local), W, threshold, cuts);
            n = encode_slice_regs<false, TILES>(wv, W, flag, nullptr, lane);
        } else {
            for (int64_t w = lane; w < W; w += 32) local += static_cast<u64>(__popcll(base[w]));
            flag = flag_from(warp_sum_u64(local), W, threshold, cuts);
            n = encode_slice<false>(base, W, flag, nullptr, lane);
        }
        if (lane == 0) {
            flags[s] = flag;
            sizes[s] = n;
        }
    }
    if (lane == 0) wsize[warp] = n;
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 t = 0;
#pragma unroll
        for (int w = 0; w < kWarpsPerBlock; ++w) t += wsize[w];
        block_sums[blockIdx.x] = t;
    }
}

// Pass 3: offsets of the block's slices from the scanned block sums, then the streams.
template <int TILES>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) ewah_emit_blocks_kernel(
    const u64* __restrict__ words, int64_t S, int64_t W, const int32_t* __restrict__ flags,
    const u64* __restrict__ sizes, const u64* __restrict__ block_off, u64 capacity,
    u64* __restrict__ off, u64* __restrict__ out, int32_t* __restrict__ out_len) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t s0 = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock;
    const int64_t s = s0 + warp;
    // The slice itself is input of the whole call: it is loaded before the wait for the two passes before this one
    // (programmatic dependent launch), so that this read overlaps their tail and the scan.
    u64 wv[TILES > 0 ? TILES : 1];
    if constexpr (TILES > 0) {
        if (s < S) load_slice<TILES>(words + s * W, W, lane, wv);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // every warp adds up the sizes of the block's slices before its own
    u64 mine = (lane < kWarpsPerBlock && s0 + lane < S) ? sizes[s0 + lane] : 0ull;
    u64 before = (lane < warp) ? mine : 0ull;
    before = warp_sum_u64(before);
    if (s >= S) return;
    const u64 o = block_off[blockIdx.x] + before;
    const u64 n_expected = __shfl_sync(0xffffffffu, mine, warp);
    if (lane == 0) off[s] = o;
    if (o + n_expected > capacity) {
        if (lane == 0) out_len[s] = static_cast<int32_t>(n_expected);
        return;
    }
    u64 n;
    if constexpr (TILES > 0) {
        n = encode_slice_regs<true, TILES>(wv, W, flags[s], out + o, lane);
    } else {
        n = encode_slice<true>(words + s * W, W, flags[s], out + o, lane);
    }
    if (lane == 0) out_len[s] = static_cast<int32_t>(n);
}

// Launch as a programmatic dependent of the kernel before it in the stream: the kernel may start while that one
// drains and must execute griddepcontrol.wait before it reads what earlier kernels of the stream wrote.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), unsigned grid, unsigned block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline unsigned warp_blocks(int64_t S) { return static_cast<unsigned>((S + kWarpsPerBlock - 1) / kWarpsPerBlock); }

int check_sw(const char* name, const void* words, int64_t S, int64_t W) {
    if (S < 0 || W <= 0) {
        set_error("%s: bad S/W", name);
        return BSI_ERR_INVALID;
    }
    if (S > 0 && words == nullptr) {
        set_error("%s: words is null", name);
        return BSI_ERR_INVALID;
    }
    if ((S + kWarpsPerBlock - 1) / kWarpsPerBlock > 0x7fffffffll) {
        set_error("%s: too many slices for one launch", name);
        return BSI_ERR_UNSUPPORTED;
    }
    return require_sm100();
}

}  // namespace
}  // namespace bsi

using bsi::u64;

extern "C" int bsi_b200_ewah_flags(const uint64_t* words, int64_t S, int64_t W, double threshold,
                                   uint64_t* counts, int32_t* flags, bsi_stream_t stream_) {
    using namespace bsi;
    if (int rc = check_sw("ewah_flags", words, S, W)) return rc;
    if (S == 0) return BSI_OK;
    if (flags == nullptr) return fail(BSI_ERR_INVALID, "ewah_flags: flags is null");
    ewah_flags_kernel<false><<<warp_blocks(S), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream_)>>>(
        reinterpret_cast<const u64*>(words), S, W, threshold, reinterpret_cast<u64*>(counts), flags, nullptr);
    return check_launch("ewah_flags launch");
}

extern "C" int bsi_b200_ewah_size(const uint64_t* words, int64_t S, int64_t W, const int32_t* flags,
                                  uint64_t* sizes, bsi_stream_t stream_) {
    using namespace bsi;
    if (int rc = check_sw("ewah_size", words, S, W)) return rc;
    if (S == 0) return BSI_OK;
    if (flags == nullptr || sizes == nullptr) return fail(BSI_ERR_INVALID, "ewah_size: null pointer");
    ewah_size_kernel<<<warp_blocks(S), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream_)>>>(
        reinterpret_cast<const u64*>(words), S, W, flags, reinterpret_cast<u64*>(sizes));
    return check_launch("ewah_size launch");
}

extern "C" int bsi_b200_ewah_offsets(const uint64_t* sizes, int64_t S, uint64_t* off, uint64_t* total,
                                     bsi_stream_t stream_) {
    using namespace bsi;
    if (S < 0) return fail(BSI_ERR_INVALID, "ewah_offsets: bad S");
    if (S > 0 && (sizes == nullptr || off == nullptr)) return fail(BSI_ERR_INVALID, "ewah_offsets: null pointer");
    if (int rc = require_sm100()) return rc;
    ewah_offsets_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream_)>>>(
        reinterpret_cast<const u64*>(sizes), S, reinterpret_cast<u64*>(off), reinterpret_cast<u64*>(total));
    return check_launch("ewah_offsets launch");
}

extern "C" int bsi_b200_ewah_emit(const uint64_t* words, int64_t S, int64_t W, const int32_t* flags,
                                  const uint64_t* off, uint64_t* out, int32_t* out_len,
                                  bsi_stream_t stream_) {
    using namespace bsi;
    if (int rc = check_sw("ewah_emit", words, S, W)) return rc;
    if (S == 0) return BSI_OK;
    if (flags == nullptr || off == nullptr || out == nullptr || out_len == nullptr)
        return fail(BSI_ERR_INVALID, "ewah_emit: null pointer");
    ewah_emit_kernel<<<warp_blocks(S), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream_)>>>(
        reinterpret_cast<const u64*>(words), S, W, flags, reinterpret_cast<const u64*>(off), nullptr, 0ull,
        reinterpret_cast<u64*>(out), out_len);
    return check_launch("ewah_emit launch");
}

extern "C" int bsi_b200_ewah_decode(const uint64_t* in, const uint64_t* off, const int32_t* len,
                                    int64_t S, int64_t W, uint64_t* out, bsi_stream_t stream_) {
    using namespace bsi;
    if (int rc = check_sw("ewah_decode", in, S, W)) return rc;
    if (S == 0) return BSI_OK;
    if (off == nullptr || len == nullptr || out == nullptr) return fail(BSI_ERR_INVALID, "ewah_decode: null pointer");
    ewah_decode_kernel<<<warp_blocks(S), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream_)>>>(
        reinterpret_cast<const u64*>(in), reinterpret_cast<const u64*>(off), len, S, W,
        reinterpret_cast<u64*>(out));
    return check_launch("ewah_decode launch");
}

extern "C" int64_t bsi_b200_ewah_scratch_bytes(int64_t S) {
    // sizes [S], block sums and block offsets [ceil(S / 8)] each, 3 words for the flag bounds; rounded up generously
    return S < 0 ? 0 : (2 * S + 16) * static_cast<int64_t>(sizeof(uint64_t));
}

namespace bsi {
namespace {

// Flag bounds of one (W, threshold), computed on the device with the reference's expression the first time the pair
// is seen and kept on the host afterwards. That first time synchronises the stream (the three numbers come back to
// the host); while a stream is being captured nothing is cached and the kernels evaluate the expression per slice.
int flag_cuts(int64_t W, double threshold, u64* scratch3, cudaStream_t stream, FlagCuts* out) {
    struct Entry { int64_t W; double thr; FlagCuts cuts; };
    static std::mutex mu;
    static std::vector<Entry> cache;
    out->first_zero = 0;
    out->last_zero = -1;
    out->regular = 0;     // "irregular": evaluate per slice
    {
        std::lock_guard<std::mutex> lock(mu);
        for (const Entry& e : cache)
            if (e.W == W && memcmp(&e.thr, &threshold, sizeof(double)) == 0) {
                *out = e.cuts;
                return BSI_OK;
            }
    }
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        (void)cudaGetLastError();
        return BSI_OK;
    }
    ewah_cuts_kernel<<<1, 1024, 0, stream>>>(W, threshold, reinterpret_cast<long long*>(scratch3));
    if (int rc = check_launch("ewah_encode flag bounds launch")) return rc;
    long long h[3] = {0, -1, 0};
    BSI_CUDA_TRY(cudaMemcpyAsync(h, scratch3, sizeof(h), cudaMemcpyDeviceToHost, stream));
    BSI_CUDA_TRY(cudaStreamSynchronize(stream));
    FlagCuts c;
    c.first_zero = h[0];
    c.last_zero = h[1];
    c.regular = static_cast<int>(h[2]);
    *out = c;
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() < 64) cache.push_back(Entry{W, threshold, c});
    return BSI_OK;
}

}  // namespace
}  // namespace bsi

extern "C" int bsi_b200_ewah_encode(const uint64_t* words, int64_t S, int64_t W, double threshold,
                                    void* scratch, int64_t scratch_bytes,
                                    uint64_t* out, int64_t capacity, uint64_t* off, int32_t* out_len,
                                    int32_t* flags, uint64_t* total, bsi_stream_t stream_) {
    using namespace bsi;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (int rc = check_sw("ewah_encode", words, S, W)) return rc;
    if (S == 0) return BSI_OK;
    if (scratch == nullptr || scratch_bytes < bsi_b200_ewah_scratch_bytes(S) ||
        (reinterpret_cast<uintptr_t>(scratch) & 7) != 0)
        return fail(BSI_ERR_INVALID, "ewah_encode: scratch too small or misaligned");
    if (out == nullptr || off == nullptr || out_len == nullptr || flags == nullptr || capacity < 0)
        return fail(BSI_ERR_INVALID, "ewah_encode: null pointer");
    const int64_t nb = (S + kWarpsPerBlock - 1) / kWarpsPerBlock;
    u64* sizes = static_cast<u64*>(scratch);
    u64* block_sums = sizes + S;
    u64* block_off = block_sums + nb;
    u64* cut_words = block_off + nb;
    FlagCuts cuts;
    if (int rc = flag_cuts(W, threshold, cut_words, stream, &cuts)) return rc;
    const u64* w64 = reinterpret_cast<const u64*>(words);
    const unsigned grid = warp_blocks(S);
#define BSI_EWAH_SIZES(T) ewah_sizes_kernel<T><<<grid, kWarpsPerBlock * 32, 0, stream>>>(w64, S, W, threshold, cuts, flags, sizes, block_sums)
    if (W <= 32) BSI_EWAH_SIZES(1);
    else if (W <= 64) BSI_EWAH_SIZES(2);
    else if (W <= 128) BSI_EWAH_SIZES(4);
    else if (W <= 256) BSI_EWAH_SIZES(8);
    else BSI_EWAH_SIZES(0);
#undef BSI_EWAH_SIZES
    if (int rc = check_launch("ewah_encode sizes launch")) return rc;
    BSI_CUDA_TRY(launch_dependent(ewah_block_offsets_kernel, 1u, 1024u, stream, static_cast<const u64*>(block_sums), nb,
                                  block_off, reinterpret_cast<u64*>(total)));
    if (int rc = check_launch("ewah_encode offsets launch")) return rc;
#define BSI_EWAH_EMIT(T) BSI_CUDA_TRY(launch_dependent(ewah_emit_blocks_kernel<T>, grid, kWarpsPerBlock * 32u, stream, \
        w64, S, W, static_cast<const int32_t*>(flags), static_cast<const u64*>(sizes),                                \
        static_cast<const u64*>(block_off), static_cast<u64>(capacity), reinterpret_cast<u64*>(off),                  \
        reinterpret_cast<u64*>(out), out_len))
    if (W <= 32) BSI_EWAH_EMIT(1);
    else if (W <= 64) BSI_EWAH_EMIT(2);
    else if (W <= 128) BSI_EWAH_EMIT(4);
    else if (W <= 256) BSI_EWAH_EMIT(8);
    else BSI_EWAH_EMIT(0);
#undef BSI_EWAH_EMIT
    return check_launch("ewah_encode emit launch");
}

// ---- allocation-free variant ----------------------------------------------------------------------
// Same pipeline as bsi_b200_ewah_encode, for hosts that have no way to hand us scratch memory:
// a plugin living inside a process whose own memory manager has already claimed the device, a
// language binding (cgo, JNI, ctypes) that only owns its input and output buffers, or a serving
// loop that must not call cudaMalloc/cudaFree because those serialise the whole device. The
// per-slice popcounts and stream sizes, which the regular entry point keeps in caller-provided
// scratch, live in one fixed array inside the library image instead. Every GPU that loads the
// library carries this array until the process exits, which is why it is kept small: room for
// BSI_B200_EWAH_STATIC_MAX_SLICES slices (2 x 8 bytes each = 1 MiB).
static __device__ __align__(256) unsigned long long g_ewah_static_scratch[2 * BSI_B200_EWAH_STATIC_MAX_SLICES];

namespace bsi {
namespace {

// On the host the array's name is only a handle for the runtime, not a device address; the address
// that kernels may dereference is looked up once per device, with that device current.
int static_scratch_address(u64** out) {
    // one slot per device; host threads that race on a first call store the same address, hence relaxed atomics
    static std::atomic<u64*> cached[64];
    int dev = 0;
    BSI_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        void* p = nullptr;
        BSI_CUDA_TRY(cudaGetSymbolAddress(&p, g_ewah_static_scratch));
        *out = static_cast<u64*>(p);
        return BSI_OK;
    }
    u64* addr = cached[dev].load(std::memory_order_relaxed);
    if (addr == nullptr) {
        void* p = nullptr;
        BSI_CUDA_TRY(cudaGetSymbolAddress(&p, g_ewah_static_scratch));
        if (p == nullptr) return fail(BSI_ERR_CUDA, "ewah_encode_static: cudaGetSymbolAddress returned null");
        addr = static_cast<u64*>(p);
        cached[dev].store(addr, std::memory_order_relaxed);
    }
    *out = addr;
    return BSI_OK;
}

}  // namespace
}  // namespace bsi

extern "C" int bsi_b200_ewah_encode_static(const uint64_t* words, int64_t S, int64_t W, double threshold,
                                           uint64_t* out, int64_t capacity, uint64_t* off, int32_t* out_len,
                                           int32_t* flags, uint64_t* total, bsi_stream_t stream_) {
    using namespace bsi;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (S > BSI_B200_EWAH_STATIC_MAX_SLICES) {
        set_error("ewah_encode_static: S = %lld exceeds the built-in scratch of %d slices; "
                  "use bsi_b200_ewah_encode with caller-provided scratch",
                  static_cast<long long>(S), BSI_B200_EWAH_STATIC_MAX_SLICES);
        return BSI_ERR_UNSUPPORTED;
    }
    if (int rc = check_sw("ewah_encode_static", words, S, W)) return rc;
    if (S == 0) return BSI_OK;
    if (out == nullptr || off == nullptr || out_len == nullptr || flags == nullptr || capacity < 0)
        return fail(BSI_ERR_INVALID, "ewah_encode_static: null pointer");
    u64* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    // Nothing in the scratch has to start at zero: the first kernel writes counts[s] and sizes[s]
    // for every s < S before anything reads them, so leftovers of an earlier call are never seen.
    u64* counts = scratch;
    u64* sizes = scratch + BSI_B200_EWAH_STATIC_MAX_SLICES;
    ewah_flags_kernel<true><<<warp_blocks(S), kWarpsPerBlock * 32, 0, stream>>>(
        reinterpret_cast<const u64*>(words), S, W, threshold, counts, flags, sizes);
    if (int rc = check_launch("ewah_encode_static flags launch")) return rc;
    ewah_offsets_kernel<<<1, 1024, 0, stream>>>(sizes, S, reinterpret_cast<u64*>(off),
                                               reinterpret_cast<u64*>(total));
    if (int rc = check_launch("ewah_encode_static offsets launch")) return rc;
    ewah_emit_kernel<<<warp_blocks(S), kWarpsPerBlock * 32, 0, stream>>>(
        reinterpret_cast<const u64*>(words), S, W, flags, reinterpret_cast<const u64*>(off), sizes,
        static_cast<u64>(capacity), reinterpret_cast<u64*>(out), out_len);
    return check_launch("ewah_encode_static emit launch");
}
