/*
 * bsi_b200 -- C ABI of the B200 (sm_100a) bit-sliced-index (BSI) tensor-dot library.
 *
 * Plain pointers and sizes only; no torch types. Every pointer is a DEVICE pointer unless
 * the comment says "host". Every function enqueues its work on `stream` (a cudaStream_t)
 * of the CURRENT device and returns without synchronising, unless stated otherwise.
 * The caller owns all memory. Return value: 0 on success, a BSI_ERR_* code otherwise;
 * bsi_b200_last_error() gives the detail of the last failure on the calling thread.
 *
 * Each entry point names the interface of the reference (gguzunsjsu/bsiPytorch, paths
 * relative to its checkout) that it replaces.
 *
 * Layouts (row-major, same as the reference):
 *   words   [rows, S, W]  uint64, W = ceil(D/64); bit t of word w of slice s is bit s of the
 *                         two's-complement value of element 64*w + t (zero beyond D)
 *   scales  [rows, chunks] float32 (chunk mode, chunks = ceil(D/256)) or [rows] (row mode):
 *                         2^shift of each 256-element chunk / each row
 *   q8      [rows, ld8]   int8, the clamped integers, zero padded to ld8 >= 256*chunks
 *   out     [Q, ldo]      float32
 */
#ifndef BSI_B200_H_
#define BSI_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSI_B200_VERSION 100

enum {
    BSI_OK = 0,
    BSI_ERR_INVALID = 1,     /* bad argument (null pointer, negative size, misaligned buffer) */
    BSI_ERR_UNSUPPORTED = 2, /* valid request that this build does not implement */
    BSI_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed */
    BSI_ERR_DEVICE = 4,      /* not an sm_100 device */
    BSI_ERR_TIMEOUT = 5      /* a bounded device-side wait ran out (see bsi_b200_device_status) */
};

/* Input element types; the same codes the reference's launchers use
 * (bsi_vector_cuda.cpp:353-358). */
enum { BSI_DTYPE_F32 = 0, BSI_DTYPE_F16 = 1, BSI_DTYPE_BF16 = 2 };

/* Dot engines. */
enum {
    BSI_ENGINE_AUTO = 0,    /* tcgen05 */
    BSI_ENGINE_TCGEN05 = 1, /* int8 recombination, tcgen05.mma kind::i8, TMEM accumulators, TMA */
    BSI_ENGINE_SIMT = 2,    /* dp4a on the CUDA cores (cross-check engine) */
    BSI_ENGINE_BMMA = 3     /* mma.sync b1 AND+POPC directly on the slice words */
};

typedef void* bsi_stream_t; /* cudaStream_t */

const char* bsi_b200_status_string(int status);
const char* bsi_b200_last_error(void);
int bsi_b200_version(void);

/* Reads (and clears) the device-side status word that kernels set when one of their bounded
 * waits gives up. Synchronises the device. *status_out (host): 0 = clean. */
int bsi_b200_device_status(int* status_out);

/* ---- quantise + bit-slice pack -------------------------------------------------------
 * One pass over x: v = half_away(double(float(x)) * 10^decimal_places); shift from the
 * largest |v| of each 256-element chunk (chunk_mode=1) or each row (chunk_mode=0);
 * q = round-shift, clamp to `bits`-bit two's complement; writes bit slices, 2^shift
 * scales and (optionally) the int8 image. Any of words/scales/shifts/q8 may be NULL.
 *
 * Replaces, for queries (chunk_mode=1): launch_compute_chunk_shift_scale_from_input +
 * launch_quantize_shift_pack_chunk_batch (bsi_cuda_kernels_quant.cuh:524-557, 596-636) and
 * the zero-fill before them (bsi_vector_cuda.cpp:427); for keys and the row-scale mode
 * (chunk_mode=0): launch_quantize_round_to_int64_batch + launch_compute_row_shift_scale +
 * launch_apply_row_shift_clamp + launch_pack_bits_all_ballot_batch
 * (bsi_cuda_kernels_quant.cuh:638-716, bsi_cuda_kernels_pack.cuh:204-230) and
 * launch_compute_row_shift_scale_from_input + launch_quantize_shift_pack_row_batch
 * (bsi_cuda_kernels_quant.cuh:490-522, 559-594).
 *
 * x: [rows, D] with row stride ldx (elements). bits in [2, 8]. ld8: row stride of q8 in
 * bytes (>= 256*ceil(D/256), multiple of 16); columns D..256*ceil(D/256)-1 are written as zero,
 * columns beyond that are left untouched (q8 may be a column block of a wider matrix). */
int bsi_b200_quantize_pack(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx,
                           int decimal_places, int bits, int chunk_mode,
                           uint64_t* words, float* scales, int32_t* shifts,
                           int8_t* q8, int64_t ld8, bsi_stream_t stream);

/* The same with the reference's outlier clipping (BSI_FIXED_CLIP_K, bsi_cuda_kernels_quant.cuh:82-108,
 * bsi_vector_cuda.cpp:295-307): for clip_k > 0 the shift of a group comes from
 * min(max |v|, clip_k * mean |v|), and values beyond the range saturate at the clamp. clip_k <= 0 is
 * bsi_b200_quantize_pack. */
int bsi_b200_quantize_pack_clip(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx,
                                int decimal_places, int bits, int chunk_mode, float clip_k,
                                uint64_t* words, float* scales, int32_t* shifts,
                                int8_t* q8, int64_t ld8, bsi_stream_t stream);

/* The same again with one more optional output for chunk mode: sq_norms [rows, ceil(D/256)] float32, the sum of
 * squares of each chunk's de-shifted integers, (2^shift)^2 * sum a^2 (exact; infinity for a chunk that took the
 * 64-bit fallback). Registered for the int8 image (bsi_b200_register_query_bounds) it lets a dot prove by
 * Cauchy-Schwarz that its float32 chain cannot round. NULL: bsi_b200_quantize_pack_clip. */
int bsi_b200_quantize_pack_norms(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx,
                                 int decimal_places, int bits, int chunk_mode, float clip_k,
                                 uint64_t* words, float* scales, int32_t* shifts,
                                 int8_t* q8, int64_t ld8, float* sq_norms, bsi_stream_t stream);

/* ---- variable-slice mode (the reference's default when no BSI_FIXED_BITS* variable is set) ------
 * The decimal integers v = half_away(double(float(x)) * 10^decimal_places) are sliced as they are,
 * without a shift; the number of slices follows from the largest |v| (bit_width(max|v|) + 2, at least
 * 2; bsi_vector_cuda.cpp:746-754), per batch for queries and per row for keys.
 *
 * bsi_b200_decimal_absmax: row_absmax[r] = max |v| and row_negative[r] = 1 if any v < 0 of row r.
 * Replaces the torch reductions over the int64 tensor in build_bsi_queries_cuda_batch_data
 * (bsi_vector_cuda.cpp:1089-1099, 1156-1159) after launch_quantize_round_to_int64_batch
 * (bsi_cuda_kernels_quant.cuh:638-668). */
int bsi_b200_decimal_absmax(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx,
                            int decimal_places, uint64_t* row_absmax, int32_t* row_negative,
                            bsi_stream_t stream);

/* bsi_b200_pack_plain: words [rows, slices, W] = the low `slices` bits of the two's-complement v (any
 * of words / lo8 may be NULL). lo8 / hi8 [rows, ld8]: v as two signed 8-bit digits for the tensor-core
 * dot, v = 128 * hi + lo, lo in [0, 127] (the caller checks |v| < 2^14 through decimal_absmax); with
 * hi8 == NULL, lo8 receives v itself (|v| <= 127). Columns up to 256*ceil(D/256) are written, zero
 * beyond D. Replaces launch_quantize_round_to_int64_batch + launch_pack_bits_all_ballot[_batch]
 * (bsi_cuda_kernels_quant.cuh:638-668, bsi_cuda_kernels_pack.cuh:176-230). Partial last words rely on
 * zero-initialised `words`, as the reference's packer does. */
int bsi_b200_pack_plain(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx, int decimal_places,
                        int slices, uint64_t* words, int8_t* lo8, int8_t* hi8, int64_t ld8,
                        bsi_stream_t stream);

/* Slice words -> int8 image (sign-extends the top slice). Used when a caller holds only the
 * bit slices (e.g. words built by the reference). No counterpart in the reference, whose dot
 * consumes the slices directly (bsi_cuda_kernels_dot.cuh:1436-1517). */
int bsi_b200_recombine_i8(const uint64_t* words, int64_t rows, int bits, int64_t W,
                          int8_t* q8, int64_t ld8, bsi_stream_t stream);

/* ---- dot core ------------------------------------------------------------------------
 * out[q][r] = ( sum over chunks c, ascending, each step rounded to float32, of
 *               float(I[q][r][c]) * qs[q][c] * bw0[r] ) * scale_inv,
 * I[q][r][c] = sum_{d in chunk c} a8[q][d] * k8[r][d]   (int32, exact; equals the weighted
 * popcount sum over the slice pairs). qs_stride = chunks for chunk scales, 0 for one scale per
 * row. dbg_iacc (optional, [Q, R, chunks] int32) receives I.
 *
 * Replaces launch_popcount_weighted_keys_literal_fused_multiq in its fixed-bit modes
 * (bsi_cuda_kernels_dot.cuh:2616-3090; kernels :1285-1556, :1558-1920, :1922-2307).
 * a8/k8 rows must be 16-byte aligned with lda/ldk multiples of 16 and >= 256*chunks. */
int bsi_b200_dot_i8(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride,
                    const int8_t* k8, int64_t ldk, const float* bw0,
                    int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                    float* out, int64_t ldo, int32_t* dbg_iacc, int engine,
                    bsi_stream_t stream);

/* The dot with the layer epilogue fused in: y[q][r] = cast(out[q][r]) + cast(bias[r]) in y_dtype
 * (BSI_DTYPE_*), where out is exactly what bsi_b200_dot_i8 would produce; both terms are narrowed
 * before the add and the sum is narrowed again, as torch does for `scores.to(dtype) + bias.to(dtype)`.
 * bias may be NULL. Replaces the dot launch plus the two elementwise kernels of
 * BSIQuantizedLinear.forward (bsi_ops/benchmarks/verify_accuracy_bsi.py:177-195): the float32
 * [Q, R] intermediate is never written. */
int bsi_b200_linear_i8(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride,
                       const int8_t* k8, int64_t ldk, const float* bw0, const float* bias,
                       int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                       void* y, int64_t ldy, int y_dtype, bsi_stream_t stream);

/* bsi_b200_linear_i8 with the layer's activation applied to the finished (cast + bias) value before
 * it is stored: BSI_ACT_RELU gives max(y, 0) in y's type, what `F.relu(fc1(x))` of the OPT decoder
 * layer computes (the reference leaves the activation to a separate torch kernel). */
#define BSI_ACT_NONE 0
#define BSI_ACT_RELU 1
int bsi_b200_linear_i8_act(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride,
                           const int8_t* k8, int64_t ldk, const float* bw0, const float* bias,
                           int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                           void* y, int64_t ldy, int y_dtype, int activation, bsi_stream_t stream);

/* ---- tensor-parallel layer: peer memory on one node, one process per GPU -----------------------
 * The reference has no multi-GPU code. These calls carry the exchange of a layer whose BSI linears
 * are sharded along R over the GPUs of one node: packed activations and linear outputs are stored
 * straight into the buffers of the ranks that consume them, over NVLink, with plain stores. */
#define BSI_B200_MAX_PEERS 16
#define BSI_B200_PEER_HANDLE_BYTES 64

/* cudaMalloc'ed, zero-filled buffer other processes of this node can map; handle64 receives the
 * BSI_B200_PEER_HANDLE_BYTES bytes to send them (CUDA IPC). Free with bsi_b200_peer_free. */
int bsi_b200_peer_alloc(int64_t bytes, void** dev_ptr, void* handle64);
int bsi_b200_peer_free(void* dev_ptr);
/* Maps a buffer another process exported (peer access is enabled on first use); close before the
 * owner frees it. */
int bsi_b200_peer_open(const void* handle64, void** peer_ptr);
int bsi_b200_peer_close(void* peer_ptr);

/* Barrier over the n ranks, enqueued on `stream`: flags[r] points at rank r's array of n + 1 uint32
 * (in a peer buffer, zero at start; flags[rank] is the caller's own). Slot n of a rank's own array
 * counts the barriers it has passed, so the launch carries no epoch argument and can be replayed from
 * a captured graph; every rank must run the same sequence of barriers. The kernel first publishes
 * everything this GPU wrote before it on the stream, stores its new count into slot `rank` of every
 * rank's array, then waits until every slot of its own array has reached that count (the comparison
 * survives wrap-around). A wait that exceeds timeout_ms gives up and sets the device status to
 * 64 + the missing rank (bsi_b200_device_status), so a lost rank cannot hang the GPU. */
int bsi_b200_peer_barrier(uint32_t* const* flags, int rank, int n, int64_t timeout_ms, bsi_stream_t stream);

/* Optional bounds for a key image. The chunk terms of the dot, I_c * 2^shift, are integers; while every prefix of
 * their sum stays below 2^24 in magnitude no float32 addition of the reference's chain rounds, and accumulating the
 * terms as int32 gives the same bits with a third of the epilogue's arithmetic. A prefix is bounded by
 * query_abs_max x (largest 2^shift of the query row) x (sum of |k| over key row r) and by query_abs_max x (sum of the
 * row's 2^shift) x (largest sum of |k| over one 256-element chunk of key row r), and, by Cauchy-Schwarz, by the
 * product of the L2 norms of the de-shifted query row and of the key row. With key_abs_sum (device, float32 [3, R]:
 * the R row sums of |k|, the R chunk maxima, the R row sums of k^2) registered for k8, the tensor-core dots that are
 * handed this k8 with this R test the bounds per tile and take the integer route where one holds (the float32 chain
 * elsewhere; results identical either way). The third bound also needs the query side
 * (bsi_b200_register_query_bounds).
 * query_abs_max: largest magnitude of a query integer (64 for 7-bit fixed queries, 128 when unknown). Registering
 * again replaces the entry; unregister before the arrays are freed. BSI_B200_EXACT_INT=0 switches the route off. */
int bsi_b200_register_key_bounds(const int8_t* k8, const float* key_abs_sum, int64_t R, int query_abs_max);
int bsi_b200_unregister_key_bounds(const int8_t* k8);
/* Query side of the Cauchy-Schwarz bound: sq_norms as written by bsi_b200_quantize_pack_norms for the int8 image a8
 * (stride floats per row, one value per chunk). Dots handed this a8 read it until it is unregistered. */
int bsi_b200_register_query_bounds(const int8_t* a8, const float* sq_norms, int64_t stride);
int bsi_b200_unregister_query_bounds(const int8_t* a8);
/* Test hook: number of (warp, tile) pairs of the paired tensor-core kernel that took the integer route since the
 * last call on this device; synchronises and clears the counter. */
int bsi_b200_debug_exact_int_tiles(unsigned long long* count_out);

/* Linear whose finished output is re-quantised for the next linear inside the epilogue, so that the
 * layer-type [Q, R] matrix is never written: y = activation(cast(out) + cast(bias)) in layer_dtype
 * (BSI_DTYPE_F16 / BF16) is what bsi_b200_linear_i8_act would store; here every 256-column chunk of y
 * is quantised as bsi_b200_quantize_pack (chunk mode, `bits`, decimal_places) would quantise it and the
 * int8 image / chunk scales go to n_dst places: q8_dst[i] + q * ld8 + r and
 * scale_dst[i] + q * scale_ld + r / 256 (pointers already offset to this linear's first output column /
 * chunk; own memory or peer mappings). Same integers as the two-kernel sequence. R % 256 == 0,
 * decimal_places in [0, 3]; a chunk holding NaN, inf or |y * 10^dp| >= 2^23 cannot be expressed on this
 * path: it is stored as zeros and the device status is set to 48 (bsi_b200_device_status).
 * OPT: fc1 -> ReLU -> fc2 (the reference runs dot, two elementwise kernels, ReLU and the fc2 packer). */
int bsi_b200_linear_i8_requant(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride,
                               const int8_t* k8, int64_t ldk, const float* bw0, const float* bias,
                               int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                               int layer_dtype, int activation, int decimal_places, int bits,
                               int n_dst, int8_t* const* q8_dst, int64_t ld8,
                               float* const* scale_dst, int64_t scale_ld, bsi_stream_t stream);

/* Chunk-mode quantise + pack of activations (int8 image and chunk scales only) written to several
 * places at once: the int8 image to q8_dst[i] + row * ld8 + col for i < n_q8_dst, the chunk scales to
 * scale_dst[i] + row * scale_ld + chunk for i < n_scale_dst. The pointers already include the column /
 * row offset of this rank's block inside each destination matrix; they may be peer mappings. D must be a
 * multiple of 256, x 16-byte aligned with ldx * sizeof(x) % 16 == 0. */
int bsi_b200_quantize_pack_multi(const void* x, int dtype, int64_t rows, int64_t D, int64_t ldx,
                                 int decimal_places, int bits, int n_q8_dst, int8_t* const* q8_dst,
                                 int64_t ld8, int n_scale_dst, float* const* scale_dst, int64_t scale_ld,
                                 bsi_stream_t stream);

/* Residual add + LayerNorm + activation pack in one pass over a token block, for a 16-bit layer type
 * (dtype BSI_DTYPE_F16 / BF16; x, delta, gamma, beta and x_out all of that type, rows contiguous, H
 * elements each): x_out = x + delta (delta may be NULL; x_out may be x), y = LayerNorm(x_out) with float32
 * statistics, rounded to the layer type, then quantised per 256-element chunk exactly as
 * bsi_b200_quantize_pack (chunk mode) quantises it; the int8 image and chunk scales go to the
 * destinations as in bsi_b200_quantize_pack_multi. Replaces, in the OPT decoder layer, the residual add,
 * the LayerNorm and the packer of the following BSI linears (three passes over the hidden states in the
 * reference's flow: two torch kernels, then the query builder). H % 256 == 0, H <= 16384. */
int bsi_b200_add_layernorm_pack(const void* x, const void* delta, const void* gamma, const void* beta,
                                float eps, int dtype, int64_t rows, int64_t H, void* x_out,
                                int decimal_places, int bits, int n_q8_dst, int8_t* const* q8_dst,
                                int64_t ld8, int n_scale_dst, float* const* scale_dst, int64_t scale_ld,
                                bsi_stream_t stream);

/* bsi_b200_linear_i8_act whose output rows are dealt out to n_dst matrices: row q goes to
 * y_dst[q / rows_per_dst] at local row q % rows_per_dst, column r, leading dimension ldy (the
 * pointers already include this rank's column offset; they may be peer mappings).
 * rows_per_dst must be a multiple of 32 and n_dst * rows_per_dst >= Q. This is the all-to-all that
 * turns the [Q, R/G] output block of a rank back into token shards, done by the epilogue's stores. */
int bsi_b200_linear_i8_scatter(const int8_t* a8, int64_t lda, const float* qs, int64_t qs_stride,
                               const int8_t* k8, int64_t ldk, const float* bw0, const float* bias,
                               int64_t Q, int64_t R, int64_t chunks, float scale_inv,
                               int n_dst, void* const* y_dst, int64_t rows_per_dst, int64_t ldy,
                               int y_dtype, int activation, bsi_stream_t stream);

/* Same result computed from the slice words with mma.sync b1 AND+POPC, argument order of the
 * reference launcher (bsi_cuda_kernels_dot.cuh:2616-2635) minus the tile hints and index
 * arrays. Bw is [R, Sb]; only Bw[r][0] = 2^shift_r enters (the slice weights are +-2^j * Bw[r][0],
 * bsi_vector_cuda.cpp:1148-1157). Requires W % 4 == 0, Sa <= 8, Sb <= 8. */
int bsi_b200_dot_words(const uint64_t* A, const float* qs, int64_t qs_stride, int Sa, int64_t W,
                       const uint64_t* B, const float* Bw, int Sb, int64_t R, int64_t Q,
                       float scale_inv, int64_t ldo, float* out, int32_t* dbg_iacc,
                       bsi_stream_t stream);

/* ---- EWAH / verbatim slice encoder ---------------------------------------------------
 * words [S, W] (S = any number of slices, e.g. rows*bits).
 * flags: p = popcount/(64 W); M = 1 - (1-p)^128 - p^128 (float64); compress = (M <= threshold).
 * Replaces launch_slice_popcount_sum + launch_compress_flags_from_density
 * (bsi_cuda_kernels_ewah.cuh:71-81, 104-115). counts may be NULL. */
int bsi_b200_ewah_flags(const uint64_t* words, int64_t S, int64_t W, double threshold,
                        uint64_t* counts, int32_t* flags, bsi_stream_t stream);

/* Number of uint64 each slice encodes to. Replaces launch_ewah_size (ewah.cuh:164-175). */
int bsi_b200_ewah_size(const uint64_t* words, int64_t S, int64_t W, const int32_t* flags,
                       uint64_t* sizes, bsi_stream_t stream);

/* Exclusive prefix sum of sizes -> off [S]; total (device, 1 element) = sum. Replaces the
 * cumsum glue of bsi_vector_cuda.cpp:929-939. */
int bsi_b200_ewah_offsets(const uint64_t* sizes, int64_t S, uint64_t* off, uint64_t* total,
                          bsi_stream_t stream);

/* Writes [RLW, literals...]* per slice at out + off[s]; out_len[s] = words written.
 * RLW = run_bit | (run_len & 0xFFFFFFFF) << 1 | literal_count << 33.
 * Replaces launch_ewah_emit (ewah.cuh:234-247); identical streams. */
int bsi_b200_ewah_emit(const uint64_t* words, int64_t S, int64_t W, const int32_t* flags,
                       const uint64_t* off, uint64_t* out, int32_t* out_len, bsi_stream_t stream);

/* Decodes S streams (in + off[s], len[s] words) into out [S, W], zero padded.
 * Replaces the per-slice launch_ewah_decompress loop (ewah.cuh:35-42, bsi_cuda.cpp:402-414). */
int bsi_b200_ewah_decode(const uint64_t* in, const uint64_t* off, const int32_t* len,
                         int64_t S, int64_t W, uint64_t* out, bsi_stream_t stream);

/* One call: flags -> sizes -> offsets -> emit. scratch: device buffer of at least
 * bsi_b200_ewah_scratch_bytes(S) bytes. capacity: uint64 slots available at out; a stream that
 * would exceed it is not written and *total (device) still reports the needed size.
 * Replaces build_bsi_vector_from_float_tensor_hybrid's encode half (bsi_vector_cuda.cpp:900-952). */
int64_t bsi_b200_ewah_scratch_bytes(int64_t S);
int bsi_b200_ewah_encode(const uint64_t* words, int64_t S, int64_t W, double threshold,
                         void* scratch, int64_t scratch_bytes,
                         uint64_t* out, int64_t capacity, uint64_t* off, int32_t* out_len,
                         int32_t* flags, uint64_t* total, bsi_stream_t stream);

/* The same encoder for callers that cannot give the library any scratch memory and cannot let it
 * allocate: code hosted inside a process whose memory manager already owns the device, bindings
 * that hold nothing but their inputs and outputs, loops where a cudaMalloc/cudaFree (which
 * serialise the device) is not acceptable. It has no counterpart in the reference, whose builder
 * allocates its temporaries through torch on every call (bsi_vector_cuda.cpp:900-941).
 *
 * The popcounts and sizes live in an array compiled into the library: BSI_B200_EWAH_STATIC_MAX_SLICES
 * slices at most, 1 MiB held on every GPU that loads the library until the process exits. A larger S
 * is refused with BSI_ERR_UNSUPPORTED. The function calls no cudaMalloc, cudaFree or other allocating
 * routine. Its first call on a device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current); make that first call before any stream capture
 * begins. All calls share the one array, so two calls whose kernels may overlap on the GPU (different
 * streams, or different host threads) race on it: order them on one stream or with events. Inputs and
 * outputs are the caller's, exactly as for bsi_b200_ewah_encode. */
#define BSI_B200_EWAH_STATIC_MAX_SLICES 65536
int bsi_b200_ewah_encode_static(const uint64_t* words, int64_t S, int64_t W, double threshold,
                                uint64_t* out, int64_t capacity, uint64_t* off, int32_t* out_len,
                                int32_t* flags, uint64_t* total, bsi_stream_t stream);

/* ---- layer epilogue ------------------------------------------------------------------
 * y[q][r] = cast(out[q][r]) + cast(bias[r]) in y_dtype (BSI_DTYPE_*), one pass.
 * Replaces the two torch elementwise kernels of BSIQuantizedLinear.forward
 * (bsi_ops/benchmarks/verify_accuracy_bsi.py:193-195). bias may be NULL. */
int bsi_b200_cast_bias(const float* out, int64_t ldo, const float* bias, int64_t Q, int64_t R,
                       void* y, int64_t ldy, int y_dtype, bsi_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* BSI_B200_H_ */
