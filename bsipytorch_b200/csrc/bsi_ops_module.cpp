// pybind11 module `bsi_ops`: the reference's CUDA entry points (bsi_ops/csrc/cuda/bsi_cuda.cpp:
// 1010-1078) with the same names, argument order, defaults, return tuples and capsule names, on
// top of the bsi_b200 C ABI. Host logic only: tensors are allocated here, every kernel lives in
// libbsi_b200.so.
//
// Modes: the fixed-bit block-floating path of the reference (queries BSI_FIXED_BITS_QUERIES bits,
// default 7, with per-256-element chunk scales when BSI_FIXED_CHUNK_SCALE != 0, default on; keys
// BSI_FIXED_BITS_KEYS bits, default 6, per-row scale). The reference needs those variables to be
// set to reach this path (its README's fixed76 recipe); here they are the defaults. Setting a
// variable to 0 selects the reference's variable-slice mode for that side: the decimal integers
// are sliced without a shift and the slice count follows from the data (pack_variable below).
#include <torch/extension.h>
#include <pybind11/stl.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "bsi_b200.h"

namespace py = pybind11;

namespace {

// ---- environment (bsi_vector_cuda.cpp:254-358, bsi_cuda.cpp:108-143) ----------------------------
int env_int(const char* name, int fallback) {
    const char* s = std::getenv(name);
    return s ? std::atoi(s) : fallback;
}

int fixed_bits(const char* specific, int fallback) {
    int v = fallback;
    if (const char* s = std::getenv(specific)) v = std::atoi(s);
    else if (const char* g = std::getenv("BSI_FIXED_BITS")) v = std::atoi(g);
    TORCH_CHECK(v == 0 || (v >= 2 && v <= 8), specific, " must be 0 (variable-slice mode) or in [2, 8], got ", v);
    return v;
}
int bits_queries() { return fixed_bits("BSI_FIXED_BITS_QUERIES", 7); }
int bits_keys() { return fixed_bits("BSI_FIXED_BITS_KEYS", 6); }
bool chunk_scale_enabled() { return env_int("BSI_FIXED_CHUNK_SCALE", 1) != 0; }
bool profile_enabled() { return env_int("BSI_PROFILE", 0) != 0; }
// BSI_FIXED_CLIP_K (bsi_vector_cuda.cpp:295-307): > 0 caps the magnitude that selects a group's shift at
// clip_k * mean |v|. The reference reads it once per process; here it is read per call like the other switches.
float clip_k_from_env() {
    const char* s = std::getenv("BSI_FIXED_CLIP_K");
    const float v = s ? std::strtof(s, nullptr) : 0.0f;
    return v > 0.0f ? v : 0.0f;
}
// The builders honour the variable; the fused additions below (single-call layer, packers that write into
// exchange buffers, re-quantising epilogue) have no clipping variant and refuse to run with it.
void check_clip(const char* what) {
    TORCH_CHECK(!(clip_k_from_env() > 0.0f), what, " does not implement BSI_FIXED_CLIP_K > 0 (outlier clipping); "
                "use the build_bsi_* entry points");
}
int engine_from_env() {
    const char* s = std::getenv("BSI_B200_ENGINE");
    if (!s || !*s || std::string(s) == "auto") {
        // BSI_TC_DOT=0 is the reference's switch to its non-tensor-core kernel, re-read on every launch
        // (bsi_cuda_kernels_dot.cuh:2642); here it selects the CUDA-core (dp4a) engine, which evaluates the
        // same recurrence, so verify_tc_dot_correctness.py compares two engines as it does in the reference.
        const char* tc = std::getenv("BSI_TC_DOT");
        if (tc && *tc && std::atoi(tc) == 0) return BSI_ENGINE_SIMT;
        return BSI_ENGINE_AUTO;
    }
    const std::string v(s);
    if (v == "tcgen05") return BSI_ENGINE_TCGEN05;
    if (v == "simt") return BSI_ENGINE_SIMT;
    if (v == "bmma") return BSI_ENGINE_BMMA;
    if (v.rfind("tcgen05:", 0) == 0) return 1000 + std::atoi(v.c_str() + 8);  // pinned tile width
    TORCH_CHECK(false, "BSI_B200_ENGINE must be auto, tcgen05, tcgen05:<64|128|256>, simt or bmma");
}

void check_status(int rc, const char* what) {
    TORCH_CHECK(rc == BSI_OK, what, " failed: ", bsi_b200_status_string(rc), " (", bsi_b200_last_error(), ")");
}

bsi_stream_t current_stream() { return static_cast<bsi_stream_t>(at::cuda::getCurrentCUDAStream().stream()); }

int dtype_code(const at::Tensor& t) {
    if (t.scalar_type() == at::kHalf) return BSI_DTYPE_F16;
    if (t.scalar_type() == at::kBFloat16) return BSI_DTYPE_BF16;
    return BSI_DTYPE_F32;
}

at::Tensor slice_weight_base(int S, const at::Device& dev) {
    // +-2^i with the top slice negative (bsi_cuda.cpp:217-236, bsi_vector_cuda.cpp:1028); cached per
    // (S, device) like the reference's make_slice_weights_cuda_cached (bsi_vector_cuda.cpp:69-88).
    static std::unordered_map<int64_t, at::Tensor> cache;
    const int64_t key = (static_cast<int64_t>(dev.index()) << 8) | S;
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    std::vector<float> w(S);
    for (int i = 0; i < S; ++i) w[i] = std::ldexp(1.0f, i) * ((i == S - 1) ? -1.0f : 1.0f);
    at::Tensor t = torch::tensor(w, torch::dtype(torch::kFloat32)).to(dev);
    cache[key] = t;
    return t;
}

// ---- holders behind the capsules (bsi_cuda.cpp:146-215) ------------------------------------------
struct PackedBatch {
    at::Tensor words;          // [rows, S, W] int64
    at::Tensor slice_weights;  // [rows, S] float32
    at::Tensor scales;         // [rows, chunks] (chunk mode) or [rows] (row mode) float32: 2^shift
    at::Tensor q8;             // [rows, ld8] int8
    at::Tensor sq_norms;       // [rows, chunks] float32 (chunk mode): (2^shift)^2 * sum of squares of the chunk's integers
    bool chunk_mode = false;
    bool variable = false;     // variable-slice mode: no shift, q8 holds the integers (their low digit when q8_hi is set)
    at::Tensor q8_hi;          // [rows, ld8] int8: v = 128 * q8_hi + q8 (only when some |v| > 127)
    std::vector<int> row_slices;   // variable-slice keys: slice count of every row (bit_width(max|v|) + 2)
    int S = 0;
    int W = 0;
    int64_t rows = 0;
    int64_t d = 0;
    int64_t chunks = 0;
    int decimals = 0;
    float quantize_ms = 0.f;
};

struct PrebuiltBSIKeysCUDA {
    PackedBatch b;
    int64_t num_keys = 0;
    float threshold = 0.2f;
    at::Tensor abs_sum;      // [3, num_keys] float32: sum of |k| over each row of the int8 image, the largest such sum
                             // over one 256-element chunk of the row, the row's sum of k^2
    ~PrebuiltBSIKeysCUDA() {
        if (abs_sum.defined() && b.q8.defined()) bsi_b200_unregister_key_bounds(b.q8.data_ptr<int8_t>());
    }
    // Row sums of |k| for the exact-integer route of the tensor-core dots (bsi_b200_register_key_bounds).
    void compute_bounds() {
        if (!b.q8.defined() || b.q8.numel() == 0 || b.variable) return;
        c10::cuda::CUDAGuard guard(b.q8.device());
        at::Tensor k32 = b.q8.to(at::kInt);
        at::Tensor squares = (k32 * k32).sum(1);                                             // at most 2^24 for 16384 x 32^2
        at::Tensor per_chunk = k32.abs_().view({b.q8.size(0), -1, 256}).sum(2);              // [R, chunks]
        abs_sum = at::stack({per_chunk.sum(1), per_chunk.amax(1), squares}, 0).to(at::kFloat).contiguous();
    }
    // Called before every dot on these keys: the bound depends on the width of the queries of that dot.
    void register_bounds(int query_bits) const {
        if (!abs_sum.defined()) return;
        const int qmax = (query_bits >= 2 && query_bits <= 8) ? (1 << (query_bits - 1)) : 128;
        bsi_b200_register_key_bounds(b.q8.data_ptr<int8_t>(), abs_sum.data_ptr<float>(), num_keys, qmax);
    }
};

// Registers a query batch's chunk sums of squares for the duration of one dot call (the Cauchy-Schwarz side of the
// exact-integer route); the kernel gets the pointers at launch, so the entry can go when the call returns.
struct ScopedQueryBounds {
    const int8_t* a8 = nullptr;
    explicit ScopedQueryBounds(const PackedBatch& qb) {
        if (qb.sq_norms.defined() && qb.chunk_mode && qb.q8.defined() && qb.q8.numel() > 0) {
            a8 = qb.q8.data_ptr<int8_t>();
            bsi_b200_register_query_bounds(a8, qb.sq_norms.data_ptr<float>(), qb.sq_norms.size(1));
        }
    }
    ~ScopedQueryBounds() {
        if (a8 != nullptr) bsi_b200_unregister_query_bounds(a8);
    }
    ScopedQueryBounds(const ScopedQueryBounds&) = delete;
    ScopedQueryBounds& operator=(const ScopedQueryBounds&) = delete;
};

struct PrebuiltBSIQueryBatchCUDA {
    PackedBatch b;
    size_t mem_bytes = 0;
};

struct PrebuiltBSIQueryCUDA {
    std::shared_ptr<PackedBatch> parent;  // the batch this row is a view of
    int64_t row = 0;
    bool twos_complement = false;
    size_t mem_bytes = 0;
};

template <typename T>
T* from_capsule(const py::capsule& cap, const char* name) {
    TORCH_CHECK(cap.name() != nullptr && std::string(cap.name()) == name, "Expected a ", name, " capsule");
    return reinterpret_cast<T*>(cap.get_pointer());
}

// The device a call works on: its first CUDA tensor's, else the current one. Every entry point switches to it for
// its duration (c10::cuda::CUDAGuard), so that allocations, the current stream and the library's per-device caches
// all mean the device the data lives on, whichever device is current in the caller.
at::Device work_device(const at::Tensor& t) {
    return t.is_cuda() ? t.device() : at::Device(at::kCUDA, c10::cuda::current_device());
}
void same_device(const at::Tensor& a, const at::Tensor& b, const char* what) {
    TORCH_CHECK(!a.defined() || !b.defined() || !a.is_cuda() || !b.is_cuda() || a.device() == b.device(), what,
                ": tensors live on different CUDA devices (", a.device(), " and ", b.device(), ")");
}

uint64_t g_last_quantize_ns = 0, g_last_pack_ns = 0, g_last_total_ns = 0;

// Quantise + pack `x` ([rows, d], f32/f16/bf16, CPU or CUDA) in one kernel.
// lean = true skips the bit slices and slice weights (only the int8 image and the scales are
// produced): what the fused linear path needs.
PackedBatch pack(const at::Tensor& input, int decimal_places, int bits, bool chunk_mode, bool profile,
                 bool lean = false) {
    TORCH_CHECK(input.dim() == 2, "expects 2D tensor [rows, d]");
    const float clip_k = clip_k_from_env();
    const auto dev = work_device(input);
    c10::cuda::CUDAGuard guard(dev);
    at::Tensor x = input.detach();
    if (!(x.scalar_type() == at::kFloat || x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16))
        x = x.to(at::kFloat);
    x = x.to(dev, /*non_blocking=*/false).contiguous();

    PackedBatch b;
    b.rows = x.size(0);
    b.d = x.size(1);
    b.S = bits;
    b.W = b.d > 0 ? static_cast<int>((b.d + 63) / 64) : 1;
    b.chunks = (b.d + 255) / 256;
    b.decimals = decimal_places;
    b.chunk_mode = chunk_mode;
    const int64_t ld8 = std::max<int64_t>(b.chunks, 1) * 256;
    auto opt = [&](at::ScalarType t) { return at::TensorOptions().dtype(t).device(dev); };
    // Partial last words / empty inputs rely on zero-initialised words, as the reference's do.
    const bool ragged = (b.d % 64) != 0 || b.rows == 0 || b.d == 0;
    if (!lean)
        b.words = ragged ? at::zeros({b.rows, bits, b.W}, opt(at::kLong)) : at::empty({b.rows, bits, b.W}, opt(at::kLong));
    if (chunk_mode) b.scales = at::ones({b.rows, std::max<int64_t>(b.chunks, 0)}, opt(at::kFloat));
    else b.scales = at::ones({b.rows}, opt(at::kFloat));
    b.q8 = at::empty({b.rows, ld8}, opt(at::kChar));
    if (chunk_mode && b.rows > 0 && b.d > 0) b.sq_norms = at::empty({b.rows, b.chunks}, opt(at::kFloat));
    if (b.rows == 0 || b.d == 0) {
        b.q8.zero_();
        if (lean) b.words = at::zeros({b.rows, bits, b.W}, opt(at::kLong));
        b.slice_weights = slice_weight_base(bits, dev).unsqueeze(0).expand({b.rows, bits}).contiguous();
        return b;
    }

    cudaEvent_t e0 = nullptr, e1 = nullptr;
    auto stream = at::cuda::getCurrentCUDAStream();
    if (profile) {
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, stream.stream());
    }
    check_status(bsi_b200_quantize_pack_norms(x.data_ptr(), dtype_code(x), b.rows, b.d, b.d, decimal_places, bits,
                                              chunk_mode ? 1 : 0, clip_k,
                                              lean ? nullptr : reinterpret_cast<uint64_t*>(b.words.data_ptr<int64_t>()),
                                              b.scales.data_ptr<float>(), nullptr, b.q8.data_ptr<int8_t>(), ld8,
                                              b.sq_norms.defined() ? b.sq_norms.data_ptr<float>() : nullptr,
                                              current_stream()),
                 "bsi_b200_quantize_pack_norms");
    if (profile) {
        cudaEventRecord(e1, stream.stream());
        cudaEventSynchronize(e1);
        cudaEventElapsedTime(&b.quantize_ms, e0, e1);
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    if (lean) return b;
    auto base = slice_weight_base(bits, dev).unsqueeze(0);
    if (chunk_mode) b.slice_weights = base.expand({b.rows, bits}).contiguous();
    else b.slice_weights = (base * b.scales.unsqueeze(1)).contiguous();  // bsi_vector_cuda.cpp:1042,1157
    return b;
}

int variable_slices(uint64_t max_abs) {
    // bsi_vector_cuda.cpp:746-754: bit_width(max |v|) + 2 slices, 2 when everything is zero, at most 64
    int width = 0;
    while (width < 64 && (max_abs >> width) != 0) ++width;
    return max_abs ? std::min(64, std::max(1, width) + 2) : 2;
}

// Variable-slice mode (the reference without BSI_FIXED_BITS*: bsi_vector_cuda.cpp:1086-1166 for query batches,
// bsi_cuda.cpp:912-1007 for keys, whose per-row builder lives in bsiCPP): v = half_away(x * 10^dp), no shift.
// Queries: one slice count for the batch, from the largest |v|; a row uses two's-complement slice weights when it
// holds a negative value, unsigned ones otherwise. Keys: every row has its own count (kept in row_slices for the
// stats); they are stored at the width of the widest row, sign-extended, which leaves every value unchanged.
// The tensor-core dot reads the integers as signed 8-bit digits: queries up to two digits (|v| < 2^14), keys one
// (|v| <= 127); anything larger is refused rather than computed some other way.
PackedBatch pack_variable(const at::Tensor& input, int decimal_places, bool for_keys) {
    TORCH_CHECK(input.dim() == 2, "expects 2D tensor [rows, d]");
    const auto dev = work_device(input);
    c10::cuda::CUDAGuard guard(dev);
    at::Tensor x = input.detach();
    if (!(x.scalar_type() == at::kFloat || x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16))
        x = x.to(at::kFloat);
    x = x.to(dev, /*non_blocking=*/false).contiguous();
    PackedBatch b;
    b.variable = true;
    b.rows = x.size(0);
    b.d = x.size(1);
    b.W = b.d > 0 ? static_cast<int>((b.d + 63) / 64) : 1;
    b.chunks = (b.d + 255) / 256;
    b.decimals = decimal_places;
    b.chunk_mode = false;
    auto opt = [&](at::ScalarType t) { return at::TensorOptions().dtype(t).device(dev); };
    at::Tensor absmax = at::zeros({b.rows}, opt(at::kLong));
    at::Tensor negative = at::zeros({b.rows}, opt(at::kInt));
    if (b.rows > 0 && b.d > 0)
        check_status(bsi_b200_decimal_absmax(x.data_ptr(), dtype_code(x), b.rows, b.d, b.d, decimal_places,
                                             reinterpret_cast<uint64_t*>(absmax.data_ptr<int64_t>()), negative.data_ptr<int>(),
                                             current_stream()),
                     "bsi_b200_decimal_absmax");
    at::Tensor absmax_h = absmax.to(at::kCPU);     // the reference synchronises here too (.item(), bsi_vector_cuda.cpp:1093-1096)
    uint64_t max_abs = 0;
    b.row_slices.resize(static_cast<size_t>(b.rows));
    for (int64_t r = 0; r < b.rows; ++r) {
        const uint64_t m = static_cast<uint64_t>(absmax_h.data_ptr<int64_t>()[r]);
        max_abs = std::max(max_abs, m);
        b.row_slices[static_cast<size_t>(r)] = variable_slices(m);
    }
    b.S = variable_slices(max_abs);
    if (!for_keys) std::fill(b.row_slices.begin(), b.row_slices.end(), b.S);
    TORCH_CHECK(max_abs <= (for_keys ? 127ull : 16383ull), "variable-slice mode: |value * 10^decimal_places| reaches ", max_abs,
                for_keys ? "; keys beyond 127 (8 bits) are not supported" : "; queries beyond 16383 (two 8-bit digits) are not supported",
                " by the tensor-core dot");
    const int64_t ld8 = std::max<int64_t>(b.chunks, 1) * 256;
    b.words = at::zeros({b.rows, b.S, b.W}, opt(at::kLong));
    b.q8 = at::empty({b.rows, ld8}, opt(at::kChar));
    const bool two_digits = max_abs > 127;
    if (two_digits) b.q8_hi = at::empty({b.rows, ld8}, opt(at::kChar));
    if (b.rows > 0 && b.d > 0) {
        check_status(bsi_b200_pack_plain(x.data_ptr(), dtype_code(x), b.rows, b.d, b.d, decimal_places, b.S,
                                         reinterpret_cast<uint64_t*>(b.words.data_ptr<int64_t>()), b.q8.data_ptr<int8_t>(),
                                         two_digits ? b.q8_hi.data_ptr<int8_t>() : nullptr, ld8, current_stream()),
                     "bsi_b200_pack_plain");
    } else {
        b.q8.zero_();
    }
    b.scales = at::ones({b.rows}, opt(at::kFloat));
    // +2^i everywhere, or with the top slice negative for rows that hold a negative value (bsi_vector_cuda.cpp:1156-1162)
    std::vector<float> wu(static_cast<size_t>(b.S)), wt(static_cast<size_t>(b.S));
    for (int i = 0; i < b.S; ++i) {
        wu[static_cast<size_t>(i)] = std::ldexp(1.0f, i);
        wt[static_cast<size_t>(i)] = (i == b.S - 1) ? -std::ldexp(1.0f, i) : std::ldexp(1.0f, i);
    }
    at::Tensor unsigned_w = torch::tensor(wu, torch::dtype(torch::kFloat32)).to(dev).unsqueeze(0);
    at::Tensor twos_w = torch::tensor(wt, torch::dtype(torch::kFloat32)).to(dev).unsqueeze(0);
    b.slice_weights = at::where(negative.ne(0).unsqueeze(1), twos_w, unsigned_w).contiguous();
    return b;
}

void require_fixed_queries(const char* what) {
    TORCH_CHECK(bits_queries() > 0, what, " needs the fixed-bit query mode (BSI_FIXED_BITS_QUERIES in [2, 8])");
}

// Queries get chunk scales when enabled and the word count allows 256-bit chunks
// (bsi_vector_cuda.cpp:980-994).
PackedBatch pack_queries(const at::Tensor& q2d, int decimal_places, bool lean = false) {
    const int bits = bits_queries();
    if (bits == 0) {
        g_last_quantize_ns = g_last_pack_ns = g_last_total_ns = 0;
        return pack_variable(q2d, decimal_places, /*for_keys=*/false);
    }
    const int64_t d = q2d.size(1);
    const int W = d > 0 ? static_cast<int>((d + 63) / 64) : 1;
    const bool chunk = chunk_scale_enabled() && (W % 4 == 0);
    const bool profile = profile_enabled() && q2d.is_cuda();
    PackedBatch b = pack(q2d, decimal_places, bits, chunk, profile, lean);
    // One fused kernel does quantise and pack; its time is reported as the pack time.
    g_last_quantize_ns = 0;
    g_last_pack_ns = profile ? static_cast<uint64_t>(b.quantize_ms * 1.0e6) : 0;
    g_last_total_ns = g_last_pack_ns;
    return b;
}

size_t batch_mem_bytes(const PackedBatch& b) {
    size_t n = static_cast<size_t>(b.words.numel() * b.words.element_size()) +
               static_cast<size_t>(b.slice_weights.numel() * b.slice_weights.element_size());
    if (b.chunk_mode) n += static_cast<size_t>(b.scales.numel() * b.scales.element_size());
    return n;
}

// ---- builders -------------------------------------------------------------------------------------
py::tuple build_bsi_keys_cuda(torch::Tensor K, int decimalPlaces, float compress_threshold) {
    TORCH_CHECK(K.dim() == 2, "K must be 2D [num_keys, d]");
    auto* holder = new PrebuiltBSIKeysCUDA();
    const int kbits = bits_keys();
    holder->b = kbits == 0 ? pack_variable(K, decimalPlaces, /*for_keys=*/true)
                           : pack(K, decimalPlaces, kbits, /*chunk_mode=*/false, /*profile=*/false);
    holder->num_keys = K.size(0);
    holder->threshold = compress_threshold;
    holder->compute_bounds();
    uint64_t total_mem_bytes = static_cast<uint64_t>(holder->b.words.numel() * holder->b.words.element_size());
    if (holder->b.variable) {   // what the reference's per-row vectors would hold: each row its own slice count
        total_mem_bytes = 0;
        for (int sb : holder->b.row_slices) total_mem_bytes += static_cast<uint64_t>(sb) * holder->b.W * 8;
    }
    py::capsule cap(holder, "PrebuiltBSIKeysCUDA", [](PyObject* c) {
        delete reinterpret_cast<PrebuiltBSIKeysCUDA*>(PyCapsule_GetPointer(c, "PrebuiltBSIKeysCUDA"));
    });
    return py::make_tuple(cap, total_mem_bytes, holder->num_keys, K.size(1), holder->b.W);
}

py::capsule build_bsi_queries_cuda_batch_packed(torch::Tensor q2d, int decimalPlaces, float compress_threshold) {
    TORCH_CHECK(q2d.dim() == 2, "q must be 2D [Q, d]");
    (void)compress_threshold;  // ignored by the reference too (bsi_cuda.cpp:350)
    auto* holder = new PrebuiltBSIQueryBatchCUDA();
    holder->b = pack_queries(q2d, decimalPlaces);
    holder->mem_bytes = batch_mem_bytes(holder->b);
    return py::capsule(holder, "PrebuiltBSIQueryBatchCUDA", [](PyObject* c) {
        delete reinterpret_cast<PrebuiltBSIQueryBatchCUDA*>(PyCapsule_GetPointer(c, "PrebuiltBSIQueryBatchCUDA"));
    });
}

py::capsule row_capsule(const std::shared_ptr<PackedBatch>& parent, int64_t row, bool twos) {
    auto* h = new PrebuiltBSIQueryCUDA();
    h->parent = parent;
    h->row = row;
    h->twos_complement = twos;
    h->mem_bytes = static_cast<size_t>(parent->S) * static_cast<size_t>(parent->W) * sizeof(int64_t);
    return py::capsule(h, "PrebuiltBSIQueryCUDA", [](PyObject* c) {
        delete reinterpret_cast<PrebuiltBSIQueryCUDA*>(PyCapsule_GetPointer(c, "PrebuiltBSIQueryCUDA"));
    });
}

py::list build_bsi_queries_cuda_batch(torch::Tensor q2d, int decimalPlaces, float compress_threshold) {
    TORCH_CHECK(q2d.dim() == 2, "q must be 2D [Q, d]");
    (void)compress_threshold;
    auto parent = std::make_shared<PackedBatch>(pack_queries(q2d, decimalPlaces));
    py::list out;
    for (int64_t qi = 0; qi < parent->rows; ++qi) out.append(row_capsule(parent, qi, false));
    return out;
}

// 1-D query: one scale for the whole vector folded into the slice weights
// (bsi_vector_cuda.cpp:778-852, bsi_cuda.cpp:238-270).
py::tuple build_bsi_query_cuda(torch::Tensor q, int decimalPlaces, float compress_threshold) {
    TORCH_CHECK(q.dim() == 1, "q must be 1D [d]");
    (void)compress_threshold;
    auto parent = std::make_shared<PackedBatch>(
        bits_queries() == 0 ? pack_variable(q.unsqueeze(0), decimalPlaces, /*for_keys=*/false)
                            : pack(q.unsqueeze(0), decimalPlaces, bits_queries(), /*chunk_mode=*/false, /*profile=*/false));
    const bool has_negative = q.numel() > 0 && (parent->variable ? parent->slice_weights.lt(0).any().item<bool>()
                                                                 : parent->q8.lt(0).any().item<bool>());
    py::capsule cap = row_capsule(parent, 0, has_negative);
    const uint64_t mem = static_cast<uint64_t>(parent->words.numel() * parent->words.element_size());
    return py::make_tuple(cap, mem, parent->S, parent->W);
}

// ---- EWAH helpers ---------------------------------------------------------------------------------
struct EwahStream {
    at::Tensor stream, off, len, flags;
    int64_t total = 0;
};

EwahStream ewah_encode(const at::Tensor& words2d, double threshold) {
    TORCH_CHECK(words2d.dim() == 2 && words2d.scalar_type() == at::kLong && words2d.is_cuda(),
                "words must be a CUDA int64 tensor [S, W]");
    c10::cuda::CUDAGuard guard(words2d.device());
    auto w = words2d.contiguous();
    const int64_t S = w.size(0), W = w.size(1);
    auto o64 = at::TensorOptions().dtype(at::kLong).device(w.device());
    auto o32 = at::TensorOptions().dtype(at::kInt).device(w.device());
    EwahStream e;
    e.off = at::empty({S}, o64);
    e.len = at::empty({S}, o32);
    e.flags = at::empty({S}, o32);
    auto total = at::zeros({1}, o64);
    const int64_t capacity = S * (W + 1);  // worst case: every slice verbatim, or alternating words
    e.stream = at::empty({std::max<int64_t>(capacity, 1)}, o64);
    auto scratch = at::empty({std::max<int64_t>(bsi_b200_ewah_scratch_bytes(S), 8)},
                             at::TensorOptions().dtype(at::kByte).device(w.device()));
    if (S > 0) {
        check_status(bsi_b200_ewah_encode(reinterpret_cast<const uint64_t*>(w.data_ptr<int64_t>()), S, W, threshold,
                                          scratch.data_ptr(), scratch.numel(),
                                          reinterpret_cast<uint64_t*>(e.stream.data_ptr<int64_t>()), capacity,
                                          reinterpret_cast<uint64_t*>(e.off.data_ptr<int64_t>()),
                                          e.len.data_ptr<int>(), e.flags.data_ptr<int>(),
                                          reinterpret_cast<uint64_t*>(total.data_ptr<int64_t>()), current_stream()),
                     "bsi_b200_ewah_encode");
    }
    e.total = total.item<int64_t>();
    e.stream = e.stream.narrow(0, 0, e.total);
    return e;
}

at::Tensor ewah_decode(const EwahStream& e, int64_t W) {
    const int64_t S = e.off.size(0);
    c10::cuda::CUDAGuard guard(e.off.device());
    same_device(e.off, e.stream, "ewah_decode");
    auto out = at::empty({S, W}, at::TensorOptions().dtype(at::kLong).device(e.off.device()));
    if (S > 0) {
        check_status(bsi_b200_ewah_decode(reinterpret_cast<const uint64_t*>(e.stream.data_ptr<int64_t>()),
                                          reinterpret_cast<const uint64_t*>(e.off.data_ptr<int64_t>()),
                                          e.len.data_ptr<int>(), S, W,
                                          reinterpret_cast<uint64_t*>(out.data_ptr<int64_t>()), current_stream()),
                     "bsi_b200_ewah_decode");
    }
    return out;
}

// EWAH round trip of a 1-D query (bsi_cuda.cpp:386-431): encode the slices, decode them back into
// the verbatim words the dot consumes; mem_bytes = compressed + verbatim.
py::tuple build_bsi_query_cuda_hybrid(torch::Tensor q, int decimalPlaces, double compress_threshold) {
    TORCH_CHECK(q.dim() == 1, "q must be 1D [d]");
    auto parent = std::make_shared<PackedBatch>(
        bits_queries() == 0 ? pack_variable(q.unsqueeze(0), decimalPlaces, /*for_keys=*/false)
                            : pack(q.unsqueeze(0), decimalPlaces, bits_queries(), /*chunk_mode=*/false, /*profile=*/false));
    const bool has_negative = q.numel() > 0 && (parent->variable ? parent->slice_weights.lt(0).any().item<bool>()
                                                                 : parent->q8.lt(0).any().item<bool>());
    auto words2d = parent->words.view({parent->S, parent->W});
    EwahStream e = ewah_encode(words2d, compress_threshold);
    parent->words = ewah_decode(e, parent->W).view({1, parent->S, parent->W});
    py::capsule cap = row_capsule(parent, 0, has_negative);
    const uint64_t mem = static_cast<uint64_t>(e.total * 8 + parent->words.numel() * parent->words.element_size());
    reinterpret_cast<PrebuiltBSIQueryCUDA*>(cap.get_pointer())->mem_bytes = mem;
    return py::make_tuple(cap, mem, parent->S, parent->W);
}

// ---- dot ------------------------------------------------------------------------------------------
py::tuple run_dot(const PackedBatch& qb, const PrebuiltBSIKeysCUDA& keys, bool want_iacc, at::Tensor* iacc_out) {
    const int64_t Q = qb.rows, R = keys.num_keys;
    same_device(qb.q8, keys.b.q8, "queries and keys");
    c10::cuda::CUDAGuard guard(keys.b.q8.device());
    TORCH_CHECK(Q > 0 && qb.S > 0 && qb.W > 0, "Empty query batch");
    TORCH_CHECK(qb.W == keys.b.W, "Word count mismatch between query batch and keys");
    TORCH_CHECK(R > 0, "Empty keys");
    TORCH_CHECK(qb.decimals == keys.b.decimals, "Decimal mismatch between queries and keys: q=", qb.decimals,
                " k=", keys.b.decimals);
    if (qb.chunk_mode) TORCH_CHECK(keys.b.W % 4 == 0, "Chunk scales require W64 multiple of 4");
    const int total_decimals = qb.decimals + keys.b.decimals;
    const double scale_inv = total_decimals > 0 ? 1.0 / std::pow(10.0, total_decimals) : 1.0;  // bsi_cuda.cpp:710-711

    auto fopt = at::TensorOptions().dtype(at::kFloat).device(qb.q8.device());
    at::Tensor out = at::empty({Q, R}, fopt);
    at::Tensor iacc;
    if (want_iacc) iacc = at::empty({Q, R, qb.chunks}, fopt.dtype(at::kInt));

    const bool profile = profile_enabled();
    auto stream = at::cuda::getCurrentCUDAStream();
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    float kernel_ms = 0.f;
    if (profile) {
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, stream.stream());
    }
    const int engine = engine_from_env();
    const int64_t qs_stride = qb.chunk_mode ? qb.chunks : 0;
    keys.register_bounds(qb.variable ? 8 : qb.S);
    ScopedQueryBounds query_bounds(qb);
    if (qb.variable || keys.b.variable) {
        TORCH_CHECK(engine != BSI_ENGINE_BMMA, "the b1 mma.sync engine reads fixed-bit slices; variable-slice operands use the int8 engines");
        TORCH_CHECK(!want_iacc, "the per-chunk accumulator dump is defined for the fixed-bit mode");
    }
    if (qb.variable && qb.q8_hi.defined()) {
        // Two-digit queries, v = 128 * hi + lo: one exact integer dot per digit with unit scales, then
        // (128 * I_hi + I_lo) * bw0[r] * scale_inv. Every intermediate is an integer below 2^24 times a power of two
        // wherever the reference's own float32 accumulation (bsi_cuda_kernels_dot.cuh:597-654) is exact, so the two agree.
        at::Tensor out_hi = at::empty({Q, R}, fopt);
        for (int digit = 0; digit < 2; ++digit) {
            const at::Tensor& a8 = digit == 0 ? qb.q8 : qb.q8_hi;
            at::Tensor& dst = digit == 0 ? out : out_hi;
            check_status(bsi_b200_dot_i8(a8.data_ptr<int8_t>(), a8.size(1), qb.scales.data_ptr<float>(), 0,
                                         keys.b.q8.data_ptr<int8_t>(), keys.b.q8.size(1), keys.b.scales.data_ptr<float>(),
                                         Q, R, qb.chunks, 1.0f, dst.data_ptr<float>(), R, nullptr, engine, current_stream()),
                         "bsi_b200_dot_i8");
        }
        out.add_(out_hi, 128.0f).mul_(static_cast<float>(scale_inv));
    } else if (engine == BSI_ENGINE_BMMA) {
        check_status(bsi_b200_dot_words(reinterpret_cast<const uint64_t*>(qb.words.data_ptr<int64_t>()),
                                        qb.scales.data_ptr<float>(), qs_stride, qb.S, qb.W,
                                        reinterpret_cast<const uint64_t*>(keys.b.words.data_ptr<int64_t>()),
                                        keys.b.slice_weights.data_ptr<float>(), keys.b.S, R, Q,
                                        static_cast<float>(scale_inv), R, out.data_ptr<float>(),
                                        want_iacc ? iacc.data_ptr<int>() : nullptr, current_stream()),
                     "bsi_b200_dot_words");
    } else {
        check_status(bsi_b200_dot_i8(qb.q8.data_ptr<int8_t>(), qb.q8.size(1), qb.scales.data_ptr<float>(), qs_stride,
                                     keys.b.q8.data_ptr<int8_t>(), keys.b.q8.size(1), keys.b.scales.data_ptr<float>(),
                                     Q, R, qb.chunks, static_cast<float>(scale_inv), out.data_ptr<float>(), R,
                                     want_iacc ? iacc.data_ptr<int>() : nullptr, engine, current_stream()),
                     "bsi_b200_dot_i8");
    }
    if (profile) {
        cudaEventRecord(e1, stream.stream());
        cudaEventSynchronize(e1);
        cudaEventElapsedTime(&kernel_ms, e0, e1);
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    if (iacc_out) *iacc_out = iacc;
    const uint64_t ns_total = static_cast<uint64_t>(kernel_ms * 1.0e6);
    const double per_query = Q > 0 ? static_cast<double>(ns_total) / static_cast<double>(Q) : 0.0;
    const double per_scalar = (Q > 0 && R > 0) ? static_cast<double>(ns_total) / (static_cast<double>(Q) * R) : 0.0;
    return py::make_tuple(out, ns_total, per_query, per_scalar);
}

py::tuple batch_dot_product_multiquery_cuda_batch_caps(py::capsule query_batch_cap, py::capsule keyset_cuda_cap) {
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(keyset_cuda_cap, "PrebuiltBSIKeysCUDA");
    TORCH_CHECK(keys != nullptr, "Invalid CUDA keys capsule");
    auto* qb = from_capsule<PrebuiltBSIQueryBatchCUDA>(query_batch_cap, "PrebuiltBSIQueryBatchCUDA");
    TORCH_CHECK(qb != nullptr, "Invalid CUDA query-batch capsule");
    return run_dot(qb->b, *keys, false, nullptr);
}

// Rebuilds a batch from per-row capsules. Rows that are, in order, all the rows of one parent
// batch (what build_bsi_queries_cuda_batch returns) reuse it without copying; any other list is
// gathered row by row (the reference always re-stacks, bsi_cuda.cpp:487-518).
PackedBatch batch_from_list(const py::list& caps) {
    const int64_t Q = static_cast<int64_t>(py::len(caps));
    std::vector<PrebuiltBSIQueryCUDA*> rows(Q);
    for (int64_t i = 0; i < Q; ++i) {
        TORCH_CHECK(py::isinstance<py::capsule>(caps[i]), "Each item must be a capsule");
        rows[i] = from_capsule<PrebuiltBSIQueryCUDA>(py::cast<py::capsule>(caps[i]), "PrebuiltBSIQueryCUDA");
        TORCH_CHECK(rows[i] != nullptr && rows[i]->parent, "Invalid BSI query capsule at index ", i);
    }
    const auto& p0 = rows[0]->parent;
    bool whole = (p0->rows == Q);
    for (int64_t i = 0; i < Q && whole; ++i) whole = (rows[i]->parent == p0 && rows[i]->row == i);
    if (whole) return *p0;
    PackedBatch b;
    b.S = p0->S; b.W = p0->W; b.d = p0->d; b.chunks = p0->chunks; b.decimals = p0->decimals;
    b.chunk_mode = p0->chunk_mode; b.rows = Q; b.variable = p0->variable;
    bool any_hi = false;
    for (int64_t i = 0; i < Q; ++i) any_hi = any_hi || rows[i]->parent->q8_hi.defined();
    std::vector<at::Tensor> words, weights, scales, q8, q8_hi;
    for (int64_t i = 0; i < Q; ++i) {
        const auto& p = rows[i]->parent;
        TORCH_CHECK(p->W == b.W, "Word count mismatch across queries");
        TORCH_CHECK(p->decimals == b.decimals, "Decimal mismatch across queries not supported");
        TORCH_CHECK(p->S == b.S, "Mixed slice counts across queries are not supported");
        TORCH_CHECK(p->variable == b.variable, "Mixed fixed-bit and variable-slice queries in the same group");
        TORCH_CHECK(p->chunk_mode == b.chunk_mode, "Mixed chunk-scale and non-chunk-scale queries in the same group");
        words.push_back(p->words[rows[i]->row]);
        weights.push_back(p->slice_weights[rows[i]->row]);
        scales.push_back(p->scales[rows[i]->row]);
        q8.push_back(p->q8[rows[i]->row]);
        if (any_hi) q8_hi.push_back(p->q8_hi.defined() ? p->q8_hi[rows[i]->row] : at::zeros_like(p->q8[rows[i]->row]));
    }
    if (any_hi) b.q8_hi = at::stack(q8_hi).contiguous();
    b.row_slices.assign(static_cast<size_t>(Q), b.S);
    b.words = at::stack(words).contiguous();
    b.slice_weights = at::stack(weights).contiguous();
    b.scales = at::stack(scales).contiguous();
    b.q8 = at::stack(q8).contiguous();
    {
        bool all = true;
        for (int64_t i = 0; i < Q; ++i) all = all && rows[i]->parent->sq_norms.defined();
        if (all && Q > 0) {
            std::vector<at::Tensor> n2;
            for (int64_t i = 0; i < Q; ++i) n2.push_back(rows[i]->parent->sq_norms[rows[i]->row]);
            b.sq_norms = at::stack(n2).contiguous();
        }
    }
    return b;
}

py::tuple batch_dot_product_multiquery_cuda_caps(py::list query_caps_list, py::capsule keyset_cuda_cap) {
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(keyset_cuda_cap, "PrebuiltBSIKeysCUDA");
    TORCH_CHECK(keys != nullptr, "Invalid CUDA keys capsule");
    TORCH_CHECK(keys->num_keys > 0 && py::len(query_caps_list) > 0, "Empty keys or queries");
    PackedBatch b = batch_from_list(query_caps_list);
    return run_dot(b, *keys, false, nullptr);
}

// ---- stats ----------------------------------------------------------------------------------------
py::dict bsi_keys_cuda_stats(py::capsule keyset_cuda_cap) {
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(keyset_cuda_cap, "PrebuiltBSIKeysCUDA");
    py::dict sb;
    if (keys->b.variable) {   // histogram of the per-row slice counts, as the reference groups its keys (bsi_cuda.cpp:956-999)
        std::unordered_map<int, int64_t> hist;
        for (int v : keys->b.row_slices) ++hist[v];
        for (const auto& kv : hist) sb[py::int_(kv.first)] = py::int_(kv.second);
    } else {
        sb[py::int_(keys->b.S)] = py::int_(keys->num_keys);
    }
    py::dict out;
    out["W"] = py::int_(keys->b.W);
    out["d"] = py::int_(keys->b.d);
    out["num_keys"] = py::int_(keys->num_keys);
    out["decimals"] = py::int_(keys->b.decimals);
    out["threshold"] = py::float_(keys->threshold);
    out["Sb_counts"] = sb;
    return out;
}

py::dict bsi_query_caps_stats(py::list query_caps_list) {
    const int64_t Q = static_cast<int64_t>(py::len(query_caps_list));
    TORCH_CHECK(Q > 0, "Empty query capsule list");
    std::unordered_map<int, int64_t> counts;
    int W = -1;
    for (int64_t i = 0; i < Q; ++i) {
        TORCH_CHECK(py::isinstance<py::capsule>(query_caps_list[i]), "Each item must be a capsule");
        auto* q = from_capsule<PrebuiltBSIQueryCUDA>(py::cast<py::capsule>(query_caps_list[i]), "PrebuiltBSIQueryCUDA");
        counts[q->parent->S] += 1;
        if (W < 0) W = q->parent->W;
        else TORCH_CHECK(q->parent->W == W, "Word count mismatch across queries");
    }
    py::dict s_counts;
    for (const auto& kv : counts) s_counts[py::int_(kv.first)] = py::int_(kv.second);
    py::dict out;
    out["Q"] = py::int_(Q);
    out["W"] = py::int_(W);
    out["S_counts"] = s_counts;
    return out;
}

std::string cuda_builder_version() { return "BSI_B200_SM100A_V" + std::to_string(bsi_b200_version()); }

// ---- additions (no counterpart in the reference module) -------------------------------------------
// One call for a whole linear layer: pack x, dot with the keys, cast to x's dtype and add the bias.
// Same arithmetic as BSIQuantizedLinear.forward (verify_accuracy_bsi.py:118-215) without the
// capsule round trip, the float32 [Q, R] re-read by two elementwise kernels, or host syncs.
at::Tensor bsi_linear_forward(torch::Tensor x2d, py::capsule keyset_cuda_cap, c10::optional<torch::Tensor> bias,
                              int decimalPlaces) {
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(keyset_cuda_cap, "PrebuiltBSIKeysCUDA");
    TORCH_CHECK(x2d.dim() == 2 && x2d.is_cuda(), "x must be a 2D CUDA tensor");
    same_device(x2d, keys->b.q8, "activations and keys");
    c10::cuda::CUDAGuard guard(x2d.device());
    const int engine = engine_from_env();
    // two-digit variable-slice queries need two dots and a combine: they take the unfused route below
    const bool fused = (engine == BSI_ENGINE_AUTO || engine == BSI_ENGINE_TCGEN05) && bits_queries() > 0;
    PackedBatch qb = pack_queries(x2d, decimalPlaces, /*lean=*/fused);
    const int64_t Q = qb.rows, R = keys->num_keys;
    TORCH_CHECK(Q > 0 && R > 0, "Empty queries or keys");
    TORCH_CHECK(qb.W == keys->b.W, "Word count mismatch between query batch and keys");
    TORCH_CHECK(qb.decimals == keys->b.decimals, "Decimal mismatch between queries and keys: q=", qb.decimals,
                " k=", keys->b.decimals);
    const int total_decimals = qb.decimals + keys->b.decimals;
    const double scale_inv = total_decimals > 0 ? 1.0 / std::pow(10.0, total_decimals) : 1.0;
    at::ScalarType yt = x2d.scalar_type();
    if (!(yt == at::kFloat || yt == at::kHalf || yt == at::kBFloat16)) yt = at::kFloat;
    at::Tensor y = at::empty({Q, R}, qb.q8.options().dtype(yt));
    const float* bptr = nullptr;
    at::Tensor b32;
    if (bias.has_value() && bias->defined()) {
        b32 = bias->to(y.device(), at::kFloat).contiguous();
        TORCH_CHECK(b32.numel() == R, "bias length mismatch");
        bptr = b32.data_ptr<float>();
    }
    const int code = yt == at::kHalf ? BSI_DTYPE_F16 : (yt == at::kBFloat16 ? BSI_DTYPE_BF16 : BSI_DTYPE_F32);
    if (fused) {
        keys->register_bounds(qb.S);
        ScopedQueryBounds query_bounds(qb);
        check_status(bsi_b200_linear_i8(qb.q8.data_ptr<int8_t>(), qb.q8.size(1), qb.scales.data_ptr<float>(),
                                        qb.chunk_mode ? qb.chunks : 0, keys->b.q8.data_ptr<int8_t>(),
                                        keys->b.q8.size(1), keys->b.scales.data_ptr<float>(), bptr, Q, R, qb.chunks,
                                        static_cast<float>(scale_inv), y.data_ptr(), R, code, current_stream()),
                     "bsi_b200_linear_i8");
        return y;
    }
    // other engines: float32 dot, then the separate cast + bias kernel
    py::tuple r = run_dot(qb, *keys, false, nullptr);
    at::Tensor out = r[0].cast<at::Tensor>();
    check_status(bsi_b200_cast_bias(out.data_ptr<float>(), R, bptr, Q, R, y.data_ptr(), R, code, current_stream()),
                 "bsi_b200_cast_bias");
    return y;
}

// Quantise + pack activations (query side: chunk scales) into tensors the caller owns: q8 [rows, >= d]
// int8 (any row stride that is a multiple of 16 bytes, e.g. a column block of a wider matrix) and
// scales [rows, d/256] float32, contiguous. This is the first half of bsi_linear_forward, split off so
// that a tensor-parallel layer can pack its own column block straight into the buffer the ranks
// exchange. d must be a multiple of 256.
void pack_queries_into(torch::Tensor x2d, torch::Tensor q8, torch::Tensor scales, int decimalPlaces) {
    require_fixed_queries("pack_queries_into");
    TORCH_CHECK(x2d.dim() == 2 && x2d.is_cuda(), "x must be a 2D CUDA tensor");
    TORCH_CHECK(q8.dim() == 2 && q8.is_cuda() && q8.scalar_type() == at::kChar && q8.stride(1) == 1, "q8 must be int8 [rows, d]");
    TORCH_CHECK(scales.is_cuda() && scales.scalar_type() == at::kFloat && scales.is_contiguous(), "scales must be contiguous float32");
    check_clip("pack_queries_into");
    same_device(x2d, q8, "pack_queries_into");
    same_device(x2d, scales, "pack_queries_into");
    c10::cuda::CUDAGuard guard(x2d.device());
    TORCH_CHECK(chunk_scale_enabled(), "pack_queries_into needs BSI_FIXED_CHUNK_SCALE=1");
    at::Tensor x = x2d.detach();
    if (!(x.scalar_type() == at::kFloat || x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16))
        x = x.to(at::kFloat);
    if (x.stride(1) != 1) x = x.contiguous();
    const int64_t rows = x.size(0), d = x.size(1);
    TORCH_CHECK(d % 256 == 0, "d must be a multiple of 256");
    TORCH_CHECK(q8.size(0) == rows && q8.size(1) >= d, "q8 shape mismatch");
    TORCH_CHECK(scales.numel() == rows * (d / 256), "scales shape mismatch");
    if (rows == 0 || d == 0) return;
    check_status(bsi_b200_quantize_pack(x.data_ptr(), dtype_code(x), rows, d, x.stride(0), decimalPlaces,
                                        bits_queries(), 1, nullptr, scales.data_ptr<float>(), nullptr,
                                        q8.data_ptr<int8_t>(), q8.stride(0), current_stream()),
                 "bsi_b200_quantize_pack");
}

// Second half of bsi_linear_forward: the dot of already packed activations with a key set, cast to
// `out_dtype`, bias added, optionally ReLU. q8 [Q, d] int8 (row stride a multiple of 16), scales
// [Q, d/256] float32 contiguous.
at::Tensor linear_from_packed(torch::Tensor q8, torch::Tensor scales, py::capsule keyset_cuda_cap,
                              c10::optional<torch::Tensor> bias, int decimalPlaces, py::object out_dtype, bool relu) {
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(keyset_cuda_cap, "PrebuiltBSIKeysCUDA");
    TORCH_CHECK(q8.dim() == 2 && q8.is_cuda() && q8.scalar_type() == at::kChar && q8.stride(1) == 1, "q8 must be int8 [Q, d]");
    TORCH_CHECK(scales.is_cuda() && scales.scalar_type() == at::kFloat && scales.is_contiguous(), "scales must be contiguous float32");
    same_device(q8, scales, "packed activations and scales");
    same_device(q8, keys->b.q8, "packed activations and keys");
    c10::cuda::CUDAGuard guard(q8.device());
    const int64_t Q = q8.size(0), R = keys->num_keys, chunks = keys->b.chunks;
    TORCH_CHECK(Q > 0 && R > 0, "Empty queries or keys");
    TORCH_CHECK(q8.size(1) == chunks * 256, "Word count mismatch between query batch and keys");
    TORCH_CHECK(scales.numel() == Q * chunks, "scales shape mismatch");
    TORCH_CHECK(decimalPlaces == keys->b.decimals, "Decimal mismatch between queries and keys: q=", decimalPlaces,
                " k=", keys->b.decimals);
    const int total_decimals = decimalPlaces + keys->b.decimals;
    const double scale_inv = total_decimals > 0 ? 1.0 / std::pow(10.0, total_decimals) : 1.0;
    const at::ScalarType yt = torch::python::detail::py_object_to_dtype(out_dtype);
    TORCH_CHECK(yt == at::kFloat || yt == at::kHalf || yt == at::kBFloat16, "out_dtype must be float32, float16 or bfloat16");
    at::Tensor y = at::empty({Q, R}, q8.options().dtype(yt));
    const float* bptr = nullptr;
    at::Tensor b32;
    if (bias.has_value() && bias->defined()) {
        b32 = bias->to(y.device(), at::kFloat).contiguous();
        TORCH_CHECK(b32.numel() == R, "bias length mismatch");
        bptr = b32.data_ptr<float>();
    }
    const int code = yt == at::kHalf ? BSI_DTYPE_F16 : (yt == at::kBFloat16 ? BSI_DTYPE_BF16 : BSI_DTYPE_F32);
    keys->register_bounds(bits_queries());
    check_status(bsi_b200_linear_i8_act(q8.data_ptr<int8_t>(), q8.stride(0), scales.data_ptr<float>(), chunks,
                                        keys->b.q8.data_ptr<int8_t>(), keys->b.q8.size(1), keys->b.scales.data_ptr<float>(),
                                        bptr, Q, R, chunks, static_cast<float>(scale_inv), y.data_ptr(), R, code,
                                        relu ? BSI_ACT_RELU : BSI_ACT_NONE, current_stream()),
                 "bsi_b200_linear_i8_act");
    return y;
}

// ---- peer memory and the stores-as-collectives of the tensor-parallel layer -----------------------
// A zero-filled device buffer other processes of the node can map, as a uint8 tensor, and the bytes of
// its CUDA IPC handle.
py::tuple peer_alloc(int64_t nbytes) {
    void* ptr = nullptr;
    char handle[BSI_B200_PEER_HANDLE_BYTES];
    check_status(bsi_b200_peer_alloc(nbytes, &ptr, handle), "bsi_b200_peer_alloc");
    const auto dev = at::Device(at::kCUDA, c10::cuda::current_device());
    at::Tensor t = at::from_blob(ptr, {nbytes}, [](void* p) { bsi_b200_peer_free(p); },
                                 at::TensorOptions().dtype(at::kByte).device(dev));
    return py::make_tuple(t, py::bytes(handle, sizeof(handle)));
}

int64_t peer_open(py::bytes handle) {
    std::string h = handle;
    TORCH_CHECK(h.size() == BSI_B200_PEER_HANDLE_BYTES, "peer handle must be ", BSI_B200_PEER_HANDLE_BYTES, " bytes");
    void* ptr = nullptr;
    check_status(bsi_b200_peer_open(h.data(), &ptr), "bsi_b200_peer_open");
    return static_cast<int64_t>(reinterpret_cast<intptr_t>(ptr));
}

void peer_close(int64_t ptr) { check_status(bsi_b200_peer_close(reinterpret_cast<void*>(static_cast<intptr_t>(ptr))), "bsi_b200_peer_close"); }

void peer_barrier(std::vector<int64_t> flag_ptrs, int rank, int64_t timeout_ms) {
    std::vector<uint32_t*> f;
    for (int64_t p : flag_ptrs) f.push_back(reinterpret_cast<uint32_t*>(static_cast<intptr_t>(p)));
    check_status(bsi_b200_peer_barrier(f.data(), rank, static_cast<int>(f.size()), timeout_ms, current_stream()),
                 "bsi_b200_peer_barrier");
}

// pack_queries_into with several destinations given as raw device addresses (own memory or peer
// mappings): the int8 image lands at q8_ptrs[i] + row * ld8 + col, the chunk scales at
// scale_ptrs[i] + 4 * (row * scale_ld + chunk).
void pack_queries_multi(torch::Tensor x2d, std::vector<int64_t> q8_ptrs, int64_t ld8, std::vector<int64_t> scale_ptrs,
                        int64_t scale_ld, int decimalPlaces) {
    require_fixed_queries("pack_queries_multi");
    TORCH_CHECK(x2d.dim() == 2 && x2d.is_cuda(), "x must be a 2D CUDA tensor");
    TORCH_CHECK(!q8_ptrs.empty() && !scale_ptrs.empty(), "destination lists must not be empty");
    c10::cuda::CUDAGuard guard(x2d.device());   // raw destinations: the caller's own or peer mappings of this device
    check_clip("pack_queries_multi");
    TORCH_CHECK(chunk_scale_enabled(), "pack_queries_multi needs BSI_FIXED_CHUNK_SCALE=1");
    at::Tensor x = x2d.detach();
    if (!(x.scalar_type() == at::kFloat || x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16))
        x = x.to(at::kFloat);
    if (x.stride(1) != 1) x = x.contiguous();
    std::vector<int8_t*> q;
    std::vector<float*> sc;
    for (int64_t p : q8_ptrs) q.push_back(reinterpret_cast<int8_t*>(static_cast<intptr_t>(p)));
    for (int64_t p : scale_ptrs) sc.push_back(reinterpret_cast<float*>(static_cast<intptr_t>(p)));
    check_status(bsi_b200_quantize_pack_multi(x.data_ptr(), dtype_code(x), x.size(0), x.size(1), x.stride(0), decimalPlaces,
                                              bits_queries(), static_cast<int>(q.size()), q.data(), ld8,
                                              static_cast<int>(sc.size()), sc.data(), scale_ld, current_stream()),
                 "bsi_b200_quantize_pack_multi");
}

// linear_from_packed whose rows are dealt out to the matrices at y_ptrs (rows_per_dst rows each, leading
// dimension ldy, element type out_dtype); returns nothing, the destinations are the caller's buffers.
void linear_from_packed_scatter(torch::Tensor q8, torch::Tensor scales, py::capsule keyset_cuda_cap,
                                c10::optional<torch::Tensor> bias, int decimalPlaces, py::object out_dtype, bool relu,
                                std::vector<int64_t> y_ptrs, int64_t rows_per_dst, int64_t ldy) {
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(keyset_cuda_cap, "PrebuiltBSIKeysCUDA");
    TORCH_CHECK(q8.dim() == 2 && q8.is_cuda() && q8.scalar_type() == at::kChar && q8.stride(1) == 1, "q8 must be int8 [Q, d]");
    TORCH_CHECK(scales.is_cuda() && scales.scalar_type() == at::kFloat && scales.is_contiguous(), "scales must be contiguous float32");
    same_device(q8, scales, "packed activations and scales");
    same_device(q8, keys->b.q8, "packed activations and keys");
    c10::cuda::CUDAGuard guard(q8.device());
    const int64_t Q = q8.size(0), R = keys->num_keys, chunks = keys->b.chunks;
    TORCH_CHECK(Q > 0 && R > 0, "Empty queries or keys");
    TORCH_CHECK(q8.size(1) == chunks * 256, "Word count mismatch between query batch and keys");
    TORCH_CHECK(scales.numel() == Q * chunks, "scales shape mismatch");
    TORCH_CHECK(decimalPlaces == keys->b.decimals, "Decimal mismatch between queries and keys");
    const int total_decimals = decimalPlaces + keys->b.decimals;
    const double scale_inv = total_decimals > 0 ? 1.0 / std::pow(10.0, total_decimals) : 1.0;
    const at::ScalarType yt = torch::python::detail::py_object_to_dtype(out_dtype);
    TORCH_CHECK(yt == at::kFloat || yt == at::kHalf || yt == at::kBFloat16, "out_dtype must be float32, float16 or bfloat16");
    const float* bptr = nullptr;
    at::Tensor b32;
    if (bias.has_value() && bias->defined()) {
        b32 = bias->to(q8.device(), at::kFloat).contiguous();
        TORCH_CHECK(b32.numel() == R, "bias length mismatch");
        bptr = b32.data_ptr<float>();
    }
    std::vector<void*> y;
    for (int64_t p : y_ptrs) y.push_back(reinterpret_cast<void*>(static_cast<intptr_t>(p)));
    const int code = yt == at::kHalf ? BSI_DTYPE_F16 : (yt == at::kBFloat16 ? BSI_DTYPE_BF16 : BSI_DTYPE_F32);
    keys->register_bounds(bits_queries());
    check_status(bsi_b200_linear_i8_scatter(q8.data_ptr<int8_t>(), q8.stride(0), scales.data_ptr<float>(), chunks,
                                            keys->b.q8.data_ptr<int8_t>(), keys->b.q8.size(1),
                                            keys->b.scales.data_ptr<float>(), bptr, Q, R, chunks,
                                            static_cast<float>(scale_inv), static_cast<int>(y.size()), y.data(),
                                            rows_per_dst, ldy, code, relu ? BSI_ACT_RELU : BSI_ACT_NONE, current_stream()),
                 "bsi_b200_linear_i8_scatter");
}

// linear_from_packed whose finished output (cast + bias, optional ReLU, in `layer_dtype`) is re-quantised
// inside the epilogue for the next linear: the int8 image goes to q8_ptrs[i] + q * ld8 + r, the chunk scales
// to scale_ptrs[i] + 4 * (q * scale_ld + r / 256). Nothing is returned.
void linear_from_packed_requant(torch::Tensor q8, torch::Tensor scales, py::capsule keyset_cuda_cap,
                                c10::optional<torch::Tensor> bias, int decimalPlaces, py::object layer_dtype, bool relu,
                                std::vector<int64_t> q8_ptrs, int64_t ld8, std::vector<int64_t> scale_ptrs,
                                int64_t scale_ld) {
    require_fixed_queries("linear_from_packed_requant");
    check_clip("linear_from_packed_requant");
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(keyset_cuda_cap, "PrebuiltBSIKeysCUDA");
    TORCH_CHECK(q8.dim() == 2 && q8.is_cuda() && q8.scalar_type() == at::kChar && q8.stride(1) == 1, "q8 must be int8 [Q, d]");
    TORCH_CHECK(scales.is_cuda() && scales.scalar_type() == at::kFloat && scales.is_contiguous(), "scales must be contiguous float32");
    TORCH_CHECK(q8_ptrs.size() == scale_ptrs.size() && !q8_ptrs.empty(), "destination lists must match");
    same_device(q8, scales, "packed activations and scales");
    same_device(q8, keys->b.q8, "packed activations and keys");
    c10::cuda::CUDAGuard guard(q8.device());
    const int64_t Q = q8.size(0), R = keys->num_keys, chunks = keys->b.chunks;
    TORCH_CHECK(Q > 0 && R > 0, "Empty queries or keys");
    TORCH_CHECK(q8.size(1) == chunks * 256, "Word count mismatch between query batch and keys");
    TORCH_CHECK(scales.numel() == Q * chunks, "scales shape mismatch");
    TORCH_CHECK(decimalPlaces == keys->b.decimals, "Decimal mismatch between queries and keys");
    const int total_decimals = decimalPlaces + keys->b.decimals;
    const double scale_inv = total_decimals > 0 ? 1.0 / std::pow(10.0, total_decimals) : 1.0;
    const at::ScalarType yt = torch::python::detail::py_object_to_dtype(layer_dtype);
    TORCH_CHECK(yt == at::kHalf || yt == at::kBFloat16, "layer_dtype must be float16 or bfloat16");
    const float* bptr = nullptr;
    at::Tensor b32;
    if (bias.has_value() && bias->defined()) {
        b32 = bias->to(q8.device(), at::kFloat).contiguous();
        TORCH_CHECK(b32.numel() == R, "bias length mismatch");
        bptr = b32.data_ptr<float>();
    }
    std::vector<int8_t*> qd;
    std::vector<float*> sd;
    for (int64_t p : q8_ptrs) qd.push_back(reinterpret_cast<int8_t*>(static_cast<intptr_t>(p)));
    for (int64_t p : scale_ptrs) sd.push_back(reinterpret_cast<float*>(static_cast<intptr_t>(p)));
    keys->register_bounds(bits_queries());
    check_status(bsi_b200_linear_i8_requant(q8.data_ptr<int8_t>(), q8.stride(0), scales.data_ptr<float>(), chunks,
                                            keys->b.q8.data_ptr<int8_t>(), keys->b.q8.size(1),
                                            keys->b.scales.data_ptr<float>(), bptr, Q, R, chunks,
                                            static_cast<float>(scale_inv), yt == at::kHalf ? BSI_DTYPE_F16 : BSI_DTYPE_BF16,
                                            relu ? BSI_ACT_RELU : BSI_ACT_NONE, decimalPlaces, bits_queries(),
                                            static_cast<int>(qd.size()), qd.data(), ld8, sd.data(), scale_ld, current_stream()),
                 "bsi_b200_linear_i8_requant");
}

// Residual add + LayerNorm + activation pack (16-bit layer types). Returns x + delta (delta optional); the
// packed LayerNorm output goes to the raw destinations as in pack_queries_multi.
at::Tensor add_layernorm_pack(torch::Tensor x, c10::optional<torch::Tensor> delta, torch::Tensor weight, torch::Tensor bias,
                              double eps, std::vector<int64_t> q8_ptrs, int64_t ld8, std::vector<int64_t> scale_ptrs,
                              int64_t scale_ld, int decimalPlaces) {
    require_fixed_queries("add_layernorm_pack");
    TORCH_CHECK(x.dim() == 2 && x.is_cuda() && x.is_contiguous(), "x must be a contiguous 2D CUDA tensor");
    TORCH_CHECK(x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16, "x must be float16 or bfloat16");
    TORCH_CHECK(weight.scalar_type() == x.scalar_type() && bias.scalar_type() == x.scalar_type() && weight.is_contiguous() &&
                    bias.is_contiguous() && weight.numel() == x.size(1) && bias.numel() == x.size(1),
                "LayerNorm weight / bias must match x");
    TORCH_CHECK(!q8_ptrs.empty() && !scale_ptrs.empty(), "destination lists must not be empty");
    same_device(x, weight, "add_layernorm_pack");
    same_device(x, bias, "add_layernorm_pack");
    c10::cuda::CUDAGuard guard(x.device());
    check_clip("add_layernorm_pack");
    TORCH_CHECK(chunk_scale_enabled(), "add_layernorm_pack needs BSI_FIXED_CHUNK_SCALE=1");
    const void* dptr = nullptr;
    at::Tensor d;
    if (delta.has_value() && delta->defined()) {
        d = delta->contiguous();
        TORCH_CHECK(d.sizes() == x.sizes() && d.scalar_type() == x.scalar_type(), "delta must match x");
        dptr = d.data_ptr();
    }
    at::Tensor out = dptr != nullptr ? at::empty_like(x) : x;
    std::vector<int8_t*> q;
    std::vector<float*> sc;
    for (int64_t p : q8_ptrs) q.push_back(reinterpret_cast<int8_t*>(static_cast<intptr_t>(p)));
    for (int64_t p : scale_ptrs) sc.push_back(reinterpret_cast<float*>(static_cast<intptr_t>(p)));
    check_status(bsi_b200_add_layernorm_pack(x.data_ptr(), dptr, weight.data_ptr(), bias.data_ptr(), static_cast<float>(eps),
                                             dtype_code(x), x.size(0), x.size(1), out.data_ptr(), decimalPlaces,
                                             bits_queries(), static_cast<int>(q.size()), q.data(), ld8,
                                             static_cast<int>(sc.size()), sc.data(), scale_ld, current_stream()),
                 "bsi_b200_add_layernorm_pack");
    return out;
}

py::dict debug_batch(const PackedBatch& b) {
    py::dict d;
    d["words"] = b.words;
    d["slice_weights"] = b.slice_weights;
    d["scales"] = b.scales;
    d["q8"] = b.q8;
    if (b.sq_norms.defined()) d["sq_norms"] = b.sq_norms;
    d["chunk_mode"] = b.chunk_mode;
    d["S"] = b.S;
    d["W"] = b.W;
    d["decimals"] = b.decimals;
    return d;
}

py::dict debug_query_batch_tensors(py::capsule cap) {
    return debug_batch(from_capsule<PrebuiltBSIQueryBatchCUDA>(cap, "PrebuiltBSIQueryBatchCUDA")->b);
}
py::dict debug_keys_tensors(py::capsule cap) {
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(cap, "PrebuiltBSIKeysCUDA");
    py::dict d = debug_batch(keys->b);
    if (keys->abs_sum.defined()) d["abs_sum"] = keys->abs_sum;   // [2, R]: what register_key_bounds is given
    return d;
}
py::dict debug_query_tensors(py::capsule cap) {
    auto* q = from_capsule<PrebuiltBSIQueryCUDA>(cap, "PrebuiltBSIQueryCUDA");
    py::dict d;
    d["words"] = q->parent->words[q->row];
    d["slice_weights"] = q->parent->slice_weights[q->row];
    d["scales"] = q->parent->scales[q->row];
    d["twos_complement"] = q->twos_complement;
    d["mem_bytes"] = q->mem_bytes;
    return d;
}

// (out, int32 per-chunk accumulators [Q, R, chunks]) for the bit-exactness checks.
py::tuple debug_dot_iacc(py::capsule query_batch_cap, py::capsule keyset_cuda_cap) {
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(keyset_cuda_cap, "PrebuiltBSIKeysCUDA");
    auto* qb = from_capsule<PrebuiltBSIQueryBatchCUDA>(query_batch_cap, "PrebuiltBSIQueryBatchCUDA");
    at::Tensor iacc;
    py::tuple r = run_dot(qb->b, *keys, true, &iacc);
    return py::make_tuple(r[0], iacc);
}

py::tuple ewah_encode_words(torch::Tensor words2d, double threshold) {
    EwahStream e = ewah_encode(words2d, threshold);
    return py::make_tuple(e.stream, e.off, e.len, e.flags);
}

at::Tensor ewah_decode_words(torch::Tensor stream, torch::Tensor off, torch::Tensor len, int64_t W) {
    EwahStream e;
    e.stream = stream.contiguous();
    e.off = off.contiguous();
    e.len = len.contiguous();
    return ewah_decode(e, W);
}

// ---- keyset persistence ---------------------------------------------------------------------------
// One file per key set, `<dir>/keyset.bsik`, holding what the dot needs in its stored form: the per-row scales and
// the bit slices as EWAH / verbatim streams (the encoder of this library, with the key set's compress threshold).
// It takes the place of the reference's save_keyset (bsiFunctions.cpp:792-808: one HybridBitmap file per slice, a
// bsiCPP format) and of its checkpoint scripts, which store the dense weights and quantise again on every load
// (benchmarks/export_bsi_checkpoint.py:57-87). Little-endian:
//   0  char[8]  "BSIKEYS\0"      8  u32 version (1)      12 u32 header bytes (80)
//   16 u64 num_keys   24 u64 d    32 u32 W   36 u32 bits  40 i32 decimal places   44 f32 compress threshold
//   48 u64 stream words           56 u64 FNV-1a of the payload     64 u32 flags (bit 0: variable-slice keys)   68.. zero
//   payload: f32 scale[num_keys] (2^shift of each row), i32 len[num_keys * bits] (encoded words per slice, in
//   row-major slice order; a slice starts where the previous one ends), u64 stream[stream words]
struct KeysetHeader {
    char magic[8];
    uint32_t version, header_bytes;
    uint64_t num_keys, d;
    uint32_t W, bits;
    int32_t decimals;
    float threshold;
    uint64_t stream_words, checksum;
    uint32_t flags, reserved0;
    uint64_t reserved1;
};
static_assert(sizeof(KeysetHeader) == 80, "keyset header layout");

uint64_t fnv1a(uint64_t h, const void* data, size_t n) {
    const unsigned char* p = static_cast<const unsigned char*>(data);
    for (size_t i = 0; i < n; ++i) {
        h ^= p[i];
        h *= 1099511628211ull;
    }
    return h;
}

std::string keyset_path(const std::string& dir_or_file) {
    const std::string suffix = ".bsik";
    if (dir_or_file.size() > suffix.size() && dir_or_file.compare(dir_or_file.size() - suffix.size(), suffix.size(), suffix) == 0)
        return dir_or_file;
    return dir_or_file + "/keyset.bsik";
}

struct KeysetImage {
    KeysetHeader h;
    at::Tensor scales, len, stream;   // host tensors: float32 [R], int32 [R * bits], int64 [stream words]
};

KeysetImage encode_keyset(const PrebuiltBSIKeysCUDA& keys) {
    const PackedBatch& b = keys.b;
    TORCH_CHECK(!b.chunk_mode && b.words.defined(), "key sets carry one scale per row and their bit slices");
    KeysetImage img;
    EwahStream e = ewah_encode(b.words.view({b.rows * b.S, b.W}), keys.threshold);
    img.scales = b.scales.to(at::kCPU).contiguous();
    img.len = e.len.to(at::kCPU).contiguous();
    img.stream = e.stream.to(at::kCPU).contiguous();
    std::memset(&img.h, 0, sizeof(img.h));
    std::memcpy(img.h.magic, "BSIKEYS", 8);
    img.h.version = 1;
    img.h.header_bytes = sizeof(KeysetHeader);
    img.h.num_keys = static_cast<uint64_t>(b.rows);
    img.h.d = static_cast<uint64_t>(b.d);
    img.h.W = static_cast<uint32_t>(b.W);
    img.h.bits = static_cast<uint32_t>(b.S);
    img.h.decimals = b.decimals;
    img.h.threshold = keys.threshold;
    img.h.stream_words = static_cast<uint64_t>(e.total);
    img.h.flags = b.variable ? 1u : 0u;
    uint64_t c = 1469598103934665603ull;
    c = fnv1a(c, img.scales.data_ptr(), img.scales.numel() * 4);
    c = fnv1a(c, img.len.data_ptr(), img.len.numel() * 4);
    c = fnv1a(c, img.stream.data_ptr(), img.stream.numel() * 8);
    img.h.checksum = c;
    return img;
}

// (bytes of the verbatim slices in device memory, bytes of the file): keyset_size_on_disk of the reference
// (bsiFunctions.cpp:776-790) for a CUDA key set.
py::tuple keyset_size_on_disk(py::capsule keyset_cuda_cap) {
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(keyset_cuda_cap, "PrebuiltBSIKeysCUDA");
    TORCH_CHECK(keys != nullptr, "Invalid CUDA keys capsule");
    KeysetImage img = encode_keyset(*keys);
    const uint64_t disk = sizeof(KeysetHeader) + img.scales.numel() * 4 + img.len.numel() * 4 + img.stream.numel() * 8;
    const uint64_t mem = static_cast<uint64_t>(keys->b.words.numel() * keys->b.words.element_size());
    return py::make_tuple(mem, disk);
}

py::none save_keyset(py::capsule keyset_cuda_cap, const std::string& out_dir) {
    auto* keys = from_capsule<PrebuiltBSIKeysCUDA>(keyset_cuda_cap, "PrebuiltBSIKeysCUDA");
    TORCH_CHECK(keys != nullptr, "Invalid CUDA keys capsule");
    KeysetImage img = encode_keyset(*keys);
    const std::string path = keyset_path(out_dir);
    if (path != out_dir) std::filesystem::create_directories(out_dir);
    std::ofstream ofs(path, std::ios::binary | std::ios::trunc);
    TORCH_CHECK(ofs.good(), "Failed to open file: ", path);
    ofs.write(reinterpret_cast<const char*>(&img.h), sizeof(img.h));
    ofs.write(static_cast<const char*>(img.scales.data_ptr()), img.scales.numel() * 4);
    ofs.write(static_cast<const char*>(img.len.data_ptr()), img.len.numel() * 4);
    ofs.write(static_cast<const char*>(img.stream.data_ptr()), img.stream.numel() * 8);
    ofs.close();
    TORCH_CHECK(ofs.good(), "Failed to write file: ", path);
    return py::none();
}

// Reads a key set written by save_keyset onto the current CUDA device: decodes the slice streams, rebuilds the int8
// image from the slices and returns what build_bsi_keys_cuda returns, without touching the dense weights.
py::tuple load_keyset(const std::string& dir_or_file) {
    const std::string path = keyset_path(dir_or_file);
    std::ifstream ifs(path, std::ios::binary);
    TORCH_CHECK(ifs.good(), "Failed to open file: ", path);
    KeysetHeader h;
    ifs.read(reinterpret_cast<char*>(&h), sizeof(h));
    TORCH_CHECK(ifs.good() && std::memcmp(h.magic, "BSIKEYS", 8) == 0, path, " is not a BSI key set file");
    TORCH_CHECK(h.version == 1 && h.header_bytes == sizeof(KeysetHeader), path, ": unsupported key set version ", h.version);
    TORCH_CHECK(h.bits >= 2 && h.bits <= 8 && h.W >= 1 && h.W == (h.d + 63) / 64 && h.num_keys < (1ull << 40) &&
                    h.stream_words <= h.num_keys * h.bits * (static_cast<uint64_t>(h.W) + 1),
                path, ": inconsistent key set header");
    const int64_t R = static_cast<int64_t>(h.num_keys), S = h.bits, W = h.W;
    auto cpu = [](at::ScalarType t) { return at::TensorOptions().dtype(t).device(at::kCPU); };
    at::Tensor scales = at::empty({R}, cpu(at::kFloat));
    at::Tensor len = at::empty({R * S}, cpu(at::kInt));
    at::Tensor stream = at::empty({static_cast<int64_t>(h.stream_words)}, cpu(at::kLong));
    ifs.read(static_cast<char*>(scales.data_ptr()), R * 4);
    ifs.read(static_cast<char*>(len.data_ptr()), R * S * 4);
    ifs.read(static_cast<char*>(stream.data_ptr()), static_cast<std::streamsize>(h.stream_words) * 8);
    TORCH_CHECK(ifs.good(), path, ": file is shorter than its header says");
    uint64_t c = 1469598103934665603ull;
    c = fnv1a(c, scales.data_ptr(), R * 4);
    c = fnv1a(c, len.data_ptr(), R * S * 4);
    c = fnv1a(c, stream.data_ptr(), h.stream_words * 8);
    TORCH_CHECK(c == h.checksum, path, ": checksum mismatch (file damaged)");
    // every slice must decode to at most W words from within the stream
    {
        const int32_t* lp = len.data_ptr<int32_t>();
        uint64_t sum = 0;
        for (int64_t i = 0; i < R * S; ++i) {
            TORCH_CHECK(lp[i] >= 1 && lp[i] <= W + 1, path, ": slice length out of range");
            sum += static_cast<uint64_t>(lp[i]);
        }
        TORCH_CHECK(sum == h.stream_words, path, ": slice lengths do not add up to the stream");
    }

    const auto dev = at::Device(at::kCUDA, c10::cuda::current_device());
    auto* holder = new PrebuiltBSIKeysCUDA();
    PackedBatch& b = holder->b;
    b.rows = R;
    b.d = static_cast<int64_t>(h.d);
    b.S = static_cast<int>(S);
    b.W = static_cast<int>(W);
    b.chunks = (b.d + 255) / 256;
    b.decimals = h.decimals;
    b.chunk_mode = false;
    EwahStream e;
    e.len = len.to(dev);
    e.off = (at::cumsum(e.len.to(at::kLong), 0) - e.len.to(at::kLong)).contiguous();
    e.stream = h.stream_words > 0 ? stream.to(dev) : at::zeros({1}, at::TensorOptions().dtype(at::kLong).device(dev));
    e.total = static_cast<int64_t>(h.stream_words);
    b.words = ewah_decode(e, W).view({R, S, W});
    b.scales = scales.to(dev);
    const int64_t ld8 = std::max<int64_t>(b.chunks, 1) * 256;
    b.q8 = at::empty({R, ld8}, at::TensorOptions().dtype(at::kChar).device(dev));
    if (R > 0)
        check_status(bsi_b200_recombine_i8(reinterpret_cast<const uint64_t*>(b.words.data_ptr<int64_t>()), R, b.S, W,
                                           b.q8.data_ptr<int8_t>(), ld8, current_stream()),
                     "bsi_b200_recombine_i8");
    b.slice_weights = (slice_weight_base(b.S, dev).unsqueeze(0) * b.scales.unsqueeze(1)).contiguous();
    if (h.flags & 1u) {   // variable-slice keys: the per-row slice counts follow from the integers again
        b.variable = true;
        at::Tensor amax = b.q8.to(at::kInt).abs().amax(1).to(at::kCPU).contiguous();
        b.row_slices.resize(static_cast<size_t>(R));
        for (int64_t r = 0; r < R; ++r)
            b.row_slices[static_cast<size_t>(r)] = variable_slices(static_cast<uint64_t>(amax.data_ptr<int>()[r]));
    }
    holder->num_keys = R;
    holder->threshold = h.threshold;
    holder->compute_bounds();
    const uint64_t total_mem_bytes = static_cast<uint64_t>(b.words.numel() * b.words.element_size());
    py::capsule cap(holder, "PrebuiltBSIKeysCUDA", [](PyObject* c) {
        delete reinterpret_cast<PrebuiltBSIKeysCUDA*>(PyCapsule_GetPointer(c, "PrebuiltBSIKeysCUDA"));
    });
    return py::make_tuple(cap, total_mem_bytes, holder->num_keys, b.d, b.W);
}

int device_status() {
    int v = 0;
    check_status(bsi_b200_device_status(&v), "bsi_b200_device_status");
    return v;
}

}  // namespace

PYBIND11_MODULE(bsi_ops, m) {
    m.attr("CUDA_BUILDER_VERSION") = cuda_builder_version();
    m.def("cuda_builder_version", &cuda_builder_version);
    m.def("build_bsi_query_cuda", &build_bsi_query_cuda, py::arg("q"), py::arg("decimal_places"),
          py::arg("compress_threshold") = 0.2f, "Build BSI query vector on CUDA");
    m.def("build_bsi_queries_cuda_batch", &build_bsi_queries_cuda_batch, py::arg("q2d"), py::arg("decimal_places"),
          py::arg("compress_threshold") = 0.2f, "Build BSI queries for a batch on CUDA");
    m.def("build_bsi_queries_cuda_batch_packed", &build_bsi_queries_cuda_batch_packed, py::arg("q2d"),
          py::arg("decimal_places"), py::arg("compress_threshold") = 0.2f,
          "Build a packed (batched) BSI query object on CUDA (no per-row capsules)");
    m.def("get_last_query_build_profile_cuda",
          []() { return py::make_tuple(g_last_quantize_ns, g_last_pack_ns, g_last_total_ns); },
          "Return (quantize_ns, pack_ns, total_ns) for the last CUDA query-batch build");
    m.def("reset_last_query_build_profile_cuda", []() { g_last_quantize_ns = g_last_pack_ns = g_last_total_ns = 0; },
          "Reset last CUDA query-batch build profile counters to zero");
    m.def("build_bsi_query_cuda_hybrid", &build_bsi_query_cuda_hybrid, py::arg("q"), py::arg("decimal_places"),
          py::arg("compress_threshold") = 0.2, "Build BSI query with EWAH compression");
    m.def("batch_dot_product_multiquery_cuda_caps", &batch_dot_product_multiquery_cuda_caps,
          py::arg("query_caps_list"), py::arg("keyset_cuda_cap"), "Multi-query batch dot product");
    m.def("batch_dot_product_multiquery_cuda_batch_caps", &batch_dot_product_multiquery_cuda_batch_caps,
          py::arg("query_batch_cap"), py::arg("keyset_cuda_cap"), "Packed-batch multi-query dot product");
    m.def("bsi_keys_cuda_stats", &bsi_keys_cuda_stats, py::arg("keyset_cuda_cap"),
          "Return shape/group stats for a CUDA BSI keyset");
    m.def("bsi_query_caps_stats", &bsi_query_caps_stats, py::arg("query_caps_list"),
          "Return shape stats for a list of CUDA BSI query capsules");
    m.def("build_bsi_keys_cuda", &build_bsi_keys_cuda, py::arg("K"), py::arg("decimal_places"),
          py::arg("compress_threshold") = 0.2f, "Build BSI keys and prepack to CUDA");

    m.def("bsi_linear_forward", &bsi_linear_forward, py::arg("x2d"), py::arg("keyset_cuda_cap"),
          py::arg("bias") = py::none(), py::arg("decimal_places") = 2,
          "pack + dot + cast + bias for one linear layer");
    m.def("pack_queries_into", &pack_queries_into, py::arg("x2d"), py::arg("q8"), py::arg("scales"),
          py::arg("decimal_places"), "Pack activations into caller-owned int8 / chunk-scale tensors");
    m.def("linear_from_packed", &linear_from_packed, py::arg("q8"), py::arg("scales"), py::arg("keyset_cuda_cap"),
          py::arg("bias"), py::arg("decimal_places"), py::arg("out_dtype"), py::arg("relu") = false,
          "Dot of packed activations with a key set, cast + bias (+ ReLU) fused");
    m.def("peer_alloc", &peer_alloc, py::arg("nbytes"), "Zero-filled device buffer other local processes can map: (uint8 tensor, handle bytes)");
    m.def("peer_open", &peer_open, py::arg("handle"), "Map a peer's buffer; returns its device address here");
    m.def("peer_close", &peer_close, py::arg("ptr"));
    m.def("peer_barrier", &peer_barrier, py::arg("flag_ptrs"), py::arg("rank"), py::arg("timeout_ms") = 2000,
          "Bounded flag barrier over the ranks, enqueued on the current stream");
    m.def("linear_from_packed_requant", &linear_from_packed_requant, py::arg("q8"), py::arg("scales"),
          py::arg("keyset_cuda_cap"), py::arg("bias"), py::arg("decimal_places"), py::arg("layer_dtype"), py::arg("relu"),
          py::arg("q8_ptrs"), py::arg("ld8"), py::arg("scale_ptrs"), py::arg("scale_ld"));
    m.def("add_layernorm_pack", &add_layernorm_pack, py::arg("x"), py::arg("delta"), py::arg("weight"), py::arg("bias"),
          py::arg("eps"), py::arg("q8_ptrs"), py::arg("ld8"), py::arg("scale_ptrs"), py::arg("scale_ld"), py::arg("decimal_places"));
    m.def("pack_queries_multi", &pack_queries_multi, py::arg("x2d"), py::arg("q8_ptrs"), py::arg("ld8"),
          py::arg("scale_ptrs"), py::arg("scale_ld"), py::arg("decimal_places"));
    m.def("linear_from_packed_scatter", &linear_from_packed_scatter, py::arg("q8"), py::arg("scales"),
          py::arg("keyset_cuda_cap"), py::arg("bias"), py::arg("decimal_places"), py::arg("out_dtype"), py::arg("relu"),
          py::arg("y_ptrs"), py::arg("rows_per_dst"), py::arg("ldy"));
    m.def("debug_query_batch_tensors", &debug_query_batch_tensors);
    m.def("debug_keys_tensors", &debug_keys_tensors);
    m.def("debug_query_tensors", &debug_query_tensors);
    m.def("debug_dot_iacc", &debug_dot_iacc);
    m.def("ewah_encode_words", &ewah_encode_words, py::arg("words"), py::arg("threshold"));
    m.def("ewah_decode_words", &ewah_decode_words, py::arg("stream"), py::arg("off"), py::arg("len"), py::arg("W"));
    m.def("save_keyset", &save_keyset, py::arg("keyset_cuda_cap"), py::arg("out_dir"),
          "Serialize a CUDA key set to <out_dir>/keyset.bsik (scales + EWAH / verbatim slice streams)");
    m.def("load_keyset", &load_keyset, py::arg("dir_or_file"),
          "Load a key set written by save_keyset; returns (capsule, total_mem_bytes, num_keys, d, W)");
    m.def("keyset_size_on_disk", &keyset_size_on_disk, py::arg("keyset_cuda_cap"), "Return (mem_in_memory, bytes_on_disk)");
    m.def("device_status", &device_status, "Read and clear the device-side timeout status word (synchronises)");
}
