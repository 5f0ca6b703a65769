// Shared helpers of the bsi_b200 library: status codes, error recording, launch checks.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/bsi_b200.h"

namespace bsi {

// Thread-local detail of the last failure; read through bsi_b200_last_error().
void set_error(const char* fmt, ...);

inline int fail(int code, const char* what) {
    set_error("%s", what);
    return code;
}

// Checks the launch that was just enqueued (configuration errors surface here).
inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return BSI_ERR_CUDA;
    }
    return BSI_OK;
}

#define BSI_CUDA_TRY(expr)                                                        \
    do {                                                                          \
        cudaError_t _e = (expr);                                                  \
        if (_e != cudaSuccess) {                                                  \
            ::bsi::set_error("%s: %s", #expr, cudaGetErrorString(_e));            \
            return BSI_ERR_CUDA;                                                  \
        }                                                                         \
    } while (0)

// Number of SMs of the current device (cached per device).
int sm_count();

// 0 when the current device is sm_100 class, an error code otherwise.
int require_sm100();

// Destinations of a linear whose output rows are dealt out to several matrices (n = 0: plain output).
struct ScatterDst {
    int n;
    int rows_per_dst;                 // multiple of 32
    void* y[BSI_B200_MAX_PEERS];      // row q -> y[q / rows_per_dst], local row q % rows_per_dst
};

// Destinations of a linear that re-quantises its finished output (n = 0: off). The output row block of a
// tile is one 256-column chunk per row, so its chunk scale is known inside the tile.
struct RequantDst {
    int n;                 // destinations (own buffer and peer mappings alike)
    int bits;              // 7 for activations
    float mult;            // 10^decimal_places, at most 1000
    int64_t ld8;           // row pitch of the int8 matrices (bytes)
    int64_t scale_ld;      // floats per row of the scale matrices
    int8_t* q8[BSI_B200_MAX_PEERS];      // already offset to this linear's first output column
    float* scales[BSI_B200_MAX_PEERS];   // already offset to this linear's first output chunk
};

// Bounds registered for a key image (bsi_b200_register_key_bounds): with them a dot can tell, per tile, that every
// prefix of a chunk sum stays below 2^24 in magnitude, where integer accumulation gives the float32 chain's bits.
struct KeyBounds {
    const float* abs_sum;    // [3, rows] device: sum of |k| per key row, largest sum over one chunk, sum of k^2
    int64_t rows;
    float query_abs_max;     // largest magnitude of a query integer in dots against these keys
};
bool lookup_key_bounds(const void* k8, KeyBounds* out);   // false: none registered (or BSI_B200_EXACT_INT=0)
struct QueryBounds {
    const float* sq_norms;   // per (row, chunk): (2^shift)^2 * sum of squares of the chunk's integers
    int64_t stride;          // floats per row
};
bool lookup_query_bounds(const void* a8, QueryBounds* out);

// True unless BSI_B200_PDL=0: the dot kernels are launched with programmatic stream serialisation (their set-up
// may overlap the tail of a dot kernel right before them on the stream).
bool pdl_enabled();

// Reads and clears the status word of the peer barrier kernels (0 = clean, 64 + p = gave up waiting for rank p).
int take_peer_status(int* v);

}  // namespace bsi
