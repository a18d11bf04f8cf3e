// Internal declarations shared by the translation units of libnnq_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>

#include "../../include/nnq.h"

namespace nnq {

struct Geometry {
    int elems;        // weights per block
    int bytes;        // block bytes in the main buffer
    int scale_bytes;  // block bytes in the separate scale buffer
};

__host__ __device__ inline Geometry geometry(int fmt) {
    switch (fmt) {
        case NNQ_Q4_0: return {32, 18, 0};
        case NNQ_Q4_1: return {32, 20, 0};
        case NNQ_Q8_0: return {32, 34, 0};
        case NNQ_Q4_K: return {256, 144, 0};
        case NNQ_Q4_K_GGML: return {256, 144, 0};
        case NNQ_Q6_K: return {256, 210, 0};
        case NNQ_MXFP4_CORE: return {32, 17, 0};
        case NNQ_MXFP4_SPLIT: return {32, 16, 1};
        case NNQ_MXFP4_GPTOSS: return {32, 16, 1};
        case NNQ_Q5_0: return {32, 22, 0};
        case NNQ_Q5_1: return {32, 24, 0};
        case NNQ_Q2_K: return {256, 84, 0};
        case NNQ_Q3_K: return {256, 110, 0};
        case NNQ_Q5_K: return {256, 176, 0};
        case NNQ_F32_DENSE: return {32, 128, 0};
        case NNQ_BF16_DENSE: return {32, 64, 0};
        default: return {0, 0, 0};
    }
}

// Tiled ("T16") device layouts used by the skinny kernels; kNone = raw blocks only.
enum TiledLayout { kTiledNone = 0, kTiledQ4K = 1, kTiledQ8_0 = 2, kTiledQ6K = 3, kTiledMxfp4 = 4, kTiledQ4_0 = 5, kTiledQ4_1 = 6 };

}  // namespace nnq

struct nnq_ctx {
    int device;
    int sm_count;
    int path;                 // nnq_path
    int *d_status;            // device status word (0 = clear)
    // split-K workspace of the skinny kernels: partial sums + arrival counters
    float *d_partials;
    size_t partials_bytes;
    unsigned int *d_counters;
    size_t counters_count;
    // bf16 copy of one weight at a time for the large-prefill GEMM: sized for the largest weight
    // created on this context (at weight creation, never inside a product call)
    void *d_dense;
    size_t dense_bytes;
    // scratch of the mixture-of-experts block (routing tables and intermediate activations)
    uint8_t *d_moe;
    size_t moe_bytes;
    // batched launch descriptors
    void *d_batch_desc;
    void *h_batch_desc;
    size_t batch_desc_bytes;
    // host staging for nnq_linear_host
    void *h_stage_x, *h_stage_y;
    void *d_stage_x, *d_stage_y;
    float *d_stage_bias;
    size_t stage_x_bytes, stage_y_bytes, stage_bias_bytes;
    cudaStream_t host_stream;
    cudaEvent_t host_event;   // completion of a host entry point's last copy (polled: lower latency than a blocking wait)
    long long launches;
    char last_error[512];
};

struct nnq_weight {
    nnq_ctx *ctx;
    int fmt;
    int64_t n, k;
    size_t nbytes, scales_nbytes;
    uint8_t *d_raw;      // raw blocks, reference layout (NULL when only the tiled copy is kept)
    uint8_t *d_scales;   // separate scale bytes (split MXFP4 layouts)
    uint8_t *d_tiled;    // re-tiled copy for the skinny kernels (same byte count, padded tiles)
    size_t tiled_bytes;
    int tiled_layout;    // nnq::TiledLayout
    int tile_sb;         // blocks of 32 weights per tile row (8; 6 for MXFP4 with K % 256 != 0)
};

namespace nnq {

// Tuning and diagnostic switches exist only in builds made with -DNNQ_DIAG; the shipped library
// reads no environment variable.
static inline const char *diag_env(const char *name) {
#ifdef NNQ_DIAG
    return getenv(name);
#else
    (void)name;
    return nullptr;
#endif
}

nnq_status fail(nnq_ctx *ctx, nnq_status s, const char *fmt, ...);
nnq_status check_cuda(nnq_ctx *ctx, cudaError_t e, const char *what);

// dequant.cu
nnq_status launch_dequant_raw(nnq_ctx *ctx, int fmt, const uint8_t *src, const uint8_t *scales,
                              int64_t nblocks, float *dst, cudaStream_t stream);

// quantize.cu
nnq_status launch_quantize(nnq_ctx *ctx, int fmt, const float *src, int64_t n, uint8_t *dst, uint8_t *scales,
                           cudaStream_t stream);

// linear_generic.cu
struct LinearArgs {
    const uint8_t *w;       // raw blocks
    const uint8_t *scales;  // separate scale bytes or NULL
    const void *x;
    const float *bias;
    void *y;
    int64_t m, n, k;
    int fmt, x_dt, y_dt;
};
nnq_status launch_linear_generic(nnq_ctx *ctx, const LinearArgs &a, cudaStream_t stream);

}  // namespace nnq
