// Tensor-core (tcgen05 / TMEM) prefill product: internal declarations.
#pragma once
#include <cuda_bf16.h>

#include "nnq_internal.h"

namespace nnq {

struct TcArgs {
    const uint8_t *w;       // raw blocks [N, K]
    const uint8_t *scales;  // separate scale bytes or NULL
    const void *x;
    const float *bias;
    void *y;
    int64_t m, n, k;
    int fmt, x_dt, y_dt;
};

// Grouped variant for the expert products of a mixture-of-experts block: the rows of x are sorted
// by expert (device-side offsets[e] .. offsets[e+1]), expert e multiplies its rows with the weight
// at w + e * w_stride (scales + e * s_stride) and adds bias + e * n. x is bf16 [rows_upper, k]
// (rows beyond offsets[experts] are never stored), y is f32 [rows_upper, n].
struct TcGroupArgs {
    const uint8_t *w, *scales;
    size_t w_stride, s_stride;
    const void *x_bf16;
    const float *bias;      // [experts][n] or NULL
    float *y;
    const int *offsets;     // device, [experts + 1]
    int experts;
    int64_t rows_upper;     // upper bound of offsets[experts] (allocation size of x and y in rows)
    int64_t n, k;
    int fmt;
    // decode-once path only: with h_out given and an MXFP4 format the product is the gate / up product
    // of an expert block (n = 2 * inter, gate rows first) and its epilogue writes
    // h_out[row, j] = clamp(silu(gate_j), +-swiglu_limit) * up_j in bf16 instead of y
    // (gemm_dense_grouped_fuses_swiglu tells)
    __nv_bfloat16 *h_out = nullptr;
    float swiglu_limit = 0.0f;
    // decode-once path only: the experts are nn-gptoss [experts, K, N] MXFP4 tensors (codes [E, K, N / 2],
    // scale bytes [E, K, N / 32], blocks along N); the decode transposes them into the [N, K] copy
    bool kn = false;
};
bool gemm_dense_grouped_fuses_swiglu(const TcGroupArgs &g);
nnq_status launch_gemm_tc_grouped(nnq_ctx *ctx, const TcGroupArgs &a, cudaStream_t stream);

// K must be a multiple of 64 (one 128-byte swizzle row of bf16 per stage).
bool gemm_tc_supported(const nnq_weight *w, int64_t m);
nnq_status launch_gemm_tc(nnq_ctx *ctx, const TcArgs &a, cudaStream_t stream);

// Large prefill (M >= 256, bf16 activations, K a multiple of 64): decode the weight to bf16 in the
// context's scratch, then a persistent TMA + tcgen05 GEMM (gemm_dense.cu).
bool gemm_dense_supported(const nnq_ctx *ctx, const nnq_weight *w, int64_t m, int x_dt);
nnq_status dense_scratch_reserve(nnq_ctx *ctx, int64_t n, int64_t k);
nnq_status launch_gemm_dense(nnq_ctx *ctx, const TcArgs &a, cudaStream_t stream);
// the GEMM alone over an already decoded bf16 [n, k] weight (a.w / a.fmt are not read)
nnq_status launch_gemm_dense_bf16(nnq_ctx *ctx, const void *w_bf16, const TcArgs &a, cudaStream_t stream);
bool gemm_dense_shape_ok(const nnq_ctx *ctx, int64_t m, int64_t n, int64_t k, int x_dt);
// the expert products of a prefill-sized MoE call: all local experts decoded at once
bool gemm_dense_grouped_supported(const nnq_ctx *ctx, const TcGroupArgs &g);
nnq_status launch_gemm_dense_grouped(nnq_ctx *ctx, const TcGroupArgs &g, cudaStream_t stream);

}  // namespace nnq
