// Tensor-core (tcgen05 / TMEM) prefill product: internal declarations.
#pragma once
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

// K must be a multiple of 64 (one 128-byte swizzle row of bf16 per stage).
bool gemm_tc_supported(const nnq_weight *w, int64_t m);
nnq_status launch_gemm_tc(nnq_ctx *ctx, const TcArgs &a, cudaStream_t stream);

}  // namespace nnq
