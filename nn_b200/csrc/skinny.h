// Skinny (M <= 16) streaming kernels on the tiled weight layout.
#pragma once
#include "comm.cuh"
#include "nnq_internal.h"

namespace nnq {

constexpr int kSkinnyMaxJobs = 8;
constexpr int kSkinnyMaxM = 16;

struct SkinnyJob {
    const nnq_weight *w;
    const void *x;
    const float *bias;
    void *y;
};

// Per-context set-up of the skinny kernels (nothing to allocate at present).
nnq_status skinny_init(nnq_ctx *ctx);
// Builds w->d_tiled from w->d_raw when the format / shape has a skinny kernel.
nnq_status build_tiled(nnq_ctx *ctx, nnq_weight *w);
// Tiled copy of raw blocks [n, k] (NULL when the format / K has no tiled layout); *sb = blocks of
// 32 weights per tile row.
nnq_status build_tiled_buffer(nnq_ctx *ctx, int fmt, const uint8_t *d_raw, const uint8_t *d_scales, int64_t n,
                              int64_t k, uint8_t **out, size_t *out_bytes, int *sb);
// Size of the tiled copy of raw blocks [n, k] (0 when the format / K has no tiled layout) and the
// repack into a buffer of that size (asynchronous on the default stream).
size_t tiled_bytes_for(int fmt, int64_t n, int64_t k, int *sb);
nnq_status repack_into(nnq_ctx *ctx, int fmt, const uint8_t *d_raw, const uint8_t *d_scales, int64_t n, int64_t k,
                       uint8_t *dst);

// The same for an nn-gptoss [K, N] MXFP4 expert tensor (blocks along N): tiles of the transposed
// product, rows = n (a multiple of 32), scales per k inside a tile.
size_t tiled_bytes_kn(int64_t n, int64_t k, int *sb);
nnq_status repack_kn_into(nnq_ctx *ctx, const uint8_t *d_codes, const uint8_t *d_scales, int64_t n, int64_t k, uint8_t *dst);

// Expert products of a mixture-of-experts block over tiled expert weights: routed rows sorted by
// expert (offset[e] .. offset[e+1]), out[r, :] = x[row source of r, :] * W_e^T + bias_e.
struct GroupedArgs {
    const uint8_t *tiled;     // expert e at tiled + e * expert_stride
    size_t expert_stride;
    const float *bias;        // [experts][n] or NULL
    const void *x;
    int x_dt;
    const int *rowtok;        // routed row -> flat assignment index (token = index / top_k); NULL: the row itself
    const int *offset;        // device, [experts + 1]
    float *out;               // [rows][n] f32
    int experts, top_k;
    int64_t n, k;
    int fmt;
    int64_t max_rows;         // upper bound of offset[experts]
    int kn_gptoss;            // 1: tiles built from nn-gptoss [K, N] expert tensors (scales along N)
};
nnq_status launch_grouped(nnq_ctx *ctx, const GroupedArgs &a, cudaStream_t stream);

// True when launch_skinny can run this weight with M rows of activations.
bool skinny_supported(const nnq_weight *w, int64_t m, int x_dt);
// One launch computing y_i = x_i * W_i^T (+ bias_i) for all jobs (same format, same M).
nnq_status launch_skinny(nnq_ctx *ctx, const SkinnyJob *jobs, int count, int x_dt, int64_t m, int y_dt,
                         cudaStream_t stream);

// Row-parallel product fused with its all-reduce (M = 1 Q4_K kernel): the warp that finishes a row
// tile sends its 16 f32 partial sums to every peer as 8-byte (value, sequence number) stores, waits
// (bounded) for the peers' pairs of the same rows, adds them in rank order, adds the bias and
// writes y. The communicator's slots must hold 8 bytes per output row.
bool skinny_fused_supported(const nnq_weight *w, int64_t m, int x_dt);
nnq_status launch_skinny_fused(nnq_ctx *ctx, const SkinnyJob &job, int x_dt, int y_dt, const FusedReduce &fr,
                               cudaStream_t stream);

}  // namespace nnq
