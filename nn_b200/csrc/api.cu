// C ABI of libnnq_b200 (see include/nnq.h): contexts, weights, validation and dispatch.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <new>

#include "nnq_internal.h"
#include "gemm_tc.h"
#include "skinny.h"

namespace nnq {

nnq_status fail(nnq_ctx *ctx, nnq_status s, const char *fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->last_error, sizeof(ctx->last_error), fmt, ap);
        va_end(ap);
    }
    return s;
}

nnq_status check_cuda(nnq_ctx *ctx, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return NNQ_OK;
    cudaGetLastError();   // the error has been taken here: a later launch check must not meet it again
    nnq_status s = e == cudaErrorMemoryAllocation ? NNQ_ERR_OUT_OF_MEMORY : NNQ_ERR_DISPATCH_FAILED;
    return fail(ctx, s, "%s: %s", what, cudaGetErrorString(e));
}

static size_t elem_size(int dt) { return dt == NNQ_F32 ? 4 : 2; }

static nnq_status set_device(nnq_ctx *ctx) {
    return check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
}

// Validation shared by nnq_weight_create and the shard constructor; mirrors
// QuantizedStorage::new (element count % block, byte length == blocks * block bytes).
static nnq_status validate_weight(nnq_ctx *ctx, int fmt, const void *data, size_t nbytes,
                                  const void *scales, size_t scales_nbytes, int64_t n, int64_t k) {
    if (fmt < 0 || fmt >= NNQ_FORMAT_COUNT) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", fmt);
    if (n < 0 || k < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative dimension [%lld, %lld]", (long long)n, (long long)k);
    Geometry g = geometry(fmt);
    if ((n * k) % g.elems != 0)
        return fail(ctx, NNQ_ERR_INVALID_SHAPE, "element count %lld is not a multiple of the block size %d",
                    (long long)(n * k), g.elems);
    if (k % g.elems != 0)
        return fail(ctx, NNQ_ERR_INVALID_SHAPE, "in_features %lld is not a multiple of the block size %d",
                    (long long)k, g.elems);
    size_t blocks = (size_t)n * (size_t)(k / g.elems);
    if (nbytes != blocks * (size_t)g.bytes)
        return fail(ctx, NNQ_ERR_DATA_LENGTH, "data length mismatch: expected %zu bytes, got %zu",
                    blocks * (size_t)g.bytes, nbytes);
    if (scales_nbytes != blocks * (size_t)g.scale_bytes)
        return fail(ctx, NNQ_ERR_DATA_LENGTH, "scale length mismatch: expected %zu bytes, got %zu",
                    blocks * (size_t)g.scale_bytes, scales_nbytes);
    if (nbytes && !data) return fail(ctx, NNQ_ERR_INVALID_ARG, "data is NULL");
    if (scales_nbytes && !scales) return fail(ctx, NNQ_ERR_INVALID_ARG, "scales is NULL");
    return NNQ_OK;
}

// Waits for everything queued on the context's host stream. The event is polled: a blocking
// stream synchronisation costs an interrupt round trip, which dominates a call that moves a few KB.
static nnq_status wait_host_stream(nnq_ctx *ctx) {
    nnq_status s = check_cuda(ctx, cudaEventRecord(ctx->host_event, ctx->host_stream), "event record");
    if (s != NNQ_OK) return s;
    for (;;) {
        cudaError_t e = cudaEventQuery(ctx->host_event);
        if (e == cudaSuccess) return NNQ_OK;
        if (e != cudaErrorNotReady) return check_cuda(ctx, e, "sync");
    }
}

static nnq_status finish_weight(nnq_ctx *ctx, nnq_weight *w) {
    // Build the tiled copy when a skinny kernel exists for this format and shape, and make the
    // bf16 scratch of the large-prefill GEMM large enough for this weight.
    nnq_status s = build_tiled(ctx, w);
    if (s == NNQ_OK && w->d_raw) s = dense_scratch_reserve(ctx, w->n, w->k);
    return s;
}

}  // namespace nnq

using namespace nnq;

extern "C" {

int nnq_version(void) { return NNQ_VERSION_MAJOR * 1000 + NNQ_VERSION_MINOR; }

const char *nnq_status_str(nnq_status s) {
    switch (s) {
        case NNQ_OK: return "ok";
        case NNQ_ERR_INVALID_ARG: return "invalid argument";
        case NNQ_ERR_NOT_QUANTIZED: return "weight tensor is not quantized";
        case NNQ_ERR_WRONG_QUANT_TYPE: return "weight quantization type mismatch";
        case NNQ_ERR_SHAPE_MISMATCH: return "quantized matmul shape mismatch";
        case NNQ_ERR_WEIGHT_RANK: return "quantized weight must be 2-D [out_features, in_features]";
        case NNQ_ERR_BIAS_MISMATCH: return "bias shape mismatch";
        case NNQ_ERR_INVALID_SHAPE: return "invalid shape";
        case NNQ_ERR_DATA_LENGTH: return "data length mismatch";
        case NNQ_ERR_RANK_MISMATCH: return "rank mismatch";
        case NNQ_ERR_UNSUPPORTED: return "unsupported";
        case NNQ_ERR_VALUE_OUT_OF_RANGE: return "value out of range";
        case NNQ_ERR_OUT_OF_MEMORY: return "backend failure: out of memory";
        case NNQ_ERR_DISPATCH_FAILED: return "backend failure: dispatch failed";
        case NNQ_ERR_TIMEOUT: return "backend failure: timeout";
        case NNQ_ERR_NO_DEVICE: return "backend failure: no usable CUDA device";
        case NNQ_ERR_OTHER: return "backend failure: other";
    }
    return "unknown status";
}

nnq_status nnq_format_geometry(nnq_format fmt, int *block_elems, int *block_bytes, int *scale_bytes) {
    if ((int)fmt < 0 || fmt >= NNQ_FORMAT_COUNT) return NNQ_ERR_INVALID_ARG;
    Geometry g = geometry(fmt);
    if (block_elems) *block_elems = g.elems;
    if (block_bytes) *block_bytes = g.bytes;
    if (scale_bytes) *scale_bytes = g.scale_bytes;
    return NNQ_OK;
}

nnq_status nnq_init(int device, nnq_ctx **out) {
    if (!out) return NNQ_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0 || device < 0 || device >= count) {
        cudaGetLastError();
        return NNQ_ERR_NO_DEVICE;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return NNQ_ERR_NO_DEVICE;
    if (prop.major != 10) return NNQ_ERR_NO_DEVICE;  // kernels are built for sm_100a only
    nnq_ctx *ctx = new (std::nothrow) nnq_ctx();
    if (!ctx) return NNQ_ERR_OUT_OF_MEMORY;
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->path = NNQ_PATH_AUTO;
    nnq_status s = set_device(ctx);
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMalloc(&ctx->d_status, sizeof(int)), "cudaMalloc status");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemset(ctx->d_status, 0, sizeof(int)), "cudaMemset status");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaStreamCreateWithFlags(&ctx->host_stream, cudaStreamNonBlocking), "stream");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaEventCreateWithFlags(&ctx->host_event, cudaEventDisableTiming), "event");
    if (s == NNQ_OK) {
        // split-K partial sums of the tensor path: at most SMs output tiles of 512 x 128 f32
        ctx->partials_bytes = (size_t)ctx->sm_count * 512 * 128 * sizeof(float);
        s = check_cuda(ctx, cudaMalloc(&ctx->d_partials, ctx->partials_bytes), "cudaMalloc split-K scratch");
        if (s != NNQ_OK) ctx->partials_bytes = 0;
    }
    if (s == NNQ_OK) s = skinny_init(ctx);
    if (s != NNQ_OK) {
        nnq_destroy(ctx);
        return s;
    }
    *out = ctx;
    return NNQ_OK;
}

void nnq_destroy(nnq_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    cudaFree(ctx->d_status);
    cudaFree(ctx->d_partials);
    cudaFree(ctx->d_dense);
    cudaFree(ctx->d_moe);
    cudaFree(ctx->d_counters);
    cudaFree(ctx->d_batch_desc);
    cudaFreeHost(ctx->h_batch_desc);
    cudaFreeHost(ctx->h_stage_x);
    cudaFreeHost(ctx->h_stage_y);
    cudaFree(ctx->d_stage_x);
    cudaFree(ctx->d_stage_y);
    cudaFree(ctx->d_stage_bias);
    if (ctx->host_event) cudaEventDestroy(ctx->host_event);
    if (ctx->host_stream) cudaStreamDestroy(ctx->host_stream);
    cudaGetLastError();
    delete ctx;
}

const char *nnq_last_error(const nnq_ctx *ctx) { return ctx ? ctx->last_error : ""; }

nnq_status nnq_set_path(nnq_ctx *ctx, nnq_path path) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if ((int)path < NNQ_PATH_AUTO || path > NNQ_PATH_TENSOR) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown path %d", (int)path);
    ctx->path = path;
    return NNQ_OK;
}

nnq_status nnq_device_status(nnq_ctx *ctx, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    nnq_status s = set_device(ctx);
    if (s != NNQ_OK) return s;
    int v = 0;
    cudaStream_t st = (cudaStream_t)stream;
    s = check_cuda(ctx, cudaMemcpyAsync(&v, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, st), "status read");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaStreamSynchronize(st), "status sync");
    if (s != NNQ_OK) return s;
    if (v == 0) return NNQ_OK;
    check_cuda(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(int), st), "status clear");
    cudaStreamSynchronize(st);
    if (v == 1) return fail(ctx, NNQ_ERR_TIMEOUT, "a bounded device wait ran out (device status word = 1)");
    if (v == 2) return fail(ctx, NNQ_ERR_UNSUPPORTED, "a decoder was stepped past its last position (max_seq): its context is full, reset it");
    return fail(ctx, NNQ_ERR_OTHER, "device status word = %d", v);
}

int64_t nnq_launch_count(const nnq_ctx *ctx) { return ctx ? ctx->launches : 0; }

// ---- weights ------------------------------------------------------------------------

static nnq_status alloc_weight(nnq_ctx *ctx, int fmt, int64_t n, int64_t k, size_t nbytes,
                               size_t scales_nbytes, nnq_weight **out) {
    nnq_weight *w = new (std::nothrow) nnq_weight();
    if (!w) return fail(ctx, NNQ_ERR_OUT_OF_MEMORY, "host allocation failed");
    memset(w, 0, sizeof(*w));
    w->ctx = ctx;
    w->fmt = fmt;
    w->n = n;
    w->k = k;
    w->nbytes = nbytes;
    w->scales_nbytes = scales_nbytes;
    nnq_status s = NNQ_OK;
    // +16 bytes of slack so that 16-byte vector loads of the last partial chunk stay in bounds
    if (nbytes) s = check_cuda(ctx, cudaMalloc(&w->d_raw, nbytes + 16), "cudaMalloc weight");
    if (s == NNQ_OK && scales_nbytes) s = check_cuda(ctx, cudaMalloc(&w->d_scales, scales_nbytes + 16), "cudaMalloc scales");
    if (s != NNQ_OK) {
        nnq_weight_destroy(w);
        return s;
    }
    *out = w;
    return NNQ_OK;
}

nnq_status nnq_weight_create(nnq_ctx *ctx, nnq_format fmt, const void *data, size_t nbytes,
                             const void *scales, size_t scales_nbytes, int64_t n, int64_t k,
                             nnq_weight **out) {
    if (!ctx || !out) return NNQ_ERR_INVALID_ARG;
    *out = nullptr;
    nnq_status s = validate_weight(ctx, fmt, data, nbytes, scales, scales_nbytes, n, k);
    if (s != NNQ_OK) return s;
    if ((s = set_device(ctx)) != NNQ_OK) return s;
    nnq_weight *w = nullptr;
    if ((s = alloc_weight(ctx, fmt, n, k, nbytes, scales_nbytes, &w)) != NNQ_OK) return s;
    if (nbytes) s = check_cuda(ctx, cudaMemcpy(w->d_raw, data, nbytes, cudaMemcpyDefault), "weight upload");
    if (s == NNQ_OK && scales_nbytes)
        s = check_cuda(ctx, cudaMemcpy(w->d_scales, scales, scales_nbytes, cudaMemcpyDefault), "scales upload");
    if (s == NNQ_OK) s = finish_weight(ctx, w);
    if (s != NNQ_OK) {
        nnq_weight_destroy(w);
        return s;
    }
    *out = w;
    return NNQ_OK;
}

nnq_status nnq_weight_create_shard(nnq_ctx *ctx, nnq_format fmt, const void *data, size_t nbytes,
                                   const void *scales, size_t scales_nbytes, int64_t n, int64_t k,
                                   int axis, int rank, int world, nnq_weight **out) {
    if (!ctx || !out) return NNQ_ERR_INVALID_ARG;
    *out = nullptr;
    nnq_status s = validate_weight(ctx, fmt, data, nbytes, scales, scales_nbytes, n, k);
    if (s != NNQ_OK) return s;
    if (world < 1 || rank < 0 || rank >= world || (axis != 0 && axis != 1))
        return fail(ctx, NNQ_ERR_INVALID_ARG, "bad shard spec axis=%d rank=%d world=%d", axis, rank, world);
    Geometry g = geometry(fmt);
    int64_t kb = k / g.elems;
    if ((s = set_device(ctx)) != NNQ_OK) return s;
    nnq_weight *w = nullptr;
    if (axis == 0) {
        if (n % world) return fail(ctx, NNQ_ERR_INVALID_SHAPE, "out_features %lld not divisible by %d ranks", (long long)n, world);
        int64_t ns = n / world;
        size_t row_b = (size_t)kb * g.bytes, row_s = (size_t)kb * g.scale_bytes;
        if ((s = alloc_weight(ctx, fmt, ns, k, ns * row_b, ns * row_s, &w)) != NNQ_OK) return s;
        if (w->nbytes)
            s = check_cuda(ctx, cudaMemcpy(w->d_raw, (const uint8_t *)data + (size_t)rank * ns * row_b, w->nbytes, cudaMemcpyDefault), "shard upload");
        if (s == NNQ_OK && w->scales_nbytes)
            s = check_cuda(ctx, cudaMemcpy(w->d_scales, (const uint8_t *)scales + (size_t)rank * ns * row_s, w->scales_nbytes, cudaMemcpyDefault), "shard scales upload");
    } else {
        // K is dealt out in units of whole blocks -- of 256 weights when K is a multiple of 256, so that
        // every shard keeps a tiled layout -- rank r taking units [r * U / world, (r + 1) * U / world):
        // the shards may differ by one unit (Qwen3-32B's down_proj: 100 super-blocks over 8 ranks = 13 or 12)
        const int64_t per_unit = (k % 256 == 0 && 256 % g.elems == 0) ? 256 / g.elems : 1;
        const int64_t units = kb / per_unit;
        if (units < world) return fail(ctx, NNQ_ERR_INVALID_SHAPE, "%lld units of K cannot be split over %d ranks", (long long)units, world);
        const int64_t b0 = (rank * units / world) * per_unit, b1 = ((rank + 1) * units / world) * per_unit;
        const int64_t kbs = b1 - b0;
        size_t row_b = (size_t)kb * g.bytes, row_s = (size_t)kb * g.scale_bytes;
        size_t sh_b = (size_t)kbs * g.bytes, sh_s = (size_t)kbs * g.scale_bytes;
        if ((s = alloc_weight(ctx, fmt, n, kbs * g.elems, n * sh_b, n * sh_s, &w)) != NNQ_OK) return s;
        if (w->nbytes)
            s = check_cuda(ctx, cudaMemcpy2D(w->d_raw, sh_b, (const uint8_t *)data + (size_t)b0 * g.bytes, row_b, sh_b, n, cudaMemcpyDefault), "shard upload");
        if (s == NNQ_OK && w->scales_nbytes)
            s = check_cuda(ctx, cudaMemcpy2D(w->d_scales, sh_s, (const uint8_t *)scales + (size_t)b0 * g.scale_bytes, row_s, sh_s, n, cudaMemcpyDefault), "shard scales upload");
    }
    if (s == NNQ_OK) s = finish_weight(ctx, w);
    if (s != NNQ_OK) {
        nnq_weight_destroy(w);
        return s;
    }
    *out = w;
    return NNQ_OK;
}

void nnq_weight_destroy(nnq_weight *w) {
    if (!w) return;
    if (w->ctx) cudaSetDevice(w->ctx->device);
    cudaFree(w->d_raw);
    cudaFree(w->d_scales);
    cudaFree(w->d_tiled);
    cudaGetLastError();
    delete w;
}

nnq_status nnq_weight_info(const nnq_weight *w, nnq_format *fmt, int64_t *n, int64_t *k,
                           size_t *nbytes, size_t *scales_nbytes) {
    if (!w) return NNQ_ERR_NOT_QUANTIZED;
    if (fmt) *fmt = (nnq_format)w->fmt;
    if (n) *n = w->n;
    if (k) *k = w->k;
    if (nbytes) *nbytes = w->nbytes;
    if (scales_nbytes) *scales_nbytes = w->scales_nbytes;
    return NNQ_OK;
}

// ---- dequantization -----------------------------------------------------------------

nnq_status nnq_dequantize(nnq_ctx *ctx, const nnq_weight *w, float *dst_dev, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (!w) return fail(ctx, NNQ_ERR_NOT_QUANTIZED, "weight tensor is not quantized");
    if (!dst_dev && w->n * w->k) return fail(ctx, NNQ_ERR_INVALID_ARG, "dst is NULL");
    nnq_status s = set_device(ctx);
    if (s != NNQ_OK) return s;
    Geometry g = geometry(w->fmt);
    return launch_dequant_raw(ctx, w->fmt, w->d_raw, w->d_scales, w->n * (w->k / g.elems), dst_dev,
                              (cudaStream_t)stream);
}

nnq_status nnq_dequantize_raw(nnq_ctx *ctx, nnq_format fmt, const void *src_dev, size_t nbytes,
                              const void *scales_dev, size_t scales_nbytes, int64_t num_elements,
                              float *dst_dev, int64_t *decoded, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if ((int)fmt < 0 || fmt >= NNQ_FORMAT_COUNT) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", (int)fmt);
    if (num_elements < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative element count");
    Geometry g = geometry(fmt);
    // number of whole blocks: limited by the element count and by the bytes present
    int64_t nb = num_elements / g.elems;
    int64_t have = (int64_t)(nbytes / (size_t)g.bytes);
    if (have < nb) nb = have;
    if (g.scale_bytes) {
        int64_t have_s = (int64_t)(scales_nbytes / (size_t)g.scale_bytes);
        if (have_s < nb) nb = have_s;
    }
    if (decoded) *decoded = nb * g.elems;
    if (nb == 0) return NNQ_OK;
    if (!src_dev || !dst_dev || (g.scale_bytes && !scales_dev)) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    bool vec16 = fmt == NNQ_Q4_K || fmt == NNQ_Q4_K_GGML || fmt == NNQ_MXFP4_SPLIT || fmt == NNQ_MXFP4_GPTOSS || fmt == NNQ_Q5_K || fmt == NNQ_F32_DENSE || fmt == NNQ_BF16_DENSE;
    if (vec16 && ((uintptr_t)src_dev & 15u)) return fail(ctx, NNQ_ERR_INVALID_ARG, "source must be 16-byte aligned for this format");
    nnq_status s = set_device(ctx);
    if (s != NNQ_OK) return s;
    return launch_dequant_raw(ctx, fmt, (const uint8_t *)src_dev, (const uint8_t *)scales_dev, nb, dst_dev,
                              (cudaStream_t)stream);
}

nnq_status nnq_quantize(nnq_ctx *ctx, nnq_format fmt, const float *src_dev, int64_t num_elements, void *dst_dev,
                        size_t dst_nbytes, void *scales_dev, size_t scales_nbytes, int64_t *blocks, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if ((int)fmt < 0 || fmt >= NNQ_FORMAT_COUNT) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", (int)fmt);
    if (fmt != NNQ_Q4_K_GGML && fmt != NNQ_MXFP4_CORE && fmt != NNQ_MXFP4_GPTOSS)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "no encoder for format %d", (int)fmt);
    if (num_elements < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative element count");
    Geometry g = geometry(fmt);
    const int64_t nb = (num_elements + g.elems - 1) / g.elems;
    if (blocks) *blocks = nb;
    if (nb == 0) return NNQ_OK;
    if (!src_dev || !dst_dev || (g.scale_bytes && !scales_dev)) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    if (dst_nbytes < (size_t)nb * g.bytes || (g.scale_bytes && scales_nbytes < (size_t)nb * g.scale_bytes))
        return fail(ctx, NNQ_ERR_DATA_LENGTH, "output holds fewer than %lld blocks", (long long)nb);
    if (((uintptr_t)dst_dev & 15u) || ((uintptr_t)src_dev & 3u)) return fail(ctx, NNQ_ERR_INVALID_ARG, "output must be 16-byte aligned");
    nnq_status s = set_device(ctx);
    if (s != NNQ_OK) return s;
    return launch_quantize(ctx, fmt, src_dev, num_elements, (uint8_t *)dst_dev, (uint8_t *)scales_dev, (cudaStream_t)stream);
}

// ---- the product --------------------------------------------------------------------

static nnq_status linear_checked(nnq_ctx *ctx, const nnq_weight *w, const void *x_dev, nnq_dtype x_dt,
                                 int64_t m, const float *bias_dev, void *y_dev, nnq_dtype y_dt) {
    if (!w) return fail(ctx, NNQ_ERR_NOT_QUANTIZED, "weight tensor is not quantized");
    if (w->ctx != ctx) return fail(ctx, NNQ_ERR_INVALID_ARG, "weight belongs to another context");
    if (m < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative row count");
    if ((int)x_dt < 0 || x_dt > NNQ_BF16 || (int)y_dt < 0 || y_dt > NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown dtype");
    if (m && w->k && !x_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "x is NULL");
    if (m && w->n && !y_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "y is NULL");
    if (((uintptr_t)x_dev & 15u) || ((uintptr_t)y_dev & 15u)) return fail(ctx, NNQ_ERR_INVALID_ARG, "x and y must be 16-byte aligned");
    return NNQ_OK;
}

static nnq_status linear_dispatch(nnq_ctx *ctx, const nnq_weight *w, const void *x_dev, nnq_dtype x_dt,
                                  int64_t m, const float *bias_dev, void *y_dev, nnq_dtype y_dt,
                                  cudaStream_t stream) {
    if (m == 0 || w->n == 0) return NNQ_OK;
    int path = ctx->path;
    bool skinny_ok = skinny_supported(w, m, x_dt);
    if (path == NNQ_PATH_SKINNY && !skinny_ok)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "skinny path does not cover format %d, N=%lld, K=%lld, M=%lld",
                    w->fmt, (long long)w->n, (long long)w->k, (long long)m);
    // Up to twice the rows the token-column kernel takes at once: two passes over the weight (the second
    // one mostly from L2) are still ahead of the tensor path, which decodes a 128-row tile for them
    // (Q4_K 4096 x 4096 at 32 rows: 2 x 7 us against 25 us; 12288 x 4096: 2 x 18 against 46).
    const int64_t cols = x_dt == NNQ_BF16 ? 16 : 8;
    if (path == NNQ_PATH_AUTO && !skinny_ok && m > cols && m <= 2 * cols && skinny_supported(w, cols, x_dt) &&
        skinny_supported(w, m - cols, x_dt)) {
        const size_t xe = x_dt == NNQ_BF16 ? 2 : 4, ye = y_dt == NNQ_BF16 ? 2 : 4;
        SkinnyJob lo = {w, x_dev, bias_dev, y_dev};
        SkinnyJob hi = {w, static_cast<const uint8_t *>(x_dev) + (size_t)cols * w->k * xe, bias_dev,
                        static_cast<uint8_t *>(y_dev) + (size_t)cols * w->n * ye};
        nnq_status s = launch_skinny(ctx, &lo, 1, x_dt, cols, y_dt, stream);
        return s != NNQ_OK ? s : launch_skinny(ctx, &hi, 1, x_dt, m - cols, y_dt, stream);
    }
    const bool tc_ok = gemm_tc_supported(w, m);
    if (path == NNQ_PATH_TENSOR && !tc_ok)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "tensor path needs K to be a multiple of 64 (K=%lld)", (long long)w->k);
    if (path == NNQ_PATH_TENSOR || (path == NNQ_PATH_AUTO && !skinny_ok && tc_ok && (m > 16 || (m >= 5 && x_dt == NNQ_BF16)))) {
        TcArgs a = {w->d_raw, w->d_scales, x_dev, bias_dev, y_dev, m, w->n, w->k, w->fmt, x_dt, y_dt};
        // hundreds of rows per weight row: decode once to bf16, then the plain GEMM
        if (gemm_dense_supported(ctx, w, m, x_dt)) return launch_gemm_dense(ctx, a, stream);
        return launch_gemm_tc(ctx, a, stream);
    }
    if ((path == NNQ_PATH_AUTO && skinny_ok) || path == NNQ_PATH_SKINNY) {
        SkinnyJob job = {w, x_dev, bias_dev, y_dev};
        return launch_skinny(ctx, &job, 1, x_dt, m, y_dt, stream);
    }
    if (w->k == 0) {
        // empty reduction: y = bias or 0
        LinearArgs a = {w->d_raw, w->d_scales, x_dev, bias_dev, y_dev, m, w->n, 0, w->fmt, x_dt, y_dt};
        return launch_linear_generic(ctx, a, stream);
    }
    LinearArgs a = {w->d_raw, w->d_scales, x_dev, bias_dev, y_dev, m, w->n, w->k, w->fmt, x_dt, y_dt};
    return launch_linear_generic(ctx, a, stream);
}

nnq_status nnq_linear(nnq_ctx *ctx, const nnq_weight *w, const void *x_dev, nnq_dtype x_dt, int64_t m,
                      const float *bias_dev, void *y_dev, nnq_dtype y_dt, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    nnq_status s = linear_checked(ctx, w, x_dev, x_dt, m, bias_dev, y_dev, y_dt);
    if (s != NNQ_OK) return s;
    if ((s = set_device(ctx)) != NNQ_OK) return s;
    return linear_dispatch(ctx, w, x_dev, x_dt, m, bias_dev, y_dev, y_dt, (cudaStream_t)stream);
}

nnq_status nnq_linear_batch(nnq_ctx *ctx, int count, const nnq_weight *const *w, const void *const *x_dev,
                            nnq_dtype x_dt, int64_t m, const float *const *bias_dev, void *const *y_dev,
                            nnq_dtype y_dt, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (count < 0 || (count && (!w || !x_dev || !y_dev))) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad batch arguments");
    nnq_status s;
    bool all_skinny = count > 0 && ctx->path != NNQ_PATH_GENERIC && ctx->path != NNQ_PATH_TENSOR;
    for (int i = 0; i < count; i++) {
        s = linear_checked(ctx, w[i], x_dev[i], x_dt, m, bias_dev ? bias_dev[i] : nullptr, y_dev[i], y_dt);
        if (s != NNQ_OK) return s;
        all_skinny = all_skinny && skinny_supported(w[i], m, x_dt) && w[i]->fmt == w[0]->fmt;
    }
    if ((s = set_device(ctx)) != NNQ_OK) return s;
    if (m == 0) return NNQ_OK;
    if (all_skinny && count <= kSkinnyMaxJobs) {
        SkinnyJob jobs[kSkinnyMaxJobs];
        for (int i = 0; i < count; i++) jobs[i] = {w[i], x_dev[i], bias_dev ? bias_dev[i] : nullptr, y_dev[i]};
        return launch_skinny(ctx, jobs, count, x_dt, m, y_dt, (cudaStream_t)stream);
    }
    for (int i = 0; i < count; i++) {
        s = linear_dispatch(ctx, w[i], x_dev[i], x_dt, m, bias_dev ? bias_dev[i] : nullptr, y_dev[i], y_dt,
                            (cudaStream_t)stream);
        if (s != NNQ_OK) return s;
    }
    return NNQ_OK;
}

// Results of at most this many bytes are written by the kernels straight into the pinned host
// buffer (it is mapped into the device's address space), which saves the device-to-host copy
// operation and its hand-over between the compute and copy engines; larger results go through
// device memory and one bulk copy. The outputs are write-only in every product kernel.
constexpr size_t kZeroCopyOutBytes = 1 << 20;

static void *mapped_output(nnq_ctx *ctx, size_t bytes) {
    static const char *env = diag_env("NNQ_HOST_ZEROCOPY");   // measurement aid: 0 keeps the copy
    if ((env && atoi(env) == 0) || bytes > kZeroCopyOutBytes) return nullptr;
    void *dev = nullptr;
    if (cudaHostGetDevicePointer(&dev, ctx->h_stage_y, 0) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return dev;
}

// Small inputs are pulled from the mapped pinned buffer by a copy kernel instead of a copy-engine
// operation: the product kernel then follows a kernel on its own engine (no engine hand-over).
constexpr size_t kKernelCopyInBytes = 256 << 10;

__global__ void __launch_bounds__(256) stage_in_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, size_t n16) {
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n16; i += (size_t)gridDim.x * 256) dst[i] = src[i];
}

// Queues the copy of the staged inputs (a multiple of 16 bytes is available in both buffers).
static nnq_status stage_in(nnq_ctx *ctx, size_t bytes, cudaStream_t st) {
    if (!ctx->h_stage_x || !ctx->d_stage_x || bytes > ctx->stage_x_bytes)
        return fail(ctx, NNQ_ERR_OUT_OF_MEMORY, "staging buffers are not allocated");
    static const char *env = diag_env("NNQ_HOST_KERNEL_COPY");   // measurement aid: 0 keeps the copy engine
    void *src = nullptr;
    if (!(env && atoi(env) == 0) && bytes <= kKernelCopyInBytes &&
        cudaHostGetDevicePointer(&src, ctx->h_stage_x, 0) == cudaSuccess) {
        const size_t n16 = (bytes + 15) / 16;
        const int grid = (int)((n16 + 255) / 256 < 16 ? (n16 + 255) / 256 : 16);
        stage_in_kernel<<<grid, 256, 0, st>>>((const uint4 *)src, (uint4 *)ctx->d_stage_x, n16);
        ctx->launches++;
        return check_cuda(ctx, cudaGetLastError(), "stage-in launch");
    }
    cudaGetLastError();
    return check_cuda(ctx, cudaMemcpyAsync(ctx->d_stage_x, ctx->h_stage_x, bytes, cudaMemcpyHostToDevice, st), "h2d");
}

static nnq_status grow(nnq_ctx *ctx, void **p, size_t *cap, size_t need, bool pinned_host) {
    if (need <= *cap) return NNQ_OK;
    size_t want = need < 4096 ? 4096 : (need + need / 2 + 255) & ~(size_t)255;
    if (*p) {
        if (pinned_host) cudaFreeHost(*p); else cudaFree(*p);
        *p = nullptr;
        *cap = 0;
    }
    cudaError_t e = pinned_host ? cudaHostAlloc(p, want, cudaHostAllocMapped | cudaHostAllocPortable) : cudaMalloc(p, want);
    if (e != cudaSuccess) return check_cuda(ctx, e, "staging allocation");
    *cap = want;
    return NNQ_OK;
}

// Makes the staging pairs (pinned host + device) hold in_bytes / out_bytes. The recorded capacity
// of a pair is dropped to zero BEFORE its buffers are replaced, so a failed allocation leaves the
// context saying "no staging" (the next call allocates again) rather than a stale size over a
// freed pointer.
static nnq_status grow_staging(nnq_ctx *ctx, size_t in_bytes, size_t out_bytes) {
    nnq_status s;
    if (in_bytes > ctx->stage_x_bytes || !ctx->h_stage_x || !ctx->d_stage_x) {
        size_t cap_h = 0, cap_d = 0;
        ctx->stage_x_bytes = 0;
        if (ctx->h_stage_x) cudaFreeHost(ctx->h_stage_x);
        if (ctx->d_stage_x) cudaFree(ctx->d_stage_x);
        ctx->h_stage_x = ctx->d_stage_x = nullptr;
        if ((s = grow(ctx, &ctx->h_stage_x, &cap_h, in_bytes, true)) != NNQ_OK) return s;
        if ((s = grow(ctx, &ctx->d_stage_x, &cap_d, in_bytes, false)) != NNQ_OK) return s;
        ctx->stage_x_bytes = cap_h < cap_d ? cap_h : cap_d;
    }
    if (out_bytes > ctx->stage_y_bytes || !ctx->h_stage_y || !ctx->d_stage_y) {
        size_t cap_h = 0, cap_d = 0;
        ctx->stage_y_bytes = 0;
        if (ctx->h_stage_y) cudaFreeHost(ctx->h_stage_y);
        if (ctx->d_stage_y) cudaFree(ctx->d_stage_y);
        ctx->h_stage_y = ctx->d_stage_y = nullptr;
        if ((s = grow(ctx, &ctx->h_stage_y, &cap_h, out_bytes, true)) != NNQ_OK) return s;
        if ((s = grow(ctx, &ctx->d_stage_y, &cap_d, out_bytes, false)) != NNQ_OK) return s;
        ctx->stage_y_bytes = cap_h < cap_d ? cap_h : cap_d;
    }
    return NNQ_OK;
}

nnq_status nnq_linear_host(nnq_ctx *ctx, const nnq_weight *w, const void *x_host, nnq_dtype x_dt, int64_t m,
                           const float *bias_host, void *y_host, nnq_dtype y_dt) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (!w) return fail(ctx, NNQ_ERR_NOT_QUANTIZED, "weight tensor is not quantized");
    if (m < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative row count");
    if ((int)x_dt < 0 || x_dt > NNQ_BF16 || (int)y_dt < 0 || y_dt > NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown dtype");
    if (m == 0 || w->n == 0) return NNQ_OK;
    if (!x_host || !y_host) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL host buffer");
    nnq_status s = set_device(ctx);
    if (s != NNQ_OK) return s;
    size_t xb = (size_t)m * w->k * elem_size(x_dt), yb = (size_t)m * w->n * elem_size(y_dt);
    size_t bb = bias_host ? (size_t)w->n * 4 : 0;
    // staging: [x | bias] share the pinned input buffer so that one copy moves both
    size_t in_bytes = ((xb + 15) & ~(size_t)15) + bb;
    if ((s = grow_staging(ctx, in_bytes, yb)) != NNQ_OK) return s;
    cudaStream_t st = ctx->host_stream;
    memcpy(ctx->h_stage_x, x_host, xb);
    size_t boff = (xb + 15) & ~(size_t)15;
    if (bb) memcpy((uint8_t *)ctx->h_stage_x + boff, bias_host, bb);
    s = stage_in(ctx, in_bytes, st);
    if (s != NNQ_OK) return s;
    const float *bias_dev = bb ? (const float *)((uint8_t *)ctx->d_stage_x + boff) : nullptr;
    void *direct = mapped_output(ctx, yb);
    void *y_dev = direct ? direct : ctx->d_stage_y;
    s = linear_checked(ctx, w, ctx->d_stage_x, x_dt, m, bias_dev, y_dev, y_dt);
    if (s == NNQ_OK) s = linear_dispatch(ctx, w, ctx->d_stage_x, x_dt, m, bias_dev, y_dev, y_dt, st);
    if (s != NNQ_OK) return s;
    if (!direct) s = check_cuda(ctx, cudaMemcpyAsync(ctx->h_stage_y, ctx->d_stage_y, yb, cudaMemcpyDeviceToHost, st), "d2h");
    if (s == NNQ_OK) s = wait_host_stream(ctx);
    if (s != NNQ_OK) return s;
    memcpy(y_host, ctx->h_stage_y, yb);
    return NNQ_OK;
}

nnq_status nnq_linear_batch_host(nnq_ctx *ctx, int count, const nnq_weight *const *w, const void *const *x_host,
                                 nnq_dtype x_dt, int64_t m, const float *const *bias_host, void *const *y_host,
                                 nnq_dtype y_dt) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    constexpr int kMaxBatch = 16;
    if (count < 0 || count > kMaxBatch || (count && (!w || !x_host || !y_host))) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad batch arguments");
    if (m < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative row count");
    if ((int)x_dt < 0 || x_dt > NNQ_BF16 || (int)y_dt < 0 || y_dt > NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown dtype");
    if (count == 0 || m == 0) return NNQ_OK;
    nnq_status s = set_device(ctx);
    if (s != NNQ_OK) return s;
    // layout of the staging buffers: every distinct activation pointer once, then the biases;
    // products that share their host activations also share the device copy (and one launch)
    size_t x_off[kMaxBatch], b_off[kMaxBatch], y_off[kMaxBatch];
    size_t in_bytes = 0, out_bytes = 0;
    for (int i = 0; i < count; i++) {
        if (!w[i]) return fail(ctx, NNQ_ERR_NOT_QUANTIZED, "weight tensor is not quantized");
        if (!x_host[i] || !y_host[i]) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL host buffer");
        int same = -1;
        for (int j = 0; j < i; j++)
            if (x_host[j] == x_host[i] && w[j]->k == w[i]->k) same = j;
        if (same >= 0) {
            x_off[i] = x_off[same];
        } else {
            x_off[i] = in_bytes;
            in_bytes += ((size_t)m * w[i]->k * elem_size(x_dt) + 255) & ~(size_t)255;
        }
        y_off[i] = out_bytes;
        out_bytes += ((size_t)m * w[i]->n * elem_size(y_dt) + 255) & ~(size_t)255;
    }
    for (int i = 0; i < count; i++) {
        b_off[i] = in_bytes;
        if (bias_host && bias_host[i]) in_bytes += ((size_t)w[i]->n * 4 + 255) & ~(size_t)255;
    }
    if ((s = grow_staging(ctx, in_bytes, out_bytes)) != NNQ_OK) return s;
    const void *xd[kMaxBatch];
    const float *bd[kMaxBatch];
    void *yd[kMaxBatch];
    void *direct = mapped_output(ctx, out_bytes);
    uint8_t *y_base = direct ? (uint8_t *)direct : (uint8_t *)ctx->d_stage_y;
    for (int i = 0; i < count; i++) {
        bool first = true;
        for (int j = 0; j < i; j++) first = first && x_off[j] != x_off[i];
        if (first) memcpy((uint8_t *)ctx->h_stage_x + x_off[i], x_host[i], (size_t)m * w[i]->k * elem_size(x_dt));
        xd[i] = (uint8_t *)ctx->d_stage_x + x_off[i];
        bd[i] = nullptr;
        if (bias_host && bias_host[i]) {
            memcpy((uint8_t *)ctx->h_stage_x + b_off[i], bias_host[i], (size_t)w[i]->n * 4);
            bd[i] = (const float *)((uint8_t *)ctx->d_stage_x + b_off[i]);
        }
        yd[i] = y_base + y_off[i];
    }
    cudaStream_t st = ctx->host_stream;
    s = stage_in(ctx, in_bytes, st);
    if (s != NNQ_OK) return s;
    s = nnq_linear_batch(ctx, count, w, xd, x_dt, m, bd, yd, y_dt, st);
    if (s != NNQ_OK) return s;
    if (!direct) s = check_cuda(ctx, cudaMemcpyAsync(ctx->h_stage_y, ctx->d_stage_y, out_bytes, cudaMemcpyDeviceToHost, st), "d2h");
    if (s == NNQ_OK) s = wait_host_stream(ctx);
    if (s != NNQ_OK) return s;
    for (int i = 0; i < count; i++) memcpy(y_host[i], (uint8_t *)ctx->h_stage_y + y_off[i], (size_t)m * w[i]->n * elem_size(y_dt));
    return NNQ_OK;
}

}  // extern "C"
