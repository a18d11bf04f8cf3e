// INT8 per-channel weights (W8A16): the reference's quantize_per_channel / dequantize_per_channel
// (crates/nn-core/src/layers/quantized/int8.rs:82-221) and Int8Linear::forward
// (int8_linear.rs:175-213) on the buffer contract of its GPU kernel spec
// (crates/nn-metal/src/int8_gemm_msl.rs:35-52): W u8 [N, K] read as signed, scale f32 [N],
// zero_point i32 [N], f32 accumulation, w = (f32(q) - f32(zp)) * scale.
//
// The product streams one byte per weight: a warp owns an output row, lanes take 16-byte chunks
// of it, bytes become floats with one byte-permute and one subtraction (the zero point rides in the
// subtraction's constant), the row's scale is applied once to the reduced sum; four rows share each
// load of the activations and up to four tokens share a pass over the weights.
#include <cuda_bf16.h>
#include <math.h>

#include "nnq_internal.h"

namespace nnq {

constexpr int kI8Threads = 256;

__device__ int g_int8_error;

__device__ __forceinline__ float blk_min(float a, float b) { return b < a ? b : a; }
__device__ __forceinline__ float blk_max(float a, float b) { return b > a ? b : a; }

// `as i32` of an f32: saturating, NaN -> 0
__device__ __forceinline__ int f32_as_i32(float v) {
    if (isnan(v)) return 0;
    if (v >= 2147483648.0f) return 2147483647;
    if (v <= -2147483648.0f) return (-2147483647 - 1);
    return (int)v;
}

// One CTA per row: minimum / maximum (order-independent), then the row's parameters and codes.
__global__ void __launch_bounds__(kI8Threads)
int8_quantize_kernel(const float *__restrict__ w, int64_t n, int64_t k, int mode, uint8_t *__restrict__ q,
                     float *__restrict__ scale, int *__restrict__ zp) {
    __shared__ float s_mn[kI8Threads / 32], s_mx[kI8Threads / 32];
    __shared__ float s_scale;
    __shared__ int s_zp, s_bad;
    for (int64_t r = blockIdx.x; r < n; r += gridDim.x) {
        const float *row = w + r * k;
        float mn = INFINITY, mx = -INFINITY;
        bool bad = false;
        for (int64_t i = threadIdx.x; i < k; i += kI8Threads) {
            float v = __ldg(row + i);
            bad |= !isfinite(v);
            mn = blk_min(mn, v);
            mx = blk_max(mx, v);
        }
        if (threadIdx.x == 0) s_bad = 0;
        __syncthreads();
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            mn = blk_min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = blk_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if ((threadIdx.x & 31) == 0) { s_mn[threadIdx.x >> 5] = mn; s_mx[threadIdx.x >> 5] = mx; }
        if (bad) s_bad = 1;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int i = 1; i < kI8Threads / 32; i++) { mn = blk_min(mn, s_mn[i]); mx = blk_max(mx, s_mx[i]); }
            float sc = 0.0f;
            int z = 0;
            if (k > 0) {
                if (mode == 0) {
                    float abs_max = blk_max(blk_max(0.0f, fabsf(mn)), fabsf(mx));
                    if (abs_max != 0.0f) sc = __fdiv_rn(abs_max, 127.0f);
                } else {
                    float range = __fsub_rn(mx, mn);
                    if (range != 0.0f) {
                        sc = __fdiv_rn(range, 255.0f);
                        z = f32_as_i32(roundf(__fsub_rn(-128.0f, __fdiv_rn(mn, sc))));
                    }
                }
            }
            s_scale = sc;
            s_zp = z;
            scale[r] = sc;
            zp[r] = z;
            if (s_bad) atomicExch(&g_int8_error, 1);
        }
        __syncthreads();
        const float sc = s_scale, zf = (float)s_zp;
        for (int64_t i = threadIdx.x; i < k; i += kI8Threads) {
            int v = 0;
            if (sc != 0.0f) {
                float qf = roundf(__fadd_rn(__fdiv_rn(__ldg(row + i), sc), zf));
                qf = qf < -128.0f ? -128.0f : (qf > 127.0f ? 127.0f : qf);   // NaN passes through and casts to 0
                v = isnan(qf) ? 0 : (int)qf;
            }
            q[r * k + i] = (uint8_t)(int8_t)v;
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kI8Threads)
int8_dequantize_kernel(const uint8_t *__restrict__ q, const float *__restrict__ scale, const int *__restrict__ zp,
                       int64_t n, int64_t k, float *__restrict__ out) {
    for (int64_t r = blockIdx.y; r < n; r += gridDim.y) {
        const float sc = __ldg(scale + r), zf = (float)__ldg(zp + r);
        for (int64_t i = (int64_t)blockIdx.x * kI8Threads + threadIdx.x; i < k; i += (int64_t)gridDim.x * kI8Threads)
            out[r * k + i] = __fmul_rn(__fsub_rn((float)(int8_t)__ldg(q + r * k + i), zf), sc);
    }
}

template <typename XT>
__device__ __forceinline__ void load_x16(const XT *p, float *o);
template <>
__device__ __forceinline__ void load_x16<float>(const float *p, float *o) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float4 v = __ldg(reinterpret_cast<const float4 *>(p) + i);
        o[4 * i] = v.x; o[4 * i + 1] = v.y; o[4 * i + 2] = v.z; o[4 * i + 3] = v.w;
    }
}
template <>
__device__ __forceinline__ void load_x16<__nv_bfloat16>(const __nv_bfloat16 *p, float *o) {
#pragma unroll
    for (int i = 0; i < 2; i++) {
        uint4 v = __ldg(reinterpret_cast<const uint4 *>(p) + i);
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            o[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
            o[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}
__device__ __forceinline__ float x_at(const float *p, int64_t i) { return __ldg(p + i); }
__device__ __forceinline__ float x_at(const __nv_bfloat16 *p, int64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void y_put(float *p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void y_put(__nv_bfloat16 *p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

constexpr int kI8LinThreads = 128;
constexpr int kI8Rows = 4;   // output rows per warp: one load of the activations serves four rows

// y[t][n] = scale[n] * sum_k (q[n][k] - zp[n]) * x[t][k] (+ bias[n]) for tokens [t0, t0 + MT)
template <typename XT, typename YT, int MT, bool VEC>
__global__ void __launch_bounds__(kI8LinThreads)
int8_linear_kernel(const uint8_t *__restrict__ q, const float *__restrict__ scale, const int *__restrict__ zp,
                   const XT *__restrict__ x, const float *__restrict__ bias, YT *__restrict__ y, int64_t m, int64_t n,
                   int64_t k, int64_t t0) {
    constexpr int R = kI8Rows;
    const int lane = threadIdx.x & 31;
    const int64_t units = (n + R - 1) / R;
    const int64_t warps = (int64_t)gridDim.x * (kI8LinThreads / 32);
    for (int64_t u = (int64_t)blockIdx.x * (kI8LinThreads / 32) + (threadIdx.x >> 5); u < units; u += warps) {
        const uint8_t *row[R];
        float zf[R], c[R];
        bool fast = true;
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int64_t rr = u * R + r < n ? u * R + r : n - 1;   // rows past the end repeat the last one; not stored
            row[r] = q + rr * k;
            const int z = __ldg(zp + rr);
            zf[r] = (float)z;
            // float(byte ^ 0x80) + 2^23 minus this constant = q - zp, exact while the constant is
            c[r] = 8388608.0f + 128.0f + zf[r];
            fast = fast && z > -4000000 && z < 4000000;
        }
        float acc[R][MT];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int t = 0; t < MT; t++) acc[r][t] = 0.0f;
        const int64_t kv = VEC ? (k & ~(int64_t)15) : 0;
        for (int64_t k0 = (int64_t)lane * 16; k0 < kv; k0 += 32 * 16) {
            uint4 raw[R];
#pragma unroll
            for (int r = 0; r < R; r++) raw[r] = __ldg(reinterpret_cast<const uint4 *>(row[r] + k0));
            float xv[MT][16];
#pragma unroll
            for (int t = 0; t < MT; t++) {
                const int64_t tt = t0 + t < m ? t0 + t : m - 1;
                load_x16<XT>(x + tt * k + k0, xv[t]);
            }
#pragma unroll
            for (int r = 0; r < R; r++) {
                const uint32_t qw[4] = {raw[r].x ^ 0x80808080u, raw[r].y ^ 0x80808080u, raw[r].z ^ 0x80808080u, raw[r].w ^ 0x80808080u};
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float f = __uint_as_float(__byte_perm(qw[i >> 2], 0x4B000000u, 0x7540u + (i & 3)));
                    const float wv = fast ? __fsub_rn(f, c[r]) : __fsub_rn(__fsub_rn(f, 8388736.0f), zf[r]);
#pragma unroll
                    for (int t = 0; t < MT; t++) acc[r][t] = fmaf(wv, xv[t][i], acc[r][t]);
                }
            }
        }
        for (int64_t i = kv + lane; i < k; i += 32) {   // ragged tail, or everything when rows are not 16-byte aligned
#pragma unroll
            for (int r = 0; r < R; r++) {
                const float wv = __fsub_rn((float)(int8_t)__ldg(row[r] + i), zf[r]);
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    const int64_t tt = t0 + t < m ? t0 + t : m - 1;
                    acc[r][t] = fmaf(wv, x_at(x, tt * k + i), acc[r][t]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int64_t rr = u * R + r;
#pragma unroll
            for (int t = 0; t < MT; t++) {
                float v = acc[r][t];
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && rr < n && t0 + t < m)
                    y_put(y, (t0 + t) * n + rr, fmaf(v, __ldg(scale + rr), bias ? __ldg(bias + rr) : 0.0f));
            }
        }
    }
}

template <typename XT, typename YT, int MT>
static void launch_i8(const uint8_t *q, const float *scale, const int *zp, const void *x, const float *bias, void *y,
                      int64_t m, int64_t n, int64_t k, int64_t t0, int grid, bool vec, cudaStream_t st) {
    if (vec) int8_linear_kernel<XT, YT, MT, true><<<grid, kI8LinThreads, 0, st>>>(q, scale, zp, (const XT *)x, bias, (YT *)y, m, n, k, t0);
    else int8_linear_kernel<XT, YT, MT, false><<<grid, kI8LinThreads, 0, st>>>(q, scale, zp, (const XT *)x, bias, (YT *)y, m, n, k, t0);
}

template <typename XT, typename YT>
static void launch_i8_m(const uint8_t *q, const float *scale, const int *zp, const void *x, const float *bias, void *y,
                        int64_t m, int64_t n, int64_t k, int grid, bool vec, long long *launches, cudaStream_t st) {
    for (int64_t t0 = 0; t0 < m; t0 += 4) {   // four tokens share a pass over the weights
        const int64_t left = m - t0;
        if (left == 1) launch_i8<XT, YT, 1>(q, scale, zp, x, bias, y, m, n, k, t0, grid, vec, st);
        else if (left == 2) launch_i8<XT, YT, 2>(q, scale, zp, x, bias, y, m, n, k, t0, grid, vec, st);
        else launch_i8<XT, YT, 4>(q, scale, zp, x, bias, y, m, n, k, t0, grid, vec, st);
        (*launches)++;
    }
}

}  // namespace nnq

using namespace nnq;

extern "C" {

nnq_status nnq_int8_quantize_per_channel(nnq_ctx *ctx, const float *w_dev, int64_t n, int64_t k, int mode, void *q_dev,
                                         float *scale_dev, int32_t *zp_dev, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (n < 0 || k < 0 || (mode != 0 && mode != 1)) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad int8 quantize arguments");
    if (n == 0) return NNQ_OK;
    if (!scale_dev || !zp_dev || (k && (!w_dev || !q_dev))) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    cudaStream_t st = (cudaStream_t)stream;
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    int *flag = nullptr;
    s = check_cuda(ctx, cudaGetSymbolAddress((void **)&flag, g_int8_error), "int8 flag");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemsetAsync(flag, 0, sizeof(int), st), "int8 flag clear");
    if (s != NNQ_OK) return s;
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    int8_quantize_kernel<<<(int)(n < cap ? n : cap), kI8Threads, 0, st>>>(w_dev, n, k, mode, (uint8_t *)q_dev, scale_dev, zp_dev);
    ctx->launches++;
    s = check_cuda(ctx, cudaGetLastError(), "int8 quantize launch");
    if (s != NNQ_OK) return s;
    int raised = 0;
    s = check_cuda(ctx, cudaMemcpyAsync(&raised, flag, sizeof(int), cudaMemcpyDeviceToHost, st), "int8 flag read");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaStreamSynchronize(st), "int8 quantize synchronize");
    if (s != NNQ_OK) return s;
    if (raised) return fail(ctx, NNQ_ERR_VALUE_OUT_OF_RANGE, "quantize_per_channel: non-finite weight value");
    return NNQ_OK;
}

nnq_status nnq_int8_dequantize_per_channel(nnq_ctx *ctx, const void *q_dev, const float *scale_dev, const int32_t *zp_dev,
                                           int64_t n, int64_t k, float *dst_dev, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (n < 0 || k < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative size");
    if (n == 0 || k == 0) return NNQ_OK;
    if (!q_dev || !scale_dev || !zp_dev || !dst_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    int64_t gx = (k + kI8Threads - 1) / kI8Threads;
    dim3 grid((unsigned)(gx < 64 ? gx : 64), (unsigned)(n < 16384 ? n : 16384));
    int8_dequantize_kernel<<<grid, kI8Threads, 0, (cudaStream_t)stream>>>((const uint8_t *)q_dev, scale_dev, zp_dev, n, k, dst_dev);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "int8 dequantize launch");
}

nnq_status nnq_int8_linear(nnq_ctx *ctx, const void *q_dev, const float *scale_dev, const int32_t *zp_dev, int64_t n,
                           int64_t k, const void *x_dev, nnq_dtype x_dt, int64_t m, const float *bias_dev, void *y_dev,
                           nnq_dtype y_dt, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (n < 0 || k < 0 || m < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative size");
    if ((int)x_dt < 0 || x_dt > NNQ_BF16 || (int)y_dt < 0 || y_dt > NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown dtype");
    if (m == 0 || n == 0) return NNQ_OK;
    if (!scale_dev || !zp_dev || !y_dev || (k && (!q_dev || !x_dev))) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    // 16-byte chunks need aligned rows and activations
    const bool vec = k % 16 == 0 && !((uintptr_t)q_dev & 15u) && !((uintptr_t)x_dev & 15u);
    const int64_t units = (n + kI8Rows - 1) / kI8Rows, per_cta = kI8LinThreads / 32;
    const int64_t want = (units + per_cta - 1) / per_cta, cap = (int64_t)ctx->sm_count * 16;
    const int grid = (int)(want < cap ? want : cap);
    if (x_dt == NNQ_F32 && y_dt == NNQ_F32) launch_i8_m<float, float>((const uint8_t *)q_dev, scale_dev, zp_dev, x_dev, bias_dev, y_dev, m, n, k, grid, vec, &ctx->launches, st);
    else if (x_dt == NNQ_F32) launch_i8_m<float, __nv_bfloat16>((const uint8_t *)q_dev, scale_dev, zp_dev, x_dev, bias_dev, y_dev, m, n, k, grid, vec, &ctx->launches, st);
    else if (y_dt == NNQ_F32) launch_i8_m<__nv_bfloat16, float>((const uint8_t *)q_dev, scale_dev, zp_dev, x_dev, bias_dev, y_dev, m, n, k, grid, vec, &ctx->launches, st);
    else launch_i8_m<__nv_bfloat16, __nv_bfloat16>((const uint8_t *)q_dev, scale_dev, zp_dev, x_dev, bias_dev, y_dev, m, n, k, grid, vec, &ctx->launches, st);
    return check_cuda(ctx, cudaGetLastError(), "int8 linear launch");
}

}  // extern "C"
