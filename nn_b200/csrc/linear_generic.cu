// Portable dequant-fused product on the RAW block layout: one warp per output row, the
// row's 32-weight chunks spread over the lanes, f32 FMA accumulation, shuffle reduction.
// It covers every format, every M and any N; the tiled kernels replace it where they
// apply. x is re-read from L2 for every row; weights are decoded once per tile of 8 tokens.
#include <cuda_bf16.h>

#include "decode.cuh"

namespace nnq {

constexpr int kRowWarps = 8;

template <typename XT>
__device__ __forceinline__ void load_x32(const XT *p, float *xv);

template <>
__device__ __forceinline__ void load_x32<float>(const float *p, float *xv) {
    const float4 *q = reinterpret_cast<const float4 *>(p);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float4 v = __ldg(q + i);
        xv[4 * i] = v.x; xv[4 * i + 1] = v.y; xv[4 * i + 2] = v.z; xv[4 * i + 3] = v.w;
    }
}

template <>
__device__ __forceinline__ void load_x32<__nv_bfloat16>(const __nv_bfloat16 *p, float *xv) {
    const uint4 *q = reinterpret_cast<const uint4 *>(p);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint4 v = __ldg(q + i);
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            xv[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
            xv[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
    }
}

template <int FMT, int MT, typename XT>
__global__ void __launch_bounds__(kRowWarps * 32)
linear_generic_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ scales,
                      const XT *__restrict__ x, const float *__restrict__ bias, void *__restrict__ y,
                      int64_t M, int64_t N, int64_t K, int y_dt) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (row >= N) return;
    const int64_t cpr = K / 32;
    for (int64_t m0 = 0; m0 < M; m0 += MT) {
        float acc[MT];
#pragma unroll
        for (int t = 0; t < MT; t++) acc[t] = 0.0f;
        for (int64_t c = lane; c < cpr; c += 32) {
            float wv[32];
            Decode<FMT>::chunk(w, scales, row * cpr + c, wv);
#pragma unroll
            for (int t = 0; t < MT; t++) {
                if (m0 + t < M) {
                    float xv[32];
                    load_x32<XT>(x + (m0 + t) * K + c * 32, xv);
#pragma unroll
                    for (int i = 0; i < 32; i++) acc[t] = fmaf(wv[i], xv[i], acc[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < MT; t++) {
            float v = acc[t];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
            if (lane == 0 && m0 + t < M) {
                if (bias) v += __ldg(bias + row);
                if (y_dt == NNQ_F32)
                    reinterpret_cast<float *>(y)[(m0 + t) * N + row] = v;
                else
                    reinterpret_cast<__nv_bfloat16 *>(y)[(m0 + t) * N + row] = __float2bfloat16_rn(v);
            }
        }
    }
}

template <int FMT>
static cudaError_t launch_fmt(const LinearArgs &a, cudaStream_t stream) {
    int grid = (int)((a.n + kRowWarps - 1) / kRowWarps);
    dim3 block(kRowWarps * 32);
#define NNQ_GO(MT, XT)                                                                       \
    linear_generic_kernel<FMT, MT, XT><<<grid, block, 0, stream>>>(                           \
        a.w, a.scales, reinterpret_cast<const XT *>(a.x), a.bias, a.y, a.m, a.n, a.k, a.y_dt)
    if (a.x_dt == NNQ_F32) {
        if (a.m == 1) NNQ_GO(1, float);
        else if (a.m <= 4) NNQ_GO(4, float);
        else NNQ_GO(8, float);
    } else {
        if (a.m == 1) NNQ_GO(1, __nv_bfloat16);
        else if (a.m <= 4) NNQ_GO(4, __nv_bfloat16);
        else NNQ_GO(8, __nv_bfloat16);
    }
#undef NNQ_GO
    return cudaGetLastError();
}

nnq_status launch_linear_generic(nnq_ctx *ctx, const LinearArgs &a, cudaStream_t stream) {
    if (a.m == 0 || a.n == 0) return NNQ_OK;
    cudaError_t e;
    switch (a.fmt) {
        case NNQ_Q4_0: e = launch_fmt<NNQ_Q4_0>(a, stream); break;
        case NNQ_Q4_1: e = launch_fmt<NNQ_Q4_1>(a, stream); break;
        case NNQ_Q8_0: e = launch_fmt<NNQ_Q8_0>(a, stream); break;
        case NNQ_Q4_K: e = launch_fmt<NNQ_Q4_K>(a, stream); break;
        case NNQ_Q4_K_GGML: e = launch_fmt<NNQ_Q4_K_GGML>(a, stream); break;
        case NNQ_Q6_K: e = launch_fmt<NNQ_Q6_K>(a, stream); break;
        case NNQ_MXFP4_CORE: e = launch_fmt<NNQ_MXFP4_CORE>(a, stream); break;
        case NNQ_MXFP4_SPLIT: e = launch_fmt<NNQ_MXFP4_SPLIT>(a, stream); break;
        case NNQ_MXFP4_GPTOSS: e = launch_fmt<NNQ_MXFP4_GPTOSS>(a, stream); break;
        case NNQ_Q5_0: e = launch_fmt<NNQ_Q5_0>(a, stream); break;
        case NNQ_Q5_1: e = launch_fmt<NNQ_Q5_1>(a, stream); break;
        case NNQ_Q2_K: e = launch_fmt<NNQ_Q2_K>(a, stream); break;
        case NNQ_Q3_K: e = launch_fmt<NNQ_Q3_K>(a, stream); break;
        case NNQ_Q5_K: e = launch_fmt<NNQ_Q5_K>(a, stream); break;
        case NNQ_F32_DENSE: e = launch_fmt<NNQ_F32_DENSE>(a, stream); break;
        case NNQ_BF16_DENSE: e = launch_fmt<NNQ_BF16_DENSE>(a, stream); break;
        default: return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", a.fmt);
    }
    ctx->launches++;
    return check_cuda(ctx, e, "linear_generic launch");
}

}  // namespace nnq
