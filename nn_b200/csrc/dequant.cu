// Raw-layout dequantization kernels: quantized blocks -> f32, bit-identical to the
// reference CPU decoders. HBM-bound on the 4-byte-per-weight output stream; one thread
// decodes one 32-weight chunk into shared memory and the block stores it coalesced.
#include "decode.cuh"

namespace nnq {

constexpr int kDeqThreads = 128;

template <int FMT>
__global__ void __launch_bounds__(kDeqThreads)
dequant_raw_kernel(const uint8_t *__restrict__ src, const uint8_t *__restrict__ scales,
                   int64_t nchunks, float *__restrict__ dst) {
    __shared__ float tile[kDeqThreads * 33];
    for (int64_t base = (int64_t)blockIdx.x * kDeqThreads; base < nchunks;
         base += (int64_t)gridDim.x * kDeqThreads) {
        int64_t c = base + threadIdx.x;
        if (c < nchunks) {
            float o[32];
            Decode<FMT>::chunk(src, scales, c, o);
#pragma unroll
            for (int i = 0; i < 32; i++) tile[threadIdx.x * 33 + i] = o[i];
        }
        __syncthreads();
        int64_t remaining = nchunks - base;
        int live = remaining < kDeqThreads ? (int)remaining : kDeqThreads;
        float *out = dst + base * 32;
        for (int idx = threadIdx.x; idx < live * 32; idx += kDeqThreads)
            out[idx] = tile[(idx >> 5) * 33 + (idx & 31)];
        __syncthreads();
    }
}

template <int FMT>
static cudaError_t launch(const uint8_t *src, const uint8_t *scales, int64_t nchunks, float *dst,
                          int sm_count, cudaStream_t stream) {
    int64_t want = (nchunks + kDeqThreads - 1) / kDeqThreads;
    int64_t cap = (int64_t)sm_count * 16;
    int grid = (int)(want < cap ? want : cap);
    if (grid < 1) grid = 1;
    dequant_raw_kernel<FMT><<<grid, kDeqThreads, 0, stream>>>(src, scales, nchunks, dst);
    return cudaGetLastError();
}

nnq_status launch_dequant_raw(nnq_ctx *ctx, int fmt, const uint8_t *src, const uint8_t *scales,
                              int64_t nblocks, float *dst, cudaStream_t stream) {
    if (nblocks == 0) return NNQ_OK;
    Geometry g = geometry(fmt);
    int64_t nchunks = nblocks * (g.elems / 32);
    cudaError_t e;
    switch (fmt) {
        case NNQ_Q4_0: e = launch<NNQ_Q4_0>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_Q4_1: e = launch<NNQ_Q4_1>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_Q8_0: e = launch<NNQ_Q8_0>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_Q4_K: e = launch<NNQ_Q4_K>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_Q4_K_GGML: e = launch<NNQ_Q4_K_GGML>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_Q6_K: e = launch<NNQ_Q6_K>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_MXFP4_CORE: e = launch<NNQ_MXFP4_CORE>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_MXFP4_SPLIT: e = launch<NNQ_MXFP4_SPLIT>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_MXFP4_GPTOSS: e = launch<NNQ_MXFP4_GPTOSS>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_Q5_0: e = launch<NNQ_Q5_0>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_Q5_1: e = launch<NNQ_Q5_1>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_Q2_K: e = launch<NNQ_Q2_K>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_Q3_K: e = launch<NNQ_Q3_K>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_Q5_K: e = launch<NNQ_Q5_K>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_F32_DENSE: e = launch<NNQ_F32_DENSE>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        case NNQ_BF16_DENSE: e = launch<NNQ_BF16_DENSE>(src, scales, nchunks, dst, ctx->sm_count, stream); break;
        default: return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", fmt);
    }
    ctx->launches++;
    return check_cuda(ctx, e, "dequant launch");
}

}  // namespace nnq
