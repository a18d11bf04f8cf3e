// f32 -> block encoders, bit-identical to the reference's CPU encoders:
//   NNQ_Q4_K_GGML   BlockQ4K::quantize over zero-padded 256-weight blocks
//                   (crates/nn-core/src/layers/quantized/linear.rs:95-162,178-254,318-336)
//   NNQ_MXFP4_CORE  quantize_tensor / quantize_block (crates/nn-core/src/layers/quantized/mxfp4.rs:94-207,307-329)
//   NNQ_MXFP4_GPTOSS  Mxfp4Tensor::quantize (crates/nn-gptoss/src/quantize.rs:64-153)
// The encoders are sequential per 32 weights (running sums in element order, five refinement
// passes), so one lane owns one 32-weight sub-block and keeps the reference's operation order;
// parallelism is across sub-blocks. A warp stages 1024 consecutive floats through shared memory
// (coalesced 4-byte loads, conflict-free padded rows). All arithmetic uses the explicit
// round-to-nearest intrinsics so nothing is fused. A load-time operation: HBM-bound on the
// 4-byte-per-weight input stream.
#include <cuda_fp16.h>
#include <math.h>

#include "decode.cuh"

namespace nnq {

constexpr int kQuantWarps = 4;

// raised by a kernel when the reference would return ValueOutOfRange
__device__ int g_quant_error;

__device__ __forceinline__ float fold_min(float acc, float v) { return v < acc ? v : acc; }   // NaN ignored, ties keep acc
__device__ __forceinline__ float fold_max(float acc, float v) { return v > acc ? v : acc; }

// nearest_int: round half away from zero; non-finite or beyond i32 raises the error
__device__ __forceinline__ int nearest_int(float v, bool &err) {
    if (!isfinite(v)) { err = true; return 0; }
    float r = roundf(v);
    if (r < -2147483648.0f || r > 2147483648.0f) { err = true; return 0; }
    return r >= 2147483648.0f ? 2147483647 : (int)r;
}

// make_qkx1_quants(15, 5, x[32])
__device__ __forceinline__ void make_qkx1(const float *x, float &scale_out, float &min_out, bool &err) {
    const int nmax = 15;
    uint32_t lw[4] = {0, 0, 0, 0};   // 32 four-bit levels
    float mn = INFINITY, mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i++) { mn = fold_min(mn, x[i]); mx = fold_max(mx, x[i]); }
    if (mx == mn) {
        if (mn >= 0.0f) { scale_out = __fdiv_rn(mn, (float)nmax); min_out = 0.0f; }
        else { scale_out = 0.0f; min_out = -mn; }
        return;
    }
    float min = fold_min(mn, 0.0f);
    float iscale = __fdiv_rn((float)nmax, __fsub_rn(mx, min));
    float scale = __fdiv_rn(1.0f, iscale);
    for (int t = 0; t < 5; t++) {
        float sumlx = 0.0f;
        int suml2 = 0;
        bool changed = false;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            float dv = __fsub_rn(x[i], min);
            int li = nearest_int(__fmul_rn(iscale, dv), err);
            li = li < 0 ? 0 : (li > nmax ? nmax : li);
            uint32_t old = (lw[i >> 3] >> (4 * (i & 7))) & 15u;
            if ((uint32_t)li != old) {
                lw[i >> 3] = (lw[i >> 3] & ~(15u << (4 * (i & 7)))) | ((uint32_t)li << (4 * (i & 7)));
                changed = true;
            }
            sumlx = __fadd_rn(sumlx, __fmul_rn(dv, (float)li));
            suml2 += li * li;
        }
        if (err) return;
        if (suml2 == 0) { scale_out = 0.0f; min_out = 0.0f; return; }
        scale = __fdiv_rn(sumlx, (float)suml2);
        if (scale == 0.0f) { scale_out = 0.0f; min_out = -min; return; }
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            float li = (float)((lw[i >> 3] >> (4 * (i & 7))) & 15u);
            sum = __fadd_rn(sum, __fsub_rn(x[i], __fmul_rn(scale, li)));
        }
        min = fold_min(__fdiv_rn(sum, 32.0f), 0.0f);
        iscale = __fdiv_rn(1.0f, scale);
        if (!changed) break;
    }
    scale_out = scale;
    min_out = -min;
}

// Loads the warp's 1024 floats (zero beyond `n`) and hands lane L the 32 values [32L, 32L+32).
__device__ __forceinline__ void stage_rows(const float *__restrict__ src, int64_t base, int64_t n, float *tile, float *x) {
    const int lane = threadIdx.x & 31;
#pragma unroll 8
    for (int r = 0; r < 32; r++) {
        int64_t idx = base + r * 32 + lane;
        tile[r * 33 + lane] = idx < n ? __ldg(src + idx) : 0.0f;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 32; i++) x[i] = tile[lane * 33 + i];
    __syncwarp();
}

__global__ void __launch_bounds__(kQuantWarps * 32)
quantize_q4k_ggml_kernel(const float *__restrict__ src, int64_t n, int64_t nblocks, uint8_t *__restrict__ out) {
    __shared__ float tiles[kQuantWarps][32 * 33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = lane & 7;                     // sub-block of the lane's block
    const int64_t groups = (nblocks + 3) / 4;   // a warp encodes four blocks at a time
    for (int64_t g = (int64_t)blockIdx.x * kQuantWarps + warp; g < groups; g += (int64_t)gridDim.x * kQuantWarps) {
        float x[32];
        stage_rows(src, g * 1024, n, tiles[warp], x);
        const int64_t blk = g * 4 + (lane >> 3);
        bool err = false;
        float s, m;
        make_qkx1(x, s, m, err);
        // maxima over the block's eight sub-blocks, folded in sub-block order from +0
        float max_scale = 0.0f, max_min = 0.0f;
#pragma unroll
        for (int t = 0; t < 8; t++) {
            max_scale = fold_max(max_scale, __shfl_sync(0xffffffffu, s, (lane & 24) | t));
            max_min = fold_max(max_min, __shfl_sync(0xffffffffu, m, (lane & 24) | t));
        }
        const float inv_scale = max_scale > 0.0f ? __fdiv_rn(63.0f, max_scale) : 0.0f;
        const float inv_min = max_min > 0.0f ? __fdiv_rn(63.0f, max_min) : 0.0f;
        uint32_t ls = (uint32_t)nearest_int(__fmul_rn(inv_scale, s), err) & 255u;   // `as u8`
        uint32_t lm = (uint32_t)nearest_int(__fmul_rn(inv_min, m), err) & 255u;
        ls = ls < 63u ? ls : 63u;
        lm = lm < 63u ? lm : 63u;
        const uint16_t dh = __half_as_ushort(__float2half_rn(__fdiv_rn(max_scale, 63.0f)));
        const uint16_t mh = __half_as_ushort(__float2half_rn(__fdiv_rn(max_min, 63.0f)));
        // levels of the lane's 32 weights with the packed (six-bit) scales
        uint32_t lw[4] = {0, 0, 0, 0};
        const float bd = __fmul_rn(f16_bits_to_f32(dh), (float)ls);
        if (bd != 0.0f) {
            const float bm = __fmul_rn(f16_bits_to_f32(mh), (float)lm);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                int q = nearest_int(__fdiv_rn(__fadd_rn(x[i], bm), bd), err);
                q = q < 0 ? 0 : (q > 15 ? 15 : q);
                lw[i >> 3] |= (uint32_t)q << (4 * (i & 7));
            }
        }
        // header: d, dmin and the 12 scale bytes, gathered by the block's first lane
        uint32_t sc_all[8], mn_all[8];
#pragma unroll
        for (int t = 0; t < 8; t++) {
            sc_all[t] = __shfl_sync(0xffffffffu, ls, (lane & 24) | t);
            mn_all[t] = __shfl_sync(0xffffffffu, lm, (lane & 24) | t);
        }
        // byte k of the quants of sub-block pair (2p, 2p+1): low nibble level k of 2p, high nibble level k of 2p+1
        uint32_t other[4];
#pragma unroll
        for (int w = 0; w < 4; w++) other[w] = __shfl_xor_sync(0xffffffffu, lw[w], 1);
        const bool odd = j & 1;
        uint32_t qb[4];
#pragma unroll
        for (int w = 0; w < 4; w++) {   // output word w = bytes 4w .. 4w+3 of the lane's 16
            uint32_t v = 0;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                int k = (odd ? 16 : 0) + 4 * w + b;
                uint32_t mine = (lw[k >> 3] >> (4 * (k & 7))) & 15u, theirs = (other[k >> 3] >> (4 * (k & 7))) & 15u;
                uint32_t lo = odd ? theirs : mine, hi = odd ? mine : theirs;
                v |= (lo | (hi << 4)) << (8 * b);
            }
            qb[w] = v;
        }
        const bool any_err = __any_sync(0xffffffffu, err);
        if (any_err) {
            if (lane == 0) atomicExch(&g_quant_error, 1);
            continue;
        }
        if (blk < nblocks) {
            uint8_t *o = out + blk * 144;
            if (j == 0) {
                uint32_t S[3] = {0, 0, 0};   // 12 scale bytes
                auto put = [&](int byte, uint32_t v) { S[byte >> 2] |= v << (8 * (byte & 3)); };
#pragma unroll
                for (int t = 0; t < 8; t++) {
                    if (t < 4) { put(t, sc_all[t]); put(t + 4, mn_all[t]); }
                    else {
                        put(t + 4, (sc_all[t] & 15u) | ((mn_all[t] & 15u) << 4));
                        put(t - 4, (sc_all[t] >> 4) << 6);
                        put(t, (mn_all[t] >> 4) << 6);
                    }
                }
                *reinterpret_cast<uint4 *>(o) = make_uint4((uint32_t)dh | ((uint32_t)mh << 16), S[0], S[1], S[2]);
            }
            *reinterpret_cast<uint4 *>(o + 16 + 32 * (j >> 1) + (odd ? 16 : 0)) = make_uint4(qb[0], qb[1], qb[2], qb[3]);
        }
    }
}

// nearest E2M1 magnitude by minimum distance, the first wins on ties
__device__ __forceinline__ uint32_t nearest_e2m1(float a) {
    const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    uint32_t best = 0;
    float best_dist = 3.40282347e+38f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float dist = fabsf(__fsub_rn(a, mag[i]));
        if (dist < best_dist) { best_dist = dist; best = i; }
    }
    return best;
}

template <bool GPTOSS>
__global__ void __launch_bounds__(kQuantWarps * 32)
quantize_mxfp4_kernel(const float *__restrict__ src, int64_t n, int64_t nblocks, uint8_t *__restrict__ out,
                      uint8_t *__restrict__ scales) {
    __shared__ float tiles[kQuantWarps][32 * 33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t groups = (nblocks + 31) / 32;
    for (int64_t g = (int64_t)blockIdx.x * kQuantWarps + warp; g < groups; g += (int64_t)gridDim.x * kQuantWarps) {
        float x[32];
        stage_rows(src, g * 1024, n, tiles[warp], x);
        const int64_t blk = g * 32 + lane;
        bool err = false;
        float max_abs = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            float a = fabsf(x[i]);
            if (GPTOSS) { if (isfinite(a) && a > max_abs) max_abs = a; }
            else { err |= !isfinite(a); if (a > max_abs) max_abs = a; }
        }
        uint32_t e = 0;
        float scale;
        if (GPTOSS) {
            uint32_t be = (__float_as_uint(max_abs) >> 23) & 255u;   // max_abs is finite and >= 0 here
            if (max_abs > 0.0f && be != 0) e = be >= 2 ? be - 2 : 0;
            if (e > 254u) e = 254u;
            scale = mx_scale_gptoss(e);
        } else {
            if (max_abs != 0.0f && !err) {
                // ceil(log2f(max_abs / 6)): the double logarithm rounded once to f32 stands for a
                // correctly rounded log2f; the integer part is exact, so only the rounding of the
                // sum matters and it agrees with the host library's
                float l = (float)log2((double)__fdiv_rn(max_abs, 6.0f));
                int eb = (int)ceilf(l) + 127;
                e = (uint32_t)(eb < 0 ? 0 : (eb > 254 ? 254 : eb));
            }
            scale = mx_scale_core(e);
        }
        uint32_t w[4] = {0, 0, 0, 0};   // 32 nibbles: byte i/2, the even element low (core) or high (gptoss)
#pragma unroll
        for (int i = 0; i < 32; i++) {
            uint32_t code = 0;
            const bool skip = GPTOSS ? !isfinite(x[i]) : (x[i] == 0.0f);
            if (!skip) code = nearest_e2m1(__fdiv_rn(fabsf(x[i]), scale)) | (x[i] < 0.0f ? 8u : 0u);
            const int nib = GPTOSS ? (i ^ 1) : i;
            w[nib >> 3] |= code << (4 * (nib & 7));
        }
        const bool any_err = __any_sync(0xffffffffu, err);
        if (any_err) {
            if (lane == 0) atomicExch(&g_quant_error, 1);
            continue;
        }
        if (blk < nblocks) {
            if (GPTOSS) {
                *reinterpret_cast<uint4 *>(out + blk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                scales[blk] = (uint8_t)e;
            } else {
                uint8_t *o = out + blk * 17;
                o[0] = (uint8_t)e;
#pragma unroll
                for (int b = 0; b < 16; b++) o[1 + b] = (uint8_t)(w[b >> 2] >> (8 * (b & 3)));
            }
        }
    }
}

nnq_status launch_quantize(nnq_ctx *ctx, int fmt, const float *src, int64_t n, uint8_t *dst, uint8_t *scales,
                           cudaStream_t stream) {
    int *flag = nullptr;
    nnq_status s = check_cuda(ctx, cudaGetSymbolAddress((void **)&flag, g_quant_error), "quantize flag");
    if (s != NNQ_OK) return s;
    s = check_cuda(ctx, cudaMemsetAsync(flag, 0, sizeof(int), stream), "quantize flag clear");
    if (s != NNQ_OK) return s;
    const int64_t nblocks = fmt == NNQ_Q4_K_GGML ? (n + 255) / 256 : (n + 31) / 32;
    const int64_t groups = fmt == NNQ_Q4_K_GGML ? (nblocks + 3) / 4 : (nblocks + 31) / 32;
    int64_t want = (groups + kQuantWarps - 1) / kQuantWarps, cap = (int64_t)ctx->sm_count * 8;
    const int grid = (int)(want < cap ? (want < 1 ? 1 : want) : cap);
    if (fmt == NNQ_Q4_K_GGML) quantize_q4k_ggml_kernel<<<grid, kQuantWarps * 32, 0, stream>>>(src, n, nblocks, dst);
    else if (fmt == NNQ_MXFP4_CORE) quantize_mxfp4_kernel<false><<<grid, kQuantWarps * 32, 0, stream>>>(src, n, nblocks, dst, nullptr);
    else quantize_mxfp4_kernel<true><<<grid, kQuantWarps * 32, 0, stream>>>(src, n, nblocks, dst, scales);
    ctx->launches++;
    s = check_cuda(ctx, cudaGetLastError(), "quantize launch");
    if (s != NNQ_OK) return s;
    int raised = 0;
    s = check_cuda(ctx, cudaMemcpyAsync(&raised, flag, sizeof(int), cudaMemcpyDeviceToHost, stream), "quantize flag read");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaStreamSynchronize(stream), "quantize synchronize");
    if (s != NNQ_OK) return s;
    if (raised) return fail(ctx, NNQ_ERR_VALUE_OUT_OF_RANGE, "non-finite value in the encoder input");
    return NNQ_OK;
}

}  // namespace nnq
