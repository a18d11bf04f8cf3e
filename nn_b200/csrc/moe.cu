// Mixture-of-experts block with block-quantized expert weights (the gpt-oss MoE layer):
// router linear -> softmax -> top-k -> renormalise -> per-expert (x W_gu + b) -> clamp(silu(gate)) * up
// -> (h W_d + b) -> routing-weighted sum per token, experts in index order.
// Follows crates/nn-gptoss/src/quantized_model.rs:99-194 (expert_forward, moe_forward).
//
// Everything stays on the device: no host round trip for the routing decisions. Tokens are
// grouped per expert with a stable counting sort (token order inside an expert, as the
// reference's assignment lists), the expert products read activations through that index list,
// and the combine step is a gather (no atomics), so results do not depend on scheduling.
//
// Scratch memory (owned by the context, grown on demand before the launches of a call):
//   idx[T,k] i32, wt[T,k] f32, pos[T,k] i32, count[E] / offset[E+1] i32, rowtok[R] i32,
//   gu[R, 2I] f32, h[R, I] f32, o[R, H] f32        with R = T * k routed rows.
#include <cuda_bf16.h>
#include <math_constants.h>

#include <new>

#include "decode.cuh"
#include <stdlib.h>

#include "gemm_tc.h"
#include "moe.h"
#include "pdl.cuh"
#include "skinny.h"

namespace nnq {

// ---------------------------------------------------------------------------------
// router: one warp per token
// ---------------------------------------------------------------------------------

template <typename XT>
__device__ __forceinline__ float ld_act(const XT *p, int64_t i);
template <>
__device__ __forceinline__ float ld_act<float>(const float *p, int64_t i) { return __ldg(p + i); }
template <>
__device__ __forceinline__ float ld_act<__nv_bfloat16>(const __nv_bfloat16 *p, int64_t i) {
    return __bfloat162float(p[i]);
}

constexpr int kMaxExperts = 64;
constexpr int kMaxTopK = 8;

// Softmax over the E logits of one token (lg, shared memory) and top-k selection by one warp.
__device__ __forceinline__ void route_token(const float *lg, int E, int top_k, int tok, int *__restrict__ idx,
                                            float *__restrict__ wt, int lane) {
    // lane e (and e + 32) holds expert e's logit
    float l0 = lane < E ? lg[lane] : -CUDART_INF_F;
    float l1 = lane + 32 < E ? lg[lane + 32] : -CUDART_INF_F;
    // softmax over the E experts (max-subtracted, f32)
    float mx = fmaxf(l0, l1);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    float p0 = lane < E ? expf(l0 - mx) : 0.0f;
    float p1 = lane + 32 < E ? expf(l1 - mx) : 0.0f;
    float sum = p0 + p1;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    p0 = p0 / sum;
    p1 = p1 / sum;
    if (lane >= E) p0 = -1.0f;
    if (lane + 32 >= E) p1 = -1.0f;
    // top-k: k rounds of (largest probability, lowest index) selection
    float sel_p = 0.0f, wsum = 0.0f;
    int sel_e = 0;
    for (int s = 0; s < top_k; s++) {
        float best = p0 >= p1 ? p0 : p1;
        int be = p0 >= p1 ? lane : lane + 32;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            float ob = __shfl_xor_sync(0xFFFFFFFFu, best, off);
            int oe = __shfl_xor_sync(0xFFFFFFFFu, be, off);
            if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
        }
        if (be == lane) p0 = -1.0f;
        if (be == lane + 32) p1 = -1.0f;
        if (lane == s) { sel_p = best; sel_e = be; }
        wsum += best;
    }
    if (lane < top_k) {
        idx[(int64_t)tok * top_k + lane] = sel_e;
        wt[(int64_t)tok * top_k + lane] = sel_p / wsum;
    }
}

// A CTA serves TOK consecutive tokens: their activations sit in shared memory as f32, the 8 warps
// share the experts (warp w: experts w, w + 8, ...; four experts at a time so that four weight
// loads are in flight per lane), every lane accumulates a strided slice of the hidden dimension,
// shuffle tree per (token, expert); a router weight row is read once per TOK tokens. Warp t then does
// the softmax and the top-k selection of token t over the logits in shared memory. The summation
// order of a logit does not depend on TOK.
template <typename XT, int TOK>
__global__ void __launch_bounds__(256)
moe_router_kernel(const XT *__restrict__ x, const float *__restrict__ rw, const float *__restrict__ rb,
                  int T, int H, int E, int top_k, int *__restrict__ idx, float *__restrict__ wt) {
    pdl_prologue();
    extern __shared__ float xs[];          // TOK tokens' activations as f32, then TOK x E logits
    float *logits = xs + (size_t)TOK * H;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tok0 = blockIdx.x * TOK;
    if (tok0 >= T) return;
    const int ntok = min(TOK, T - tok0);
    for (int i = threadIdx.x; i < ntok * H; i += 256) xs[i] = ld_act<XT>(x, (int64_t)tok0 * H + i);
    for (int i = ntok * H + threadIdx.x; i < TOK * H; i += 256) xs[i] = 0.0f;
    __syncthreads();
    constexpr int EB = 4;
    for (int e0 = warp; e0 < E; e0 += 8 * EB) {
        const float *w[EB];
#pragma unroll
        for (int j = 0; j < EB; j++) w[j] = rw + (int64_t)min(e0 + 8 * j, E - 1) * H;   // past the end: repeats the last expert, not stored
        float acc[TOK][EB];
#pragma unroll
        for (int t = 0; t < TOK; t++)
#pragma unroll
            for (int j = 0; j < EB; j++) acc[t][j] = 0.0f;
        for (int h = lane; h < H; h += 32) {
            float wv[EB];
#pragma unroll
            for (int j = 0; j < EB; j++) wv[j] = __ldg(w[j] + h);
#pragma unroll
            for (int t = 0; t < TOK; t++) {
                const float xv = xs[t * H + h];
#pragma unroll
                for (int j = 0; j < EB; j++) acc[t][j] = fmaf(xv, wv[j], acc[t][j]);
            }
        }
#pragma unroll
        for (int t = 0; t < TOK; t++)
#pragma unroll
            for (int j = 0; j < EB; j++) {
                float v = acc[t][j];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
                const int e = e0 + 8 * j;
                if (lane == 0 && e < E) logits[t * E + e] = v + __ldg(rb + e);
            }
    }
    __syncthreads();
    for (int t = warp; t < ntok; t += 8) route_token(logits + t * E, E, top_k, tok0 + t, idx, wt, lane);
}

// Fewer tokens than fill the machine one CTA each: a cluster of four CTAs serves a token, every CTA
// forms a quarter of the logits (a warp per expert, the same lane-strided sums as above: identical
// bits) and sends them into the first CTA's shared memory, which then routes the token.
constexpr int kRouterCluster = 4;

__device__ __forceinline__ void st_cluster_f32(const float *local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

template <typename XT>
__global__ void __cluster_dims__(kRouterCluster, 1, 1) __launch_bounds__(256)
moe_router_cluster_kernel(const XT *__restrict__ x, const float *__restrict__ rw, const float *__restrict__ rb,
                          int T, int H, int E, int top_k, int *__restrict__ idx, float *__restrict__ wt) {
    pdl_prologue();
    extern __shared__ float xs[];          // the token's activations as f32, then E logits (used in the first CTA)
    float *logits = xs + H;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int tok = blockIdx.x / kRouterCluster;   // the grid is exactly kRouterCluster * T CTAs
    for (int i = threadIdx.x; i < H; i += 256) xs[i] = ld_act<XT>(x, (int64_t)tok * H + i);
    __syncthreads();
    for (int e = (int)rank + kRouterCluster * warp; e < E; e += kRouterCluster * 8) {
        const float *w = rw + (int64_t)e * H;
        float acc = 0.0f;
#pragma unroll 6
        for (int h = lane; h < H; h += 32) acc = fmaf(xs[h], __ldg(w + h), acc);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
        if (lane == 0) st_cluster_f32(logits + e, 0, acc + __ldg(rb + e));
    }
    // every CTA's stores into the first CTA are complete and visible after the cluster barrier
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank == 0 && warp == 0) route_token(logits, E, top_k, tok, idx, wt, lane);
}

// ---------------------------------------------------------------------------------
// grouping: stable counting sort of the T*k assignments by expert
// ---------------------------------------------------------------------------------

// block e counts (pass 0) or lists (pass 1) the assignments of expert e in flat order
__global__ void __launch_bounds__(256)
moe_group_kernel(const int *__restrict__ idx, int total, int *__restrict__ count, const int *__restrict__ offset,
                 int *__restrict__ rowtok, int *__restrict__ pos, int pass, int e_begin) {
    const int el = blockIdx.x;          // local expert (this device holds experts e_begin .. e_begin + gridDim.x)
    const int e = e_begin + el;
    __shared__ int warp_sums[2][8];     // double-buffered: one barrier per 256 assignments
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int base = 0;                       // assignments of this expert before `start` (the same in every thread)
    for (int start = 0, it = 0; start < total; start += 256, it++) {
        int i = start + threadIdx.x;
        bool hit = i < total && idx[i] == e;
        unsigned ballot = __ballot_sync(0xFFFFFFFFu, hit);
        if (lane == 0) warp_sums[it & 1][warp] = __popc(ballot);
        __syncthreads();
        int before = 0, tot = 0;
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const int v = warp_sums[it & 1][w];
            tot += v;
            if (w < warp) before += v;
        }
        if (pass == 1 && hit) {
            int row = offset[el] + base + before + __popc(ballot & ((1u << lane) - 1u));
            rowtok[row] = i;
            pos[i] = row;
        }
        base += tot;
    }
    if (pass == 0 && threadIdx.x == 0) count[el] = base;
}

// The same grouping for decode-sized calls (total <= kGroupSmallMax assignments) in one CTA:
// warp w lists the assignments of experts w, w + 8, ... in flat order (ballot compaction), the
// counts are scanned in shared memory, then every warp writes its experts' rows.
constexpr int kGroupSmallMax = 2048;

__global__ void __launch_bounds__(256)
moe_group_small_kernel(const int *__restrict__ idx, int total, int *__restrict__ count, int *__restrict__ offset,
                       int *__restrict__ rowtok, int *__restrict__ pos, int e_begin, int e_local) {
    pdl_prologue();
    __shared__ int cnt[kMaxExperts], off[kMaxExperts + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int el = warp; el < e_local; el += 8) {
        int c = 0;
        for (int start = 0; start < total; start += 32) {
            const int i = start + lane;
            c += __popc(__ballot_sync(0xFFFFFFFFu, i < total && idx[i] == e_begin + el));
        }
        if (lane == 0) cnt[el] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < e_local; e++) {
            off[e] = acc;
            count[e] = cnt[e];
            offset[e] = acc;
            acc += cnt[e];
        }
        off[e_local] = acc;
        offset[e_local] = acc;
    }
    __syncthreads();
    for (int el = warp; el < e_local; el += 8) {
        int base = off[el];
        for (int start = 0; start < total; start += 32) {
            const int i = start + lane;
            const bool hit = i < total && idx[i] == e_begin + el;
            const unsigned ballot = __ballot_sync(0xFFFFFFFFu, hit);
            if (hit) {
                const int row = base + __popc(ballot & ((1u << lane) - 1u));
                rowtok[row] = i;
                pos[i] = row;
            }
            base += __popc(ballot);
        }
    }
}

__global__ void moe_scan_kernel(const int *__restrict__ count, int *__restrict__ offset, int E) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < E; e++) {
            offset[e] = acc;
            acc += count[e];
        }
        offset[E] = acc;
    }
}

// ---------------------------------------------------------------------------------
// expert products
// ---------------------------------------------------------------------------------

constexpr int kMoeMT = 8;     // routed rows per pass over an expert's weights
constexpr int kMoeKCH = 128;  // activation chunk staged in shared memory

// Row r of the routed (expert-sorted) order reads its activations either from the token it
// belongs to (first product) or from row r of the intermediate buffer (second product).
template <typename XT>
__device__ __forceinline__ const XT *act_row(const XT *x, const int *rowtok, int top_k, int r, int64_t K) {
    int64_t src = rowtok ? rowtok[r] / top_k : r;
    return x + src * K;
}

// Weights stored [E][K][N] with MXFP4 blocks of 32 running along N (nn-gptoss Mxfp4Tensor over
// the flattened [ne, K, N] tensor: crates/nn-gptoss/src/quantized_model.rs:69-77,
// crates/nn-gptoss/src/quantize.rs:122-163): out[r, n] = sum_k x[r, k] * W[e, k, n] + bias[e, n].
// A warp owns 256 consecutive columns (4 bytes of codes per lane and k) and one of gridDim.z
// slices of K; it keeps 8 rows of weights in flight per lane. Slice z writes its partial sums to
// out + z * slice_stride (slice 0 adds the bias); the consumer kernels add the slices in order.
constexpr int kMoeKnSplit = 4;
constexpr int kMoeKnUnroll = 8;

template <typename XT>
__global__ void __launch_bounds__(128)
moe_kn_gptoss_kernel(const uint8_t *__restrict__ data, const uint8_t *__restrict__ scales,
                     const float *__restrict__ bias, const XT *__restrict__ x, const int *__restrict__ rowtok,
                     int top_k, const int *__restrict__ offset, float *__restrict__ out, size_t slice_stride,
                     int K, int N) {
    __shared__ float xt[kMoeMT][kMoeKCH];
    const int e = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n0 = blockIdx.x * 1024 + warp * 256 + lane * 8;
    const bool col_ok = n0 < N;
    const uint8_t *wd = data + (size_t)e * K * (N / 2) + n0 / 2;
    const uint8_t *ws = scales + (size_t)e * K * (N / 32) + n0 / 32;
    const int r_begin = offset[e], r_end = offset[e + 1];
    // this CTA's slice of K (whole chunks of kMoeKCH)
    const int chunks = (K + kMoeKCH - 1) / kMoeKCH;
    const int c_lo = (int)(((long long)blockIdx.z * chunks) / gridDim.z);
    const int c_hi = (int)(((long long)(blockIdx.z + 1) * chunks) / gridDim.z);
    float *po = out + (size_t)blockIdx.z * slice_stride;
    for (int r0 = r_begin; r0 < r_end; r0 += kMoeMT) {
        const int mt = min(kMoeMT, r_end - r0);
        float acc[kMoeMT][8];
#pragma unroll
        for (int t = 0; t < kMoeMT; t++)
#pragma unroll
            for (int c = 0; c < 8; c++) acc[t][c] = 0.0f;
        for (int ch = c_lo; ch < c_hi; ch++) {
            const int k0 = ch * kMoeKCH;
            const int kn = min(kMoeKCH, K - k0);
            __syncthreads();
            for (int i = threadIdx.x; i < kMoeMT * kMoeKCH; i += 128) {
                int t = i / kMoeKCH, kk = i % kMoeKCH;
                float v = 0.0f;
                if (t < mt && kk < kn) v = ld_act<XT>(act_row<XT>(x, rowtok, top_k, r0 + t, K), k0 + kk);
                xt[t][kk] = v;
            }
            __syncthreads();
            if (col_ok) {
                for (int kk = 0; kk < kn; kk += kMoeKnUnroll) {
                    uint32_t w[kMoeKnUnroll];
                    uint32_t sc[kMoeKnUnroll];
#pragma unroll
                    for (int u = 0; u < kMoeKnUnroll; u++) {   // all loads first: 8 rows in flight
                        const size_t k = (size_t)(k0 + min(kk + u, kn - 1));
                        w[u] = __ldg(reinterpret_cast<const uint32_t *>(wd + k * (N / 2)));
                        sc[u] = __ldg(ws + k * (N / 32));
                    }
#pragma unroll
                    for (int u = 0; u < kMoeKnUnroll; u++) {
                        if (kk + u < kn) {
                            float scale = mx_scale_gptoss(sc[u]);
                            float wv[8];
#pragma unroll
                            for (int b = 0; b < 4; b++) {
                                uint32_t byte = (w[u] >> (8 * b)) & 0xFFu;
                                wv[2 * b] = e2m1_value(byte >> 4, scale);       // high nibble = even column
                                wv[2 * b + 1] = e2m1_value(byte & 15u, scale);
                            }
#pragma unroll
                            for (int t = 0; t < kMoeMT; t++) {
                                float xv = xt[t][kk + u];
#pragma unroll
                                for (int c = 0; c < 8; c++) acc[t][c] = fmaf(xv, wv[c], acc[t][c]);
                            }
                        }
                    }
                }
            }
        }
        if (col_ok) {
            for (int t = 0; t < mt; t++) {
                float *o = po + (size_t)(r0 + t) * N + n0;
#pragma unroll
                for (int c = 0; c < 8; c++) o[c] = acc[t][c] + (blockIdx.z == 0 ? __ldg(bias + (size_t)e * N + n0 + c) : 0.0f);
            }
        }
    }
}

// Weights stored per expert as [N, K] in any block format (blocks along K):
// one warp per output column, the lanes share the 32-weight chunks of the row.
template <int FMT, typename XT>
__global__ void __launch_bounds__(128)
moe_nk_kernel(const uint8_t *__restrict__ data, const uint8_t *__restrict__ scales, size_t expert_bytes,
              size_t expert_scale_bytes, const float *__restrict__ bias, const XT *__restrict__ x,
              const int *__restrict__ rowtok, int top_k, const int *__restrict__ offset,
              float *__restrict__ out, int K, int N) {
    const int e = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (n >= N) return;
    const uint8_t *wd = data + (size_t)e * expert_bytes;
    const uint8_t *ws = scales ? scales + (size_t)e * expert_scale_bytes : nullptr;
    const int64_t cpr = K / 32;
    const int r_begin = offset[e], r_end = offset[e + 1];
    for (int r0 = r_begin; r0 < r_end; r0 += kMoeMT) {
        const int mt = min(kMoeMT, r_end - r0);
        float acc[kMoeMT];
#pragma unroll
        for (int t = 0; t < kMoeMT; t++) acc[t] = 0.0f;
        for (int64_t c = lane; c < cpr; c += 32) {
            float wv[32];
            Decode<FMT>::chunk(wd, ws, (int64_t)n * cpr + c, wv);
#pragma unroll
            for (int t = 0; t < kMoeMT; t++) {
                if (t < mt) {
                    const XT *xr = act_row<XT>(x, rowtok, top_k, r0 + t, K) + c * 32;
#pragma unroll
                    for (int i = 0; i < 32; i++) acc[t] = fmaf(wv[i], ld_act<XT>(xr, i), acc[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < kMoeMT; t++) {
            float v = acc[t];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
            if (lane == 0 && t < mt) out[(size_t)(r0 + t) * N + n] = v + __ldg(bias + (size_t)e * N + n);
        }
    }
}

// h[r, j] = clamp(silu(gu[r, j]), -limit, limit) * gu[r, I + j]   (gate = first half, up = second half).
// CTA (r, c) handles row r, columns [1024 c, 1024 c + 1024), four per thread. With h_bf16 given (the
// tensor-core second product reads bf16) the f32 copy is not written.
__device__ __forceinline__ float swiglu_one(float g, float u, float limit) {
    float s = g / (1.0f + expf(-g));
    s = fminf(fmaxf(s, -limit), limit);
    return s * u;
}
__global__ void __launch_bounds__(256)
moe_swiglu_kernel(const float *__restrict__ gu, float *__restrict__ h, const int *__restrict__ offset,
                  int E, int inter, float limit, int slices, size_t slice_stride, __nv_bfloat16 *__restrict__ h_bf16) {
    pdl_prologue();
    const int64_t r = blockIdx.x;
    if (r >= offset[E]) return;
    const int j0 = blockIdx.y * 1024 + threadIdx.x * 4;
    if (j0 >= inter) return;
    const float *grow = gu + r * 2 * inter;
    float out[4];
    if (slices == 1 && (inter & 3) == 0) {
        const float4 g = *reinterpret_cast<const float4 *>(grow + j0);
        const float4 u = *reinterpret_cast<const float4 *>(grow + inter + j0);
        out[0] = swiglu_one(g.x, u.x, limit);
        out[1] = swiglu_one(g.y, u.y, limit);
        out[2] = swiglu_one(g.z, u.z, limit);
        out[3] = swiglu_one(g.w, u.w, limit);
        if (h_bf16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(out[0], out[1]), hi = __floats2bfloat162_rn(out[2], out[3]);
            *reinterpret_cast<uint2 *>(h_bf16 + r * inter + j0) = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
        } else {
            *reinterpret_cast<float4 *>(h + r * inter + j0) = make_float4(out[0], out[1], out[2], out[3]);
        }
        return;
    }
    for (int q = 0; q < 4 && j0 + q < inter; q++) {
        const int j = j0 + q;
        float g = 0.0f, u = 0.0f;
        for (int z = 0; z < slices; z++) {   // K slices of the first product, in order
            g += grow[z * slice_stride + j];
            u += grow[z * slice_stride + inter + j];
        }
        const float v = swiglu_one(g, u, limit);
        if (h_bf16) h_bf16[r * inter + j] = __float2bfloat16_rn(v);
        else h[r * inter + j] = v;
    }
}

// xg[r, :] = bf16(x[token of routed row r, :]): the gathered input of the tensor-core first product
template <typename XT>
__global__ void moe_gather_bf16_kernel(const XT *__restrict__ x, const int *__restrict__ rowtok, int top_k,
                                       const int *__restrict__ offset, int E, int H, __nv_bfloat16 *__restrict__ xg) {
    pdl_prologue();
    const int r = blockIdx.x;
    if (r >= offset[E]) return;
    const XT *src = x + (size_t)(rowtok[r] / top_k) * H;
    if (sizeof(XT) == 2 && (H & 7) == 0) {   // bf16 rows of whole 16-byte units: a plain copy
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
        uint4 *d4 = reinterpret_cast<uint4 *>(xg + (size_t)r * H);
        for (int j = threadIdx.x; j < H / 8; j += blockDim.x) d4[j] = __ldg(s4 + j);
        return;
    }
    for (int j = threadIdx.x; j < H; j += blockDim.x) xg[(size_t)r * H + j] = __float2bfloat16_rn(ld_act<XT>(src, j));
}

// y[t, :] = sum over the token's experts, in expert-index order, of weight * o[row, :]
__global__ void moe_combine_kernel(const float *__restrict__ o, const int *__restrict__ idx, const float *__restrict__ wt,
                                   const int *__restrict__ pos, int T, int H, int top_k, float *__restrict__ y,
                                   int slices, size_t slice_stride) {
    pdl_prologue();
    const int t = blockIdx.x;
    if (t >= T) return;
    int order[kMaxTopK];
    for (int s = 0; s < top_k; s++) order[s] = s;
    for (int a = 1; a < top_k; a++)   // insertion sort of the slots by expert index
        for (int b = a; b > 0 && idx[(int64_t)t * top_k + order[b]] < idx[(int64_t)t * top_k + order[b - 1]]; b--) {
            int tmp = order[b]; order[b] = order[b - 1]; order[b - 1] = tmp;
        }
    if (slices == 1 && (H & 3) == 0) {
        // slot rows and weights once per thread, then four columns at a time (same sums, same order)
        int rows[kMaxTopK];
        float ws[kMaxTopK];
        for (int s = 0; s < top_k; s++) {
            rows[s] = pos[(int64_t)t * top_k + order[s]];
            ws[s] = wt[(int64_t)t * top_k + order[s]];
        }
        const float4 *o4 = reinterpret_cast<const float4 *>(o);
        float4 *y4 = reinterpret_cast<float4 *>(y + (size_t)t * H);
        for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < H / 4; j += gridDim.y * blockDim.x) {
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int s = 0; s < top_k; s++) {
                if (rows[s] < 0) continue;   // expert held by another device
                const float4 v = o4[(size_t)rows[s] * (H / 4) + j];
                acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, ws[s]));
                acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, ws[s]));
                acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, ws[s]));
                acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, ws[s]));
            }
            y4[j] = acc;
        }
        return;
    }
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < H; j += gridDim.y * blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < top_k; s++) {
            int slot = order[s];
            int row = pos[(int64_t)t * top_k + slot];
            if (row < 0) continue;   // expert held by another device
            float v = 0.0f;
            for (int z = 0; z < slices; z++) v += o[z * slice_stride + (size_t)row * H + j];   // K slices, in order
            acc = __fadd_rn(acc, __fmul_rn(v, wt[(int64_t)t * top_k + slot]));
        }
        y[(size_t)t * H + j] = acc;
    }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------

struct MoeScratch {
    int *idx, *pos, *count, *offset, *rowtok;
    float *wt, *gu, *h, *o;
    __nv_bfloat16 *xg, *hb;     // bf16 inputs of the tensor-core products (prefill-sized calls only)
    int slices;                 // K slices whose partial sums gu / o hold (1 = complete sums)
    size_t gu_stride, o_stride; // floats between slices
    size_t bytes;
};

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// Prefill-sized calls on [N, K] expert weights go through the grouped tcgen05 products: from 32 routed
// rows per local expert on average (below that the weights are streamed once per 16 rows by the
// grouped token-column kernel, which is HBM-bound and wins; the gpt-oss block crosses over near 240 tokens).
static bool moe_tensor_mode(const nnq_moe *m, int64_t T, int k, bool routed) {
    static const char *env = diag_env("NNQ_MOE_TENSOR");   // tuning aid: 0 keeps the token-column kernel
    if (env && atoi(env) == 0) return false;
    // nn-gptoss [E, K, N] experts take the decode-once form only (a transposing decode into the context's
    // bf16 scratch, sized when the block was created) and need the single-slice output buffers that come
    // with their tiled copies
    const bool nk = m->layout == NNQ_MOE_NK && (m->fmt < NNQ_Q5_0 || m->fmt >= NNQ_F32_DENSE);
    const bool kn = m->layout == NNQ_MOE_KN_GPTOSS && m->d_gu_tiled != nullptr && m->ctx->d_dense != nullptr &&
                    (size_t)m->e_local * 2 * (size_t)m->inter * (size_t)m->hidden * 2 <= m->ctx->dense_bytes;
    return (nk || kn) && m->hidden % 64 == 0 && m->inter % 64 == 0 &&
           // 32 routed rows per expert on average: with the block's own router the T tokens spread over
           // all experts (the shards of one block agree), rows routed by the caller all go to local experts
           T * k >= (env ? atoi(env) : 32) * (int64_t)(routed ? m->e_local : m->n_experts);
}

// Carves the scratch buffer for T rows with k expert slots each; with base == NULL only the size
// is computed.
static MoeScratch carve(uint8_t *base, int64_t T, const nnq_moe *m, int k, bool routed = false) {
    MoeScratch s;
    const int64_t R = T * k;
    size_t off = 0;
    auto take = [&](size_t bytes) { uint8_t *p = base ? base + off : nullptr; off += align256(bytes); return p; };
    s.idx = (int *)take(R * 4);
    s.wt = (float *)take(R * 4);
    s.pos = (int *)take(R * 4);
    s.count = (int *)take((size_t)m->e_local * 4);
    s.offset = (int *)take((size_t)(m->e_local + 1) * 4);
    s.rowtok = (int *)take(R * 4);
    const int slices = m->layout == NNQ_MOE_KN_GPTOSS && !m->d_gu_tiled ? kMoeKnSplit : 1;   // partial sums per K slice (row kernel only)
    s.gu = (float *)take((size_t)R * 2 * m->inter * 4 * slices);
    s.h = (float *)take((size_t)R * m->inter * 4);
    s.o = (float *)take((size_t)R * m->hidden * 4 * slices);
    const bool tensor = moe_tensor_mode(m, T, k, routed);
    s.xg = tensor ? (__nv_bfloat16 *)take((size_t)R * m->hidden * 2) : nullptr;
    s.hb = tensor ? (__nv_bfloat16 *)take((size_t)R * m->inter * 2) : nullptr;
    s.slices = slices;
    s.gu_stride = (size_t)R * 2 * m->inter;
    s.o_stride = (size_t)R * m->hidden;
    s.bytes = off;
    return s;
}

static nnq_status ensure_scratch(nnq_ctx *ctx, const nnq_moe *m, int64_t T, int k, bool routed, MoeScratch *out) {
    MoeScratch need = carve(nullptr, T, m, k, routed);
    if (need.bytes > ctx->moe_bytes) {
        cudaFree(ctx->d_moe);
        ctx->d_moe = nullptr;
        ctx->moe_bytes = 0;
        nnq_status s = check_cuda(ctx, cudaMalloc(&ctx->d_moe, need.bytes), "cudaMalloc MoE scratch");
        if (s != NNQ_OK) return s;
        ctx->moe_bytes = need.bytes;
    }
    *out = carve(ctx->d_moe, T, m, k, routed);
    return NNQ_OK;
}

template <typename XT>
struct DtypeOf;
template <>
struct DtypeOf<float> { static constexpr int value = NNQ_F32; };
template <>
struct DtypeOf<__nv_bfloat16> { static constexpr int value = NNQ_BF16; };

template <typename XT>
static nnq_status launch_product(nnq_ctx *ctx, const nnq_moe *m, bool first, const XT *x, const int *rowtok, int top_k,
                           const MoeScratch &s, float *out, int64_t rows, cudaStream_t st, bool *swiglu_done = nullptr) {
    const int K = first ? m->hidden : m->inter;
    const int N = first ? 2 * m->inter : m->hidden;
    const uint8_t *d = first ? m->d_gu : m->d_dn;
    const uint8_t *sc = first ? m->d_gu_scales : m->d_dn_scales;
    const float *b = first ? m->d_gu_bias : m->d_dn_bias;
    const int E = m->e_local;
    if (s.xg) {
        // prefill-sized: grouped tcgen05 product over bf16 inputs in routed order
        Geometry g = geometry(m->fmt);
        const size_t eb = (size_t)N * (K / g.elems) * g.bytes, es = (size_t)N * (K / g.elems) * g.scale_bytes;
        TcGroupArgs a = {d, sc, eb, es, first ? (const void *)s.xg : (const void *)s.hb, b, out, s.offset, E, rows, N, K, m->fmt};
        a.kn = m->layout == NNQ_MOE_KN_GPTOSS;
        // all local experts decoded to bf16 once, then the plain grouped GEMM -- or the grouped product with
        // the decode fused in. Measured (32 experts of about 3000 x 3000, top-4; ms per block fused / decoded
        // once at 64, 128 and 256 rows per expert): MXFP4 1.24 / 0.87 at 64 rows, decoded once at every size
        // (its decode to bf16 is integer work at copy speed); Q4_K, whose fused decode streams the raw blocks
        // through the TMA ring, 0.71 / 0.88, 0.99 / 0.97, 1.23 / 1.24; Q8_0 (ring when K is a multiple of 256)
        // 0.77 / 1.12, 1.03 / 1.21, 1.30 / 1.46, but its 512-row tile has no ring; Q6_K (no ring) as measured
        // before the ring existed, from about 100 rows per expert
        int64_t dense_rows = 32;
        if (m->fmt == NNQ_Q4_K || m->fmt == NNQ_Q4_K_GGML) dense_rows = 128;
        else if (m->fmt == NNQ_Q6_K) dense_rows = 96;
        else if (m->fmt == NNQ_Q8_0 && K % 256 == 0) dense_rows = 384;
#ifdef NNQ_DIAG
        if (const char *e = getenv("NNQ_MOE_DENSE_ROWS")) dense_rows = atoi(e);
#endif
        if (a.kn && !gemm_dense_grouped_supported(ctx, a)) return fail(ctx, NNQ_ERR_UNSUPPORTED, "[E, K, N] experts: no bf16 scratch for the prefill-sized product");
        if ((a.kn || rows >= dense_rows * (int64_t)E) && gemm_dense_grouped_supported(ctx, a)) {
            if (first && swiglu_done && s.slices == 1) {
                // gate / up product: SwiGLU in the GEMM's epilogue where the decode can interleave the rows
                a.h_out = s.hb;
                a.swiglu_limit = m->limit;
                *swiglu_done = gemm_dense_grouped_fuses_swiglu(a);
                if (!*swiglu_done) a.h_out = nullptr;
            }
            return launch_gemm_dense_grouped(ctx, a, st);
        }
        return launch_gemm_tc_grouped(ctx, a, st);
    }
    if (m->d_gu_tiled) {
        GroupedArgs a = {first ? m->d_gu_tiled : m->d_dn_tiled, first ? m->gu_tile_stride : m->dn_tile_stride, b, x,
                         DtypeOf<XT>::value, rowtok, s.offset, out, E, top_k, N, K, m->fmt, rows,
                         m->layout == NNQ_MOE_KN_GPTOSS ? 1 : 0};
        return launch_grouped(ctx, a, st);
    }
    ctx->launches++;   // one of the row kernels below
    if (m->layout == NNQ_MOE_KN_GPTOSS) {
        dim3 grid((N + 1023) / 1024, E, kMoeKnSplit);
        moe_kn_gptoss_kernel<XT><<<grid, 128, 0, st>>>(d, sc, b, x, rowtok, top_k, s.offset, out,
                                                        first ? s.gu_stride : s.o_stride, K, N);
        return NNQ_OK;
    }
    Geometry g = geometry(m->fmt);
    size_t eb = (size_t)N * (K / g.elems) * g.bytes, es = (size_t)N * (K / g.elems) * g.scale_bytes;
    dim3 grid((N + 3) / 4, E);
#define NNQ_NK(F) case F: moe_nk_kernel<F, XT><<<grid, 128, 0, st>>>(d, sc, eb, es, b, x, rowtok, top_k, s.offset, out, K, N); break
    switch (m->fmt) {
        NNQ_NK(NNQ_Q4_0); NNQ_NK(NNQ_Q4_1); NNQ_NK(NNQ_Q8_0); NNQ_NK(NNQ_Q4_K); NNQ_NK(NNQ_Q4_K_GGML);
        NNQ_NK(NNQ_Q6_K); NNQ_NK(NNQ_MXFP4_CORE); NNQ_NK(NNQ_MXFP4_SPLIT); NNQ_NK(NNQ_MXFP4_GPTOSS);
        NNQ_NK(NNQ_Q5_0); NNQ_NK(NNQ_Q5_1); NNQ_NK(NNQ_Q2_K); NNQ_NK(NNQ_Q3_K); NNQ_NK(NNQ_Q5_K);
        NNQ_NK(NNQ_F32_DENSE); NNQ_NK(NNQ_BF16_DENSE);
        default: return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", (int)m->fmt);
    }
#undef NNQ_NK
    return NNQ_OK;
}

// the router keeps one token's activations in shared memory: allow more than the default 48 KB
template <typename XT>
static cudaError_t launch_router(const nnq_moe *m, const XT *x, int64_t T, int *idx, float *wt, cudaStream_t st) {
    // eight tokens per CTA once there are enough tokens to fill the machine that way (and their
    // activations fit in shared memory): the router weights are then read once per eight tokens
    const bool many = T >= 1024 && (size_t)8 * (m->hidden + kMaxExperts) * 4 <= 200 * 1024;
    const int tok = many ? 8 : 1;
    const size_t smem = (size_t)tok * (m->hidden + kMaxExperts) * 4;
    static bool configured[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !configured[dev][many]) {
        cudaError_t e = many ? cudaFuncSetAttribute(moe_router_kernel<XT, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                             : cudaFuncSetAttribute(moe_router_kernel<XT, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev][many] = true;
    }
    if (many) moe_router_kernel<XT, 8><<<(int)((T + 7) / 8), 256, smem, st>>>(x, m->d_router_w, m->d_router_b, (int)T, m->hidden, m->n_experts, m->top_k, idx, wt);
    else if (smem <= 48 * 1024 && T * kRouterCluster < (1 << 30))
        moe_router_cluster_kernel<XT><<<(int)T * kRouterCluster, 256, smem, st>>>(x, m->d_router_w, m->d_router_b, (int)T, m->hidden, m->n_experts, m->top_k, idx, wt);
    else moe_router_kernel<XT, 1><<<(int)T, 256, smem, st>>>(x, m->d_router_w, m->d_router_b, (int)T, m->hidden, m->n_experts, m->top_k, idx, wt);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// scratch that nobody allocates (see nnq_moe_forward_static)
// ---------------------------------------------------------------------------------

// Fixed scratch area living in the library's device image: every GPU that loads the library
// holds these bytes until the process exits, so the size is kept modest. All calls of
// nnq_moe_forward_static on a device share it.
constexpr size_t kStaticScratchBytes = (size_t)8 << 20;
static __device__ __align__(256) unsigned char g_moe_static_scratch[kStaticScratchBytes];

// Device address of the area, looked up once per device. In host code the array's name is only
// a stand-in for the symbol, not an address a kernel may use; cudaGetSymbolAddress (with the
// device current) gives the real one.
static nnq_status static_scratch_base(nnq_ctx *ctx, uint8_t **base) {
    static uint8_t *cached[64] = {};
    const int dev = ctx->device;
    if (dev < 0 || dev >= 64) return fail(ctx, NNQ_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (!cached[dev]) {
        void *p = nullptr;
        nnq_status s = check_cuda(ctx, cudaGetSymbolAddress(&p, g_moe_static_scratch), "cudaGetSymbolAddress");
        if (s != NNQ_OK) return s;
        cached[dev] = static_cast<uint8_t *>(p);
    }
    *base = cached[dev];
    return NNQ_OK;
}

// The launches of one forward pass over a scratch area the caller of this function provides.
// Routing comes from the block's router (given_idx == NULL: k = top_k slots per token) or from the
// caller (given_idx / given_wt: [T, k] expert indices and weights already on the device; rows
// whose expert lives elsewhere contribute nothing). route_only stops after the router.
template <typename XT>
static nnq_status run_with_scratch(nnq_ctx *ctx, const nnq_moe *m, const XT *x, int64_t T, int k, const int *given_idx,
                                   const float *given_wt, float *y, const MoeScratch &s, bool route_only, cudaStream_t st) {
    const int E = m->n_experts;
    const int total = (int)(T * k);
    const int *idx = s.idx;
    const float *wt = s.wt;
    if (given_idx) {
        idx = given_idx;
        wt = given_wt;
    } else {
        launch_router<XT>(m, x, T, s.idx, s.wt, st);
        ctx->launches++;
    }
    if (route_only) return check_cuda(ctx, cudaGetLastError(), "MoE router launch");
    const int EL = m->e_local;
    if (EL != E) cudaMemsetAsync(s.pos, 0xFF, (size_t)total * 4, st);   // -1: assignment served elsewhere
    if (total <= kGroupSmallMax) {
        launch_pdl(moe_group_small_kernel, dim3(1), dim3(256), st, idx, total, s.count, s.offset, s.rowtok, s.pos, m->e_begin, EL);
    } else {
        moe_group_kernel<<<EL, 256, 0, st>>>(idx, total, s.count, s.offset, s.rowtok, s.pos, 0, m->e_begin);
        moe_scan_kernel<<<1, 32, 0, st>>>(s.count, s.offset, EL);
        moe_group_kernel<<<EL, 256, 0, st>>>(idx, total, s.count, s.offset, s.rowtok, s.pos, 1, m->e_begin);
        ctx->launches += 2;
    }
    if (s.xg) {
        moe_gather_bf16_kernel<XT><<<total, 256, 0, st>>>(x, s.rowtok, k, s.offset, m->e_local, m->hidden, s.xg);
        ctx->launches++;
    }
    bool swiglu_done = false;
    nnq_status prc = launch_product<XT>(ctx, m, true, x, s.rowtok, k, s, s.gu, total, st, &swiglu_done);
    if (prc != NNQ_OK) return prc;
    if (!swiglu_done)
        launch_pdl(moe_swiglu_kernel, dim3((unsigned)total, (unsigned)((m->inter + 1023) / 1024)), dim3(256), st, s.gu, s.h, s.offset, m->e_local, m->inter, m->limit, s.slices, s.gu_stride, s.hb);
    prc = launch_product<float>(ctx, m, false, s.h, nullptr, k, s, s.o, total, st);
    if (prc != NNQ_OK) return prc;
    launch_pdl(moe_combine_kernel, dim3((unsigned)T, T < 1024 ? 4 : 1), dim3(256), st, s.o, idx, wt, s.pos, (int)T, m->hidden, k, y, s.slices, s.o_stride);
    ctx->launches += 3;   // grouping, SwiGLU, combine (the router and the products count themselves)
    return check_cuda(ctx, cudaGetLastError(), "MoE launch");
}

// Forward pass over the context's growable scratch buffer.
template <typename XT>
static nnq_status forward_typed(nnq_ctx *ctx, const nnq_moe *m, const XT *x, int64_t T, int k, const int *given_idx,
                                const float *given_wt, float *y, int *idx_out, float *wt_out, bool route_only, cudaStream_t st) {
    MoeScratch s;
    nnq_status rc = ensure_scratch(ctx, m, T, k, given_idx != nullptr, &s);
    if (rc != NNQ_OK) return rc;
    rc = run_with_scratch<XT>(ctx, m, x, T, k, given_idx, given_wt, y, s, route_only, st);
    if (rc != NNQ_OK) return rc;
    const size_t total = (size_t)T * k;
    if (idx_out) cudaMemcpyAsync(idx_out, s.idx, total * 4, cudaMemcpyDeviceToDevice, st);
    if (wt_out) cudaMemcpyAsync(wt_out, s.wt, total * 4, cudaMemcpyDeviceToDevice, st);
    return check_cuda(ctx, cudaGetLastError(), "MoE routing copy");
}

// Gathers rows of a [rows, H] matrix by index: out[i, :] = x[index[i], :] (the token permute of
// expert parallelism: rows sorted by destination before they are sent).
template <typename XT>
__global__ void moe_gather_rows_kernel(const XT *__restrict__ x, const int *__restrict__ index, int64_t n, int H, XT *__restrict__ out) {
    const int64_t r = blockIdx.x;
    if (r >= n) return;
    const XT *src = x + (size_t)index[r] * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) out[(size_t)r * H + j] = src[j];
}

}  // namespace nnq

using namespace nnq;

extern "C" {

static nnq_status upload(nnq_ctx *ctx, void **dst, const void *src, size_t bytes, const char *what) {
    *dst = nullptr;
    if (bytes == 0) return NNQ_OK;
    nnq_status s = check_cuda(ctx, cudaMalloc(dst, bytes + 16), what);
    if (s != NNQ_OK) return s;
    return check_cuda(ctx, cudaMemcpy(*dst, src, bytes, cudaMemcpyDefault), what);
}

nnq_status nnq_moe_create_shard(nnq_ctx *ctx, int n_experts, int expert_begin, int expert_count, int hidden,
                                int inter, int top_k, float swiglu_limit, const float *router_w,
                                const float *router_b, nnq_moe_layout layout, nnq_format fmt, const void *gate_up,
                                size_t gate_up_bytes, const void *gate_up_scales, size_t gate_up_scales_bytes,
                                const float *gate_up_bias, const void *down, size_t down_bytes,
                                const void *down_scales, size_t down_scales_bytes, const float *down_bias,
                                nnq_moe **out) {
    if (!ctx || !out) return NNQ_ERR_INVALID_ARG;
    *out = nullptr;
    if (n_experts < 1 || n_experts > kMaxExperts || top_k < 1 || top_k > kMaxTopK || top_k > n_experts ||
        hidden < 1 || inter < 1 || hidden > 49152)
        return fail(ctx, NNQ_ERR_INVALID_ARG, "bad MoE dimensions (experts %d, top_k %d, hidden %d, inter %d)", n_experts, top_k, hidden, inter);
    if (expert_begin < 0 || expert_count < 1 || expert_begin + expert_count > n_experts)
        return fail(ctx, NNQ_ERR_INVALID_ARG, "bad expert range [%d, %d) of %d", expert_begin, expert_begin + expert_count, n_experts);
    if (!router_w || !router_b || !gate_up || !down || !gate_up_bias || !down_bias) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL MoE tensor");
    if ((int)fmt < 0 || fmt >= NNQ_FORMAT_COUNT) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", (int)fmt);
    if (layout == NNQ_MOE_KN_GPTOSS && fmt != NNQ_MXFP4_GPTOSS)
        return fail(ctx, NNQ_ERR_WRONG_QUANT_TYPE, "the [E,K,N] layout holds nn-gptoss MXFP4 tensors only");
    if (layout != NNQ_MOE_KN_GPTOSS && layout != NNQ_MOE_NK) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown MoE layout %d", (int)layout);
    Geometry g = geometry(fmt);
    // blocks must not cross rows of the axis they run along
    const int64_t gu_inner = layout == NNQ_MOE_KN_GPTOSS ? 2 * (int64_t)inter : hidden;
    const int64_t dn_inner = layout == NNQ_MOE_KN_GPTOSS ? hidden : inter;
    if (gu_inner % g.elems || dn_inner % g.elems)
        return fail(ctx, NNQ_ERR_INVALID_SHAPE, "expert dimensions are not multiples of the block size %d", g.elems);
    const size_t gu_blocks = (size_t)expert_count * hidden * 2 * inter / g.elems;
    const size_t dn_blocks = (size_t)expert_count * inter * hidden / g.elems;
    if (gate_up_bytes != gu_blocks * g.bytes || down_bytes != dn_blocks * g.bytes ||
        gate_up_scales_bytes != gu_blocks * g.scale_bytes || down_scales_bytes != dn_blocks * g.scale_bytes)
        return fail(ctx, NNQ_ERR_DATA_LENGTH, "expert tensor byte length does not match its shape");
    if (g.scale_bytes && (!gate_up_scales || !down_scales)) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL scale tensor");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    nnq_moe *m = new (std::nothrow) nnq_moe();
    if (!m) return fail(ctx, NNQ_ERR_OUT_OF_MEMORY, "host allocation failed");
    memset(m, 0, sizeof(*m));
    m->ctx = ctx; m->n_experts = n_experts; m->hidden = hidden; m->inter = inter; m->top_k = top_k;
    m->e_begin = expert_begin; m->e_local = expert_count;
    m->limit = swiglu_limit; m->layout = layout; m->fmt = fmt;
    m->gu_bytes = gate_up_bytes; m->gu_scale_bytes = gate_up_scales_bytes;
    m->dn_bytes = down_bytes; m->dn_scale_bytes = down_scales_bytes;
    s = upload(ctx, (void **)&m->d_router_w, router_w, (size_t)n_experts * hidden * 4, "router weight");
    if (s == NNQ_OK) s = upload(ctx, (void **)&m->d_router_b, router_b, (size_t)n_experts * 4, "router bias");
    if (s == NNQ_OK) s = upload(ctx, (void **)&m->d_gu, gate_up, gate_up_bytes, "gate_up");
    if (s == NNQ_OK) s = upload(ctx, (void **)&m->d_gu_scales, gate_up_scales, gate_up_scales_bytes, "gate_up scales");
    if (s == NNQ_OK) s = upload(ctx, (void **)&m->d_gu_bias, gate_up_bias, (size_t)expert_count * 2 * inter * 4, "gate_up bias");
    if (s == NNQ_OK) s = upload(ctx, (void **)&m->d_dn, down, down_bytes, "down");
    if (s == NNQ_OK) s = upload(ctx, (void **)&m->d_dn_scales, down_scales, down_scales_bytes, "down scales");
    if (s == NNQ_OK) s = upload(ctx, (void **)&m->d_dn_bias, down_bias, (size_t)expert_count * hidden * 4, "down bias");
    // tiled copies for the grouped kernel
    static const char *env_tiled = diag_env("NNQ_MOE_TILED");   // tuning aid: 0 keeps the row kernels
    if (s == NNQ_OK && layout == NNQ_MOE_KN_GPTOSS && !(env_tiled && atoi(env_tiled) == 0)) {
        // [E, K, N] tensors: tiles of the transposed products (rows = N)
        const size_t gs = tiled_bytes_kn(2 * (int64_t)inter, hidden, nullptr);
        const size_t ds = tiled_bytes_kn(hidden, inter, nullptr);
        if (gs && ds) {
            const size_t gu_e = gate_up_bytes / expert_count, gus_e = gate_up_scales_bytes / expert_count;
            const size_t dn_e = down_bytes / expert_count, dns_e = down_scales_bytes / expert_count;
            s = check_cuda(ctx, cudaMalloc(&m->d_gu_tiled, gs * expert_count), "cudaMalloc tiled experts");
            if (s == NNQ_OK) s = check_cuda(ctx, cudaMalloc(&m->d_dn_tiled, ds * expert_count), "cudaMalloc tiled experts");
            for (int e = 0; e < expert_count && s == NNQ_OK; e++) {
                s = repack_kn_into(ctx, m->d_gu + e * gu_e, m->d_gu_scales + e * gus_e, 2 * (int64_t)inter, hidden, m->d_gu_tiled + e * gs);
                if (s == NNQ_OK) s = repack_kn_into(ctx, m->d_dn + e * dn_e, m->d_dn_scales + e * dns_e, hidden, inter, m->d_dn_tiled + e * ds);
            }
            if (s == NNQ_OK) s = check_cuda(ctx, cudaDeviceSynchronize(), "expert repack");
            m->gu_tile_stride = gs;
            m->dn_tile_stride = ds;
        }
    }
    if (s == NNQ_OK && layout == NNQ_MOE_NK && !(env_tiled && atoi(env_tiled) == 0)) {
        const size_t gs = tiled_bytes_for(fmt, 2 * (int64_t)inter, hidden, nullptr);
        const size_t ds = tiled_bytes_for(fmt, hidden, inter, nullptr);
        if (gs && ds) {
            const size_t gu_e = gate_up_bytes / expert_count, gus_e = gate_up_scales_bytes / expert_count;
            const size_t dn_e = down_bytes / expert_count, dns_e = down_scales_bytes / expert_count;
            s = check_cuda(ctx, cudaMalloc(&m->d_gu_tiled, gs * expert_count), "cudaMalloc tiled experts");
            if (s == NNQ_OK) s = check_cuda(ctx, cudaMalloc(&m->d_dn_tiled, ds * expert_count), "cudaMalloc tiled experts");
            for (int e = 0; e < expert_count && s == NNQ_OK; e++) {
                s = repack_into(ctx, fmt, m->d_gu + e * gu_e, m->d_gu_scales ? m->d_gu_scales + e * gus_e : nullptr,
                                2 * (int64_t)inter, hidden, m->d_gu_tiled + e * gs);
                if (s == NNQ_OK)
                    s = repack_into(ctx, fmt, m->d_dn + e * dn_e, m->d_dn_scales ? m->d_dn_scales + e * dns_e : nullptr,
                                    hidden, inter, m->d_dn_tiled + e * ds);
            }
            if (s == NNQ_OK) s = check_cuda(ctx, cudaDeviceSynchronize(), "expert repack");
            m->gu_tile_stride = gs;
            m->dn_tile_stride = ds;
        }
    }
    // bf16 scratch of the prefill-sized expert products: all local experts of the larger tensor
    if (s == NNQ_OK && ((layout == NNQ_MOE_NK && (fmt < NNQ_Q5_0 || fmt >= NNQ_F32_DENSE)) || (layout == NNQ_MOE_KN_GPTOSS && m->d_gu_tiled))) {
        s = dense_scratch_reserve(ctx, (int64_t)expert_count * 2 * inter, hidden);
        if (s == NNQ_OK) s = dense_scratch_reserve(ctx, (int64_t)expert_count * hidden, inter);
    }
    if (s != NNQ_OK) {
        nnq_moe_destroy(m);
        return s;
    }
    *out = m;
    return NNQ_OK;
}

nnq_status nnq_moe_create(nnq_ctx *ctx, int n_experts, int hidden, int inter, int top_k, float swiglu_limit,
                          const float *router_w, const float *router_b, nnq_moe_layout layout, nnq_format fmt,
                          const void *gate_up, size_t gate_up_bytes, const void *gate_up_scales,
                          size_t gate_up_scales_bytes, const float *gate_up_bias, const void *down,
                          size_t down_bytes, const void *down_scales, size_t down_scales_bytes,
                          const float *down_bias, nnq_moe **out) {
    return nnq_moe_create_shard(ctx, n_experts, 0, n_experts, hidden, inter, top_k, swiglu_limit, router_w, router_b,
                                layout, fmt, gate_up, gate_up_bytes, gate_up_scales, gate_up_scales_bytes,
                                gate_up_bias, down, down_bytes, down_scales, down_scales_bytes, down_bias, out);
}

void nnq_moe_destroy(nnq_moe *m) {
    if (!m) return;
    if (m->ctx) cudaSetDevice(m->ctx->device);
    cudaFree(m->d_router_w); cudaFree(m->d_router_b); cudaFree(m->d_gu); cudaFree(m->d_gu_scales);
    cudaFree(m->d_gu_bias); cudaFree(m->d_dn); cudaFree(m->d_dn_scales); cudaFree(m->d_dn_bias);
    cudaFree(m->d_gu_tiled); cudaFree(m->d_dn_tiled);
    cudaGetLastError();
    delete m;
}

static nnq_status moe_call(nnq_ctx *ctx, const nnq_moe *m, const void *x, nnq_dtype x_dt, int64_t tokens, float *y,
                           int *idx_out, float *wt_out, bool route_only, void *stream) {
    if (!ctx || !m) return NNQ_ERR_INVALID_ARG;
    if (m->ctx != ctx) return fail(ctx, NNQ_ERR_INVALID_ARG, "MoE block belongs to another context");
    if (tokens < 0 || tokens * m->top_k > (int64_t)1 << 30) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad token count");
    if ((int)x_dt < 0 || x_dt > NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown dtype");
    if (tokens == 0) return NNQ_OK;
    if (!x || (!route_only && !y)) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dt == NNQ_F32) return forward_typed<float>(ctx, m, (const float *)x, tokens, m->top_k, nullptr, nullptr, y, idx_out, wt_out, route_only, st);
    return forward_typed<__nv_bfloat16>(ctx, m, (const __nv_bfloat16 *)x, tokens, m->top_k, nullptr, nullptr, y, idx_out, wt_out, route_only, st);
}

nnq_status nnq_moe_forward_routed(nnq_ctx *ctx, const nnq_moe *m, const void *x_dev, nnq_dtype x_dt, int64_t rows, int slots,
                                  const int32_t *idx_dev, const float *weights_dev, float *y_dev, void *stream) {
    if (!ctx || !m) return NNQ_ERR_INVALID_ARG;
    if (m->ctx != ctx) return fail(ctx, NNQ_ERR_INVALID_ARG, "MoE block belongs to another context");
    if (slots < 1 || slots > kMaxTopK) return fail(ctx, NNQ_ERR_INVALID_ARG, "1..%d expert slots per row", kMaxTopK);
    if (rows < 0 || rows * slots > (int64_t)1 << 30) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad row count");
    if ((int)x_dt < 0 || x_dt > NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown dtype");
    if (rows == 0) return NNQ_OK;
    if (!x_dev || !y_dev || !idx_dev || !weights_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dt == NNQ_F32) return forward_typed<float>(ctx, m, (const float *)x_dev, rows, slots, idx_dev, weights_dev, y_dev, nullptr, nullptr, false, st);
    return forward_typed<__nv_bfloat16>(ctx, m, (const __nv_bfloat16 *)x_dev, rows, slots, idx_dev, weights_dev, y_dev, nullptr, nullptr, false, st);
}

nnq_status nnq_moe_gather_rows(nnq_ctx *ctx, const void *x_dev, nnq_dtype dt, const int32_t *index_dev, int64_t count, int64_t width,
                               void *out_dev, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if ((int)dt < 0 || dt > NNQ_BF16 || count < 0 || width < 1 || width > (1 << 24) || count > (int64_t)1 << 30) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad gather arguments");
    if (count == 0) return NNQ_OK;
    if (!x_dev || !index_dev || !out_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    if (dt == NNQ_F32) moe_gather_rows_kernel<float><<<(unsigned)count, 256, 0, st>>>((const float *)x_dev, index_dev, count, (int)width, (float *)out_dev);
    else moe_gather_rows_kernel<__nv_bfloat16><<<(unsigned)count, 256, 0, st>>>((const __nv_bfloat16 *)x_dev, index_dev, count, (int)width, (__nv_bfloat16 *)out_dev);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "gather launch");
}

nnq_status nnq_moe_combine_rows(nnq_ctx *ctx, const float *rows_dev, const int32_t *idx_dev, const float *weights_dev,
                                const int32_t *pos_dev, int64_t tokens, int hidden, int top_k, float *y_dev, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (tokens < 0 || hidden < 1 || top_k < 1 || top_k > kMaxTopK || tokens > (int64_t)1 << 28) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad combine arguments");
    if (tokens == 0) return NNQ_OK;
    if (!rows_dev || !idx_dev || !weights_dev || !pos_dev || !y_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    moe_combine_kernel<<<dim3((unsigned)tokens, tokens < 1024 ? 4 : 1), 256, 0, (cudaStream_t)stream>>>(rows_dev, idx_dev, weights_dev, pos_dev, (int)tokens, hidden,
                                                                                                        top_k, y_dev, 1, 0);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "combine launch");
}

nnq_status nnq_moe_forward(nnq_ctx *ctx, const nnq_moe *m, const void *x_dev, nnq_dtype x_dt, int64_t tokens,
                           float *y_dev, void *stream) {
    return moe_call(ctx, m, x_dev, x_dt, tokens, y_dev, nullptr, nullptr, false, stream);
}

nnq_status nnq_moe_route(nnq_ctx *ctx, const nnq_moe *m, const void *x_dev, nnq_dtype x_dt, int64_t tokens,
                         int32_t *idx_dev, float *weights_dev, void *stream) {
    return moe_call(ctx, m, x_dev, x_dt, tokens, nullptr, idx_dev, weights_dev, true, stream);
}

nnq_status nnq_moe_forward_static(nnq_ctx *ctx, const nnq_moe *m, const void *x_dev, nnq_dtype x_dt,
                                  int64_t tokens, float *y_dev, void *stream) {
    if (!ctx || !m) return NNQ_ERR_INVALID_ARG;
    if (m->ctx != ctx) return fail(ctx, NNQ_ERR_INVALID_ARG, "MoE block belongs to another context");
    if (tokens < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad token count");
    if ((int)x_dt < 0 || x_dt > NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown dtype");
    if (tokens == 0) return NNQ_OK;
    if (!x_dev || !y_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    // size check first: it needs no device work
    if (tokens > ((int64_t)1 << 24)) return fail(ctx, NNQ_ERR_UNSUPPORTED, "token count beyond the fixed scratch area");
    const size_t need = carve(nullptr, tokens, m, m->top_k).bytes;
    if (need > kStaticScratchBytes)
        return fail(ctx, NNQ_ERR_UNSUPPORTED,
                    "this call needs %zu bytes of scratch, the fixed area holds %zu: use nnq_moe_forward or fewer tokens",
                    need, (size_t)kStaticScratchBytes);
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    uint8_t *base = nullptr;
    if ((s = static_scratch_base(ctx, &base)) != NNQ_OK) return s;
    // Nothing in the area has to start at zero: every table and buffer is fully written by the
    // launches below before it is read (counts are stored, not accumulated), so stale contents
    // of an earlier call are harmless.
    const MoeScratch sc = carve(base, tokens, m, m->top_k);
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dt == NNQ_F32) return run_with_scratch<float>(ctx, m, (const float *)x_dev, tokens, m->top_k, nullptr, nullptr, y_dev, sc, false, st);
    return run_with_scratch<__nv_bfloat16>(ctx, m, (const __nv_bfloat16 *)x_dev, tokens, m->top_k, nullptr, nullptr, y_dev, sc, false, st);
}

}  // extern "C"
