// One decode step (one token, batch 1) of a Qwen3-shaped decoder on the device: embedding row ->
// N x [RMSNorm -> q/k/v products -> per-head QK-norm + half-split RoPE -> KV append -> grouped-query
// attention over the cache -> o product -> residual -> RMSNorm -> gate/up products -> silu * up ->
// down product -> residual] -> final RMSNorm -> vocabulary product -> greedy argmax.
// Follows crates/nn-qwen3/src/layers.rs:40-47,94-167,205-226 (MLP, attention, decoder layer),
// crates/nn-core/src/layers/rms_norm.rs:87-100, layers/attention/rope.rs:78-106 (tables),
// rope_half_split.rs:98-134 (rotation), attention/sdpa.rs:59-71, dyn_tensor/ops/math.rs:140 (silu)
// and layers/generation/autoregressive_sampling.rs:14-21 (argmax: the last of equal maxima).
//
// The quantized products are the library's own (nnq_linear / nnq_linear_batch); this file adds the
// small kernels between them. Token and position live in device memory and are advanced by the
// last kernel of a step, so the launches of one step can be captured once and replayed per token.
#include <cuda_bf16.h>
#include <math.h>
#include <string.h>

#include <new>

#include "comm.cuh"
#include "nnq_internal.h"
#include "pdl.cuh"

namespace nnq {
nnq_status comm_view(nnq_comm *c, CommView *out);   // comm.cu
}

struct nnq_decoder {
    nnq_ctx *ctx;
    nnq_decoder_config cfg;
    struct Layer {
        const nnq_weight *q, *k, *v, *o, *gate, *up, *down;
        float *in_norm, *post_norm, *q_norm, *k_norm;   // device copies
    } *layers;
    const void *d_embed;        // [vocab, hidden] bf16, caller-owned
    float *d_final_norm;
    const nnq_weight *lm_head;
    float *d_cos, *d_sin;       // [max_seq, head_dim / 2]
    float *d_kcache, *d_vcache; // [layers, kv_heads, max_seq, head_dim]
    float *d_h, *d_delta, *d_q, *d_k, *d_v, *d_qrot, *d_g, *d_u, *d_logits, *d_part;
    unsigned int *d_arrived;   // per kv head: attention CTAs that have published their record
    void *d_xn, *d_attn, *d_mid;   // activations fed to the products (f32 or bf16)
    int *d_state;               // [0] token, [1] position, [2] steps taken; then the argmax scratch
    int *d_tokens;              // generated tokens, [max_seq]
    int act_dt;
    int ready;                  // bit set of what has been supplied
    nnq_comm *comm;             // tensor parallel: exchange of the row-parallel products (NULL when tp_world = 1)
    int lh, lkv;                // query / key-value heads held by this rank
    int head_rows, head_row0;   // rows of the vocabulary projection held by this rank and the first of them
    long long host_pos;         // position of the next step as far as the host knows it (-1: unknown)
    // prompt pass: row-major [rows, width] versions of the step's buffers, allocated by the first
    // nnq_decoder_prefill call (pf_rows rows)
    int pf_rows;
    float *pf_h, *pf_delta, *pf_q, *pf_k, *pf_v, *pf_qrot, *pf_g, *pf_u;
    void *pf_xn, *pf_attn, *pf_mid;
    int *pf_tokens;
};

namespace nnq {

constexpr int kAttnRanges = 32;   // CTAs per kv head in the decode step's attention
constexpr int kAttnWarps = 4;
// Rows of a prompt that go through the layers together: large enough that the products run on the
// decode-once tensor path with several row tiles per weight tile (about 210 KB of buffers per row at
// the Qwen3-8B shape).
constexpr int kPrefillRows = 1024;
constexpr int kArgmaxBlocks = 128;

__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nw; w++) t += red[w];
    return t;
}

__device__ __forceinline__ void store_act(void *dst, int dt, int i, float v) {
    if (dt == NNQ_F32) reinterpret_cast<float *>(dst)[i] = v;
    else reinterpret_cast<__nv_bfloat16 *>(dst)[i] = __float2bfloat16_rn(v);
}

// h = embedding row of the current token (first layer), or h += delta; xn = RMSNorm(h) * w.
// One CTA; every thread keeps its (up to 8) elements in registers between the two phases.
__global__ void __launch_bounds__(1024)
dec_norm_kernel(float *__restrict__ h, const float *__restrict__ delta, const __nv_bfloat16 *__restrict__ embed,
                const int *__restrict__ state, const float *__restrict__ w, float eps, void *__restrict__ xn, int act_dt,
                int hidden) {
    pdl_prologue();
    __shared__ float red[32];
    const int tok = embed ? state[0] : 0;
    float v[8], wv[8];
    float ss = 0.0f;
#pragma unroll
    for (int r = 0; r < 8; r++) {
        const int i = threadIdx.x + r * 1024;
        v[r] = 0.0f;
        wv[r] = 0.0f;
        if (i < hidden) {
            v[r] = embed ? __bfloat162float(embed[(size_t)tok * hidden + i]) : h[i] + delta[i];
            wv[r] = w[i];
            h[i] = v[r];
            ss = fmaf(v[r], v[r], ss);
        }
    }
    for (int i = threadIdx.x + 8 * 1024; i < hidden; i += 1024) {   // wider models: the tail goes through memory
        const float t = embed ? __bfloat162float(embed[(size_t)tok * hidden + i]) : h[i] + delta[i];
        h[i] = t;
        ss = fmaf(t, t, ss);
    }
    const float mean = block_sum(ss, red) / (float)hidden;
    const float rms = sqrtf(mean + eps);
#pragma unroll
    for (int r = 0; r < 8; r++) {
        const int i = threadIdx.x + r * 1024;
        if (i < hidden) store_act(xn, act_dt, i, (v[r] / rms) * wv[r]);
    }
    for (int i = threadIdx.x + 8 * 1024; i < hidden; i += 1024) store_act(xn, act_dt, i, (h[i] / rms) * w[i]);
}

// One CTA per head (query heads, then key heads, then value heads), one thread per dimension:
// RMSNorm over the head (q, k), half-split rotation at the current position, append k / v.
__global__ void __launch_bounds__(256)
dec_qk_rope_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                   const float *__restrict__ qw, const float *__restrict__ kw, const float *__restrict__ cosv,
                   const float *__restrict__ sinv, const int *__restrict__ state, float eps, float *__restrict__ qrot,
                   float *__restrict__ kcache, float *__restrict__ vcache, int n_heads, int n_kv, int hd, int max_seq) {
    pdl_prologue();
    __shared__ float red[32];
    __shared__ float xs[256];
    const int head = blockIdx.x, d = threadIdx.x, pos = state[1];
    const int half = hd / 2;
    if (head >= n_heads + n_kv) {   // value head: plain append
        const int kvh = head - n_heads - n_kv;
        if (d < hd) vcache[((size_t)kvh * max_seq + pos) * hd + d] = v[kvh * hd + d];
        return;
    }
    const bool is_q = head < n_heads;
    const float *src = is_q ? q + head * hd : k + (head - n_heads) * hd;
    const float *w = is_q ? qw : kw;
    const float x = d < hd ? src[d] : 0.0f;
    const float mean = block_sum(x * x, red) / (float)hd;
    const float rms = sqrtf(mean + eps);
    if (d < hd) xs[d] = (x / rms) * w[d];
    __syncthreads();
    if (d >= hd) return;
    const int i = d < half ? d : d - half;
    const float c = cosv[(size_t)pos * half + i], s = sinv[(size_t)pos * half + i];
    // y1 = x1 cos - x2 sin; y2 = x1 sin + x2 cos
    const float y = d < half ? xs[d] * c - xs[d + half] * s : xs[d - half] * s + xs[d] * c;
    if (is_q) qrot[head * hd + d] = y;
    else kcache[((size_t)(head - n_heads) * max_seq + pos) * hd + d] = y;
}

// Grouped-query attention over the cache in one launch. The keys are taken in batches of 32; a
// kv head's batches are dealt to kAttnRanges CTAs (contiguous ranges) and inside a CTA to its four
// warps. For a batch, lane j forms the dot products of key j with every query head of the group (the
// query vectors sit in shared memory, the key row is read once for the whole group), the batch joins
// the running softmax of each head (maximum, sum), then the value rows are read coalesced (lane l
// owns dimensions 4l .. 4l+3) and weighted with the probabilities passed by shuffle. The warps of a
// CTA merge through shared memory into one record per head, (m, l, acc[hd]), in global memory; the
// CTA that finishes last for its kv head (an arrival counter, reset by that CTA for the next
// launch) merges the records of all ranges and writes the output rows:
// out[head, d] = sum_s acc_s[d] e^(m_s - M) / sum_s l_s e^(m_s - M).
template <int G>
__global__ void __launch_bounds__(kAttnWarps * 32)
dec_attn_kernel(const float *__restrict__ qrot, const float *__restrict__ kcache, const float *__restrict__ vcache,
                const int *__restrict__ state, float scale, float *__restrict__ part, unsigned int *__restrict__ arrived,
                void *__restrict__ out, int act_dt, int hd, int max_seq) {
    pdl_prologue();
    __shared__ __align__(16) float qs[G][128];
    __shared__ __align__(16) float wacc[kAttnWarps][G][128];
    __shared__ float wm[kAttnWarps][G], wl[kAttnWarps][G];
    __shared__ int s_last;
    const int kvh = blockIdx.x, range = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ctx = state[1] + 1;
    const int nb = (ctx + 31) >> 5;                              // batches of 32 keys in the context
    const int bper = (nb + kAttnRanges - 1) / kAttnRanges;       // batches per range
    const int used = (nb + bper - 1) / bper;                     // ranges that hold keys
    const int b_lo = range * bper, b_hi = min(nb, b_lo + bper);
    if (b_lo < b_hi) {
        for (int i = threadIdx.x; i < G * 32; i += kAttnWarps * 32)
            *reinterpret_cast<float4 *>(&qs[i >> 5][4 * (i & 31)]) = *reinterpret_cast<const float4 *>(qrot + (kvh * G + (i >> 5)) * hd + 4 * (i & 31));
        __syncthreads();
        float m[G], l[G];
        float4 acc[G];
#pragma unroll
        for (int g = 0; g < G; g++) {
            m[g] = -INFINITY;
            l[g] = 0.0f;
            acc[g] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        const float *kb = kcache + (size_t)kvh * max_seq * hd, *vb = vcache + (size_t)kvh * max_seq * hd;
        for (int b = b_lo + warp; b < b_hi; b += kAttnWarps) {
            const int b0 = b << 5, j1 = min(ctx, b0 + 32);
            const int j = b0 + lane;
            const bool valid = j < j1;
            const float4 *krow = reinterpret_cast<const float4 *>(kb + (size_t)(valid ? j : b0) * hd);
            // the value rows of the batch are wanted after the softmax: ask L2 for them now (lane j: row j)
            if (valid) {
                const char *vrow = reinterpret_cast<const char *>(vb + (size_t)j * hd);
#pragma unroll
                for (int c = 0; c < 4; c++) asm volatile("prefetch.global.L2 [%0];" ::"l"(vrow + 128 * c));
            }
            float dot[G];
#pragma unroll
            for (int g = 0; g < G; g++) dot[g] = 0.0f;
#pragma unroll 16
            for (int d4 = 0; d4 < 32; d4++) {
                const float4 kv = krow[d4];
#pragma unroll
                for (int g = 0; g < G; g++) {
                    const float4 qv = *reinterpret_cast<const float4 *>(&qs[g][4 * d4]);
                    dot[g] = fmaf(qv.x, kv.x, fmaf(qv.y, kv.y, fmaf(qv.z, kv.z, fmaf(qv.w, kv.w, dot[g]))));
                }
            }
            float p[G];
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float s = valid ? dot[g] * scale : -INFINITY;
                float bm = s;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, off));
                const float mn = fmaxf(m[g], bm);   // finite: the batch holds at least one key
                const float corr = expf(m[g] - mn);
                p[g] = expf(s - mn);
                float ps = p[g];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xFFFFFFFFu, ps, off);
                l[g] = l[g] * corr + ps;
                acc[g].x *= corr; acc[g].y *= corr; acc[g].z *= corr; acc[g].w *= corr;
                m[g] = mn;
            }
            const int nk = j1 - b0;
#pragma unroll 4
            for (int jj = 0; jj < nk; jj++) {
                const float4 vv = *reinterpret_cast<const float4 *>(vb + (size_t)(b0 + jj) * hd + 4 * lane);
#pragma unroll
                for (int g = 0; g < G; g++) {
                    const float pj = __shfl_sync(0xFFFFFFFFu, p[g], jj);
                    acc[g].x = fmaf(pj, vv.x, acc[g].x);
                    acc[g].y = fmaf(pj, vv.y, acc[g].y);
                    acc[g].z = fmaf(pj, vv.z, acc[g].z);
                    acc[g].w = fmaf(pj, vv.w, acc[g].w);
                }
            }
        }
        // the warps of the CTA -> one record per head
#pragma unroll
        for (int g = 0; g < G; g++) {
            if (lane == 0) {
                wm[warp][g] = m[g];
                wl[warp][g] = l[g];
            }
            *reinterpret_cast<float4 *>(&wacc[warp][g][4 * lane]) = acc[g];
        }
        __syncthreads();
        for (int i = threadIdx.x; i < G * 128; i += kAttnWarps * 32) {
            const int g = i >> 7, dd = i & 127;
            float M = wm[0][g];
#pragma unroll
            for (int w = 1; w < kAttnWarps; w++) M = fmaxf(M, wm[w][g]);   // warp 0 always holds a batch: finite
            float L = 0.0f, a = 0.0f;
#pragma unroll
            for (int w = 0; w < kAttnWarps; w++) {
                const float e = wm[w][g] == -INFINITY ? 0.0f : expf(wm[w][g] - M);
                L = fmaf(wl[w][g], e, L);
                a = fmaf(wacc[w][g][dd], e, a);
            }
            float *o = part + ((size_t)(kvh * kAttnRanges + range) * G + g) * (hd + 4);   // record: m, l, pad, pad, acc[hd]
            if (dd == 0) {
                o[0] = M;
                o[1] = L;
            }
            if (dd < hd) o[4 + dd] = a;
        }
    }
    // arrival: the records above are published before the count, the last CTA reads them after it
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(arrived + kvh, 1u) == (unsigned)(kAttnRanges - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // a warp per head, a lane per four dimensions; every load of a pass is issued before the first
    // is used (the records sit in L2: the pass costs one round trip, not one per range)
    for (int g = warp; g < G; g += kAttnWarps) {
        const float *rec = part + ((size_t)(kvh * kAttnRanges) * G + g) * (hd + 4);
        const size_t step = (size_t)G * (hd + 4);
        float2 ml[kAttnRanges];
#pragma unroll
        for (int s = 0; s < kAttnRanges; s++)
            ml[s] = s < used ? __ldcg(reinterpret_cast<const float2 *>(rec + s * step)) : make_float2(-INFINITY, 0.0f);
        float M = ml[0].x;
#pragma unroll
        for (int s = 1; s < kAttnRanges; s++) M = fmaxf(M, ml[s].x);
        float L = 0.0f;
#pragma unroll
        for (int s = 0; s < kAttnRanges; s++) {
            ml[s].x = s < used ? expf(ml[s].x - M) : 0.0f;
            L = fmaf(ml[s].y, ml[s].x, L);
        }
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int h = 0; h < kAttnRanges; h += 16) {
            float4 v[16];
#pragma unroll
            for (int s = 0; s < 16; s++)
                v[s] = h + s < used ? __ldcg(reinterpret_cast<const float4 *>(rec + (h + s) * step + 4) + lane) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int s = 0; s < 16; s++) {
                a.x = fmaf(v[s].x, ml[h + s].x, a.x);
                a.y = fmaf(v[s].y, ml[h + s].x, a.y);
                a.z = fmaf(v[s].z, ml[h + s].x, a.z);
                a.w = fmaf(v[s].w, ml[h + s].x, a.w);
            }
        }
        const int at = (kvh * G + g) * hd + 4 * lane;
        store_act(out, act_dt, at, a.x / L);
        store_act(out, act_dt, at + 1, a.y / L);
        store_act(out, act_dt, at + 2, a.z / L);
        store_act(out, act_dt, at + 3, a.w / L);
    }
    if (threadIdx.x == 0) arrived[kvh] = 0;   // the next launch starts after this grid has ended
}

__global__ void dec_silu_mul_kernel(const float *__restrict__ g, const float *__restrict__ u, void *__restrict__ mid,
                                    int act_dt, int n) {
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float x = g[i];
        store_act(mid, act_dt, i, (x / (1.0f + expf(-x))) * u[i]);
    }
}

// larger value wins; of equal values the larger index (the reference keeps the last maximum)
__device__ __forceinline__ void arg_better(float &bv, int &bi, float v, int i) {
    if (v > bv || (v == bv && i > bi)) {
        bv = v;
        bi = i;
    }
}

__global__ void __launch_bounds__(256)
dec_argmax_stage1_kernel(const float *__restrict__ logits, int n, float *__restrict__ bv_out, int *__restrict__ bi_out) {
    pdl_prologue();
    __shared__ float sv[8];
    __shared__ int si[8];
    float bv = -INFINITY;
    int bi = -1;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) arg_better(bv, bi, logits[i], i);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
        arg_better(bv, bi, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = bv;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) arg_better(bv, bi, sv[w], si[w]);
        bv_out[blockIdx.x] = bv;
        bi_out[blockIdx.x] = bi;
    }
}

// Records the winning token and advances the device-side (token, position) pair. state[3] is set
// by the step that fills the last position; a step that finds it set has nowhere to write:
// it raises the context's status word (2 = context full) and changes nothing.
__device__ __forceinline__ void dec_commit_token(int bi, int *state, int *tokens, int max_seq) {
    if (bi < 0) bi = 0;   // all NaN: the reference returns index 0
    const int pos = state[1];
    tokens[pos] = bi;
    state[0] = bi;
    if (pos + 1 < max_seq) state[1] = pos + 1;
    else state[3] = 1;
    state[2] += 1;
}

// picks the winner among the block maxima
__global__ void dec_argmax_stage2_kernel(const float *__restrict__ bv_in, const int *__restrict__ bi_in, int blocks,
                                         int *__restrict__ state, int *__restrict__ tokens, int max_seq, int *status) {
    pdl_prologue();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    if (state[3]) {
        atomicExch(status, 2);
        return;
    }
    float bv = -INFINITY;
    int bi = -1;
    for (int b = 0; b < blocks; b++) arg_better(bv, bi, bv_in[b], bi_in[b]);
    dec_commit_token(bi, state, tokens, max_seq);
}

// Vocabulary-parallel head: every rank holds the maximum of its slice of the logits; the ranks
// exchange (value, index) through the last 16 bytes of their communicator slots as two 8-byte
// (payload, sequence number) stores, wait (bounded) for the peers' records and all pick the same
// winner: the larger value, of equal values the larger index -- the reference's "last maximum"
// rule survives the gather because it only depends on (value, index), not on arrival order.
__global__ void dec_argmax_exchange_kernel(const float *__restrict__ bv_in, const int *__restrict__ bi_in, int blocks,
                                           int index_offset, uint8_t *const *peers, int rank, int world, size_t slot_bytes,
                                           int *__restrict__ state, int *__restrict__ tokens, int max_seq, int *status) {
    pdl_prologue();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    uint8_t *local = peers[rank];
    const unsigned seq = *reinterpret_cast<volatile unsigned *>(local) + 1u;
    const unsigned limit = comm_spin_limit(local);
    float bv = -INFINITY;
    int bi = -1;
    for (int b = 0; b < blocks; b++) arg_better(bv, bi, bv_in[b], bi_in[b]);
    if (bi >= 0) bi += index_offset;
    const int par = (int)(seq & 1u);
    const size_t mine = comm_data_offset(par, rank, world, slot_bytes) + slot_bytes - 16;
    for (int p = 0; p < world; p++) {
        if (p == rank) continue;
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(peers[p] + mine), "r"(__float_as_uint(bv)), "r"(seq) : "memory");
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(peers[p] + mine + 8), "r"((unsigned)bi), "r"(seq) : "memory");
    }
    bool ok = true;
    for (int r = 0; r < world; r++) {
        if (r == rank) continue;
        const uint8_t *src = local + comm_data_offset(par, r, world, slot_bytes) + slot_bytes - 16;
        uint32_t vb = 0, ib = 0, t0 = 0, t1 = 0;
        unsigned spins = 0;
        do {
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(vb), "=r"(t0) : "l"(src) : "memory");
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(ib), "=r"(t1) : "l"(src + 8) : "memory");
        } while ((t0 != seq || t1 != seq) && ++spins <= limit);
        if (t0 != seq || t1 != seq) {
            ok = false;
            continue;
        }
        arg_better(bv, bi, __uint_as_float(vb), (int)ib);
    }
    if (!ok) atomicExch(status, 1);
    if (state[3]) atomicExch(status, 2);
    else dec_commit_token(bi, state, tokens, max_seq);
    *reinterpret_cast<volatile unsigned *>(local) = seq;   // this exchange is complete
}

// ---- prompt pass: the same operations over a block of rows (one row per prompt token) ----

// row r: h = embedding of tokens[r] (first layer) or h += delta; xn = RMSNorm(h) * w. One CTA per row.
__global__ void __launch_bounds__(256)
dec_norm_rows_kernel(float *__restrict__ h, const float *__restrict__ delta, const __nv_bfloat16 *__restrict__ embed,
                     const int *__restrict__ tokens, const float *__restrict__ w, float eps, void *__restrict__ xn, int act_dt,
                     int hidden) {
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    float *hr = h + r * hidden;
    const float *dr = delta ? delta + r * hidden : nullptr;
    const __nv_bfloat16 *er = embed ? embed + (size_t)tokens[r] * hidden : nullptr;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = er ? __bfloat162float(er[i]) : hr[i] + dr[i];
        hr[i] = v;
        ss = fmaf(v, v, ss);
    }
    const float rms = sqrtf(block_sum(ss, red) / (float)hidden + eps);
    char *xr = reinterpret_cast<char *>(xn) + r * hidden * (act_dt == NNQ_F32 ? 4 : 2);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) store_act(xr, act_dt, i, (hr[i] / rms) * w[i]);
}

// grid (heads, rows): per-head RMSNorm + half-split rotation at position pos0 + row, append of k / v
__global__ void __launch_bounds__(256)
dec_qk_rope_rows_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                        const float *__restrict__ qw, const float *__restrict__ kw, const float *__restrict__ cosv,
                        const float *__restrict__ sinv, int pos0, float eps, float *__restrict__ qrot, float *__restrict__ kcache,
                        float *__restrict__ vcache, int n_heads, int n_kv, int hd, int max_seq) {
    __shared__ float red[32];
    __shared__ float xs[256];
    const int head = blockIdx.x, row = blockIdx.y, d = threadIdx.x, pos = pos0 + row;
    const int half = hd / 2;
    const size_t qoff = (size_t)row * n_heads * hd, kvoff = (size_t)row * n_kv * hd;
    if (head >= n_heads + n_kv) {
        const int kvh = head - n_heads - n_kv;
        if (d < hd) vcache[((size_t)kvh * max_seq + pos) * hd + d] = v[kvoff + kvh * hd + d];
        return;
    }
    const bool is_q = head < n_heads;
    const float *src = is_q ? q + qoff + head * hd : k + kvoff + (head - n_heads) * hd;
    const float *w = is_q ? qw : kw;
    const float x = d < hd ? src[d] : 0.0f;
    const float rms = sqrtf(block_sum(x * x, red) / (float)hd + eps);
    if (d < hd) xs[d] = (x / rms) * w[d];
    __syncthreads();
    if (d >= hd) return;
    const int i = d < half ? d : d - half;
    const float c = cosv[(size_t)pos * half + i], sn = sinv[(size_t)pos * half + i];
    const float y = d < half ? xs[d] * c - xs[d + half] * sn : xs[d - half] * sn + xs[d] * c;
    if (is_q) qrot[qoff + head * hd + d] = y;
    else kcache[((size_t)(head - n_heads) * max_seq + pos) * hd + d] = y;
}

// Causal attention of a block of query rows over the cache: one warp per (kv head, R consecutive
// rows) serves the G query heads of the group for all R rows (G * R = 16 query vectors in shared
// memory), so that a key / value row is read once per R rows; row r sees keys 0 .. pos0 + r (the mask
// of the reference's prompt pass: crates/nn-core/src/layers/attention/sdpa.rs:118-141). Same
// batch-of-32-keys scheme as the decode kernel, normalised output written directly.
template <int G, int R>
__global__ void __launch_bounds__(32)
dec_attn_rows_kernel(const float *__restrict__ qrot, const float *__restrict__ kcache, const float *__restrict__ vcache, int pos0,
                     int n, float scale, void *__restrict__ out, int act_dt, int n_heads, int hd, int max_seq) {
    constexpr int P = G * R;   // pair p = r * G + g
    __shared__ __align__(16) float qs[P][128];
    const int kvh = blockIdx.x, r0 = blockIdx.y * R, lane = threadIdx.x;
    const int rows = min(R, n - r0);
    const int jmax = pos0 + r0 + rows;   // keys the last row of this block sees
#pragma unroll
    for (int p = 0; p < P; p++) {
        const int row = r0 + min(p / G, rows - 1);   // rows past the end repeat the last one; not stored
        *reinterpret_cast<float4 *>(&qs[p][4 * lane]) =
            *reinterpret_cast<const float4 *>(qrot + (size_t)row * n_heads * hd + (kvh * G + p % G) * hd + 4 * lane);
    }
    __syncwarp();
    float m[P], l[P];
    float4 acc[P];
#pragma unroll
    for (int p = 0; p < P; p++) {
        m[p] = -INFINITY;
        l[p] = 0.0f;
        acc[p] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    const float *kb = kcache + (size_t)kvh * max_seq * hd, *vb = vcache + (size_t)kvh * max_seq * hd;
    for (int b0 = 0; b0 < jmax; b0 += 32) {
        const int j = b0 + lane;
        const float4 *krow = reinterpret_cast<const float4 *>(kb + (size_t)(j < jmax ? j : b0) * hd);
        float dot[P];
#pragma unroll
        for (int p = 0; p < P; p++) dot[p] = 0.0f;
#pragma unroll 8
        for (int d4 = 0; d4 < 32; d4++) {
            const float4 kv = krow[d4];
#pragma unroll
            for (int p = 0; p < P; p++) {
                const float4 qv = *reinterpret_cast<const float4 *>(&qs[p][4 * d4]);
                dot[p] = fmaf(qv.x, kv.x, fmaf(qv.y, kv.y, fmaf(qv.z, kv.z, fmaf(qv.w, kv.w, dot[p]))));
            }
        }
#pragma unroll
        for (int p = 0; p < P; p++) {
            // key j is visible to row r0 + p / G up to position pos0 + row; the first batch holds key 0
            // for every row, so the running maximum is finite from then on
            const bool valid = j <= pos0 + r0 + min(p / G, rows - 1);
            const float sc = valid ? dot[p] * scale : -INFINITY;
            float bm = sc;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, off));
            const float mn = fmaxf(m[p], bm);
            const float corr = expf(m[p] - mn);
            dot[p] = expf(sc - mn);   // the probability, kept in place of the score
            float ps = dot[p];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xFFFFFFFFu, ps, off);
            l[p] = l[p] * corr + ps;
            acc[p].x *= corr; acc[p].y *= corr; acc[p].z *= corr; acc[p].w *= corr;
            m[p] = mn;
        }
        const int nb = min(32, jmax - b0);
        for (int jj = 0; jj < nb; jj++) {
            const float4 vv = *reinterpret_cast<const float4 *>(vb + (size_t)(b0 + jj) * hd + 4 * lane);
#pragma unroll
            for (int p = 0; p < P; p++) {
                const float pj = __shfl_sync(0xFFFFFFFFu, dot[p], jj);
                acc[p].x = fmaf(pj, vv.x, acc[p].x);
                acc[p].y = fmaf(pj, vv.y, acc[p].y);
                acc[p].z = fmaf(pj, vv.z, acc[p].z);
                acc[p].w = fmaf(pj, vv.w, acc[p].w);
            }
        }
    }
#pragma unroll
    for (int p = 0; p < P; p++) {
        if (p / G >= rows) continue;
        char *orow = reinterpret_cast<char *>(out) + (size_t)(r0 + p / G) * n_heads * hd * (act_dt == NNQ_F32 ? 4 : 2);
        const int base = (kvh * G + p % G) * hd + 4 * lane;
        store_act(orow, act_dt, base, acc[p].x / l[p]);
        store_act(orow, act_dt, base + 1, acc[p].y / l[p]);
        store_act(orow, act_dt, base + 2, acc[p].z / l[p]);
        store_act(orow, act_dt, base + 3, acc[p].w / l[p]);
    }
}

// position of the last prompt token, for the commit of its greedy successor
__global__ void dec_set_pos_kernel(int *state, int pos) {
    if (threadIdx.x == 0 && blockIdx.x == 0) state[1] = pos;
}

}  // namespace nnq

using namespace nnq;

extern "C" {

static nnq_status dev_alloc(nnq_ctx *ctx, void **p, size_t bytes, const char *what) {
    nnq_status s = check_cuda(ctx, cudaMalloc(p, bytes ? bytes : 16), what);
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemset(*p, 0, bytes ? bytes : 16), what);
    return s;
}

nnq_status nnq_decoder_create(nnq_ctx *ctx, const nnq_decoder_config *cfg, nnq_decoder **out) {
    if (!ctx || !cfg || !out) return NNQ_ERR_INVALID_ARG;
    *out = nullptr;
    nnq_decoder_config c = *cfg;
    if (c.tp_world == 0) c.tp_world = 1;   // a zeroed field means no tensor parallelism
    if (c.hidden < 1 || c.n_heads < 1 || c.n_kv_heads < 1 || c.ffn < 1 || c.n_layers < 1 || c.vocab < 1 || c.max_seq < 1)
        return fail(ctx, NNQ_ERR_INVALID_ARG, "bad decoder dimensions");
    if (c.head_dim != 128) return fail(ctx, NNQ_ERR_UNSUPPORTED, "the attention kernel is written for head_dim = 128 (got %d)", c.head_dim);
    const int grp = c.n_heads % c.n_kv_heads ? 0 : c.n_heads / c.n_kv_heads;
    if (grp != 1 && grp != 2 && grp != 4 && grp != 8)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "query heads per key/value head must be 1, 2, 4 or 8");
    if (c.act_dtype != NNQ_F32 && c.act_dtype != NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown activation dtype");
    if (c.tp_world < 1 || c.tp_world > 8 || c.tp_rank < 0 || c.tp_rank >= c.tp_world)
        return fail(ctx, NNQ_ERR_INVALID_ARG, "bad tensor-parallel rank %d of %d", c.tp_rank, c.tp_world);
    if (c.n_kv_heads % c.tp_world || c.ffn % c.tp_world)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "key/value heads and the FFN width must divide by the tensor-parallel world size");
    if (!(c.rope_theta > 0.0)) return fail(ctx, NNQ_ERR_INVALID_ARG, "rope_theta must be positive");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    nnq_decoder *d = new (std::nothrow) nnq_decoder();
    if (!d) return fail(ctx, NNQ_ERR_OUT_OF_MEMORY, "host allocation failed");
    memset(d, 0, sizeof(*d));
    d->ctx = ctx;
    d->cfg = c;
    d->act_dt = c.act_dtype;
    d->lh = c.n_heads / c.tp_world;
    d->lkv = c.n_kv_heads / c.tp_world;
    d->head_rows = c.vocab;
    d->head_row0 = 0;
    d->host_pos = -1;
    d->layers = new (std::nothrow) nnq_decoder::Layer[c.n_layers]();
    if (!d->layers) {
        delete d;
        return fail(ctx, NNQ_ERR_OUT_OF_MEMORY, "host allocation failed");
    }
    const int hd = c.head_dim, half = hd / 2, qdim = d->lh * hd, kvdim = d->lkv * hd, lffn = c.ffn / c.tp_world;
    const size_t es = c.act_dtype == NNQ_F32 ? 4 : 2;
    const size_t cache = (size_t)c.n_layers * d->lkv * c.max_seq * hd * 4;
    s = dev_alloc(ctx, (void **)&d->d_cos, (size_t)c.max_seq * half * 4, "rope table");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_sin, (size_t)c.max_seq * half * 4, "rope table");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_kcache, cache, "key cache");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_vcache, cache, "value cache");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_h, (size_t)c.hidden * 4, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_delta, (size_t)c.hidden * 4, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_q, (size_t)qdim * 4, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_k, (size_t)kvdim * 4, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_v, (size_t)kvdim * 4, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_qrot, (size_t)qdim * 4, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_g, (size_t)lffn * 4, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_u, (size_t)lffn * 4, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_logits, (size_t)c.vocab * 4, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_part, (size_t)d->lh * kAttnRanges * (hd + 4) * 4, "attention partials");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_arrived, (size_t)(d->lkv > 0 ? d->lkv : 1) * 4, "attention arrival counters");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemset(d->d_arrived, 0, (size_t)(d->lkv > 0 ? d->lkv : 1) * 4), "attention arrival counters clear");
    if (s == NNQ_OK) s = dev_alloc(ctx, &d->d_xn, (size_t)c.hidden * es, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, &d->d_attn, (size_t)qdim * es, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, &d->d_mid, (size_t)lffn * es, "decoder buffer");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_state, (4 + 2 * kArgmaxBlocks) * 4, "decoder state");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_tokens, (size_t)c.max_seq * 4, "token log");
    if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->d_final_norm, (size_t)c.hidden * 4, "final norm");
    for (int l = 0; l < c.n_layers && s == NNQ_OK; l++) {
        nnq_decoder::Layer &L = d->layers[l];
        s = dev_alloc(ctx, (void **)&L.in_norm, (size_t)c.hidden * 4, "norm weight");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&L.post_norm, (size_t)c.hidden * 4, "norm weight");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&L.q_norm, (size_t)hd * 4, "norm weight");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&L.k_norm, (size_t)hd * 4, "norm weight");
    }
    if (s == NNQ_OK) {
        // tables exactly as the reference builds them: inv_freq in f32, the angle rounded to f32
        float *hc = new (std::nothrow) float[(size_t)c.max_seq * half], *hs = new (std::nothrow) float[(size_t)c.max_seq * half];
        if (!hc || !hs) s = fail(ctx, NNQ_ERR_OUT_OF_MEMORY, "host allocation failed");
        if (s == NNQ_OK) {
            for (int i = 0; i < half; i++) {
                const float inv = (float)(1.0 / pow(c.rope_theta, (double)(2 * i) / (double)hd));
                for (int p = 0; p < c.max_seq; p++) {
                    const float angle = (float)((double)p * (double)inv);
                    hc[(size_t)p * half + i] = cosf(angle);
                    hs[(size_t)p * half + i] = sinf(angle);
                }
            }
            s = check_cuda(ctx, cudaMemcpy(d->d_cos, hc, (size_t)c.max_seq * half * 4, cudaMemcpyHostToDevice), "rope table");
            if (s == NNQ_OK) s = check_cuda(ctx, cudaMemcpy(d->d_sin, hs, (size_t)c.max_seq * half * 4, cudaMemcpyHostToDevice), "rope table");
        }
        delete[] hc;
        delete[] hs;
    }
    if (s != NNQ_OK) {
        nnq_decoder_destroy(d);
        return s;
    }
    *out = d;
    return NNQ_OK;
}

static bool shape_is(const nnq_weight *w, int64_t n, int64_t k) { return w && w->n == n && w->k == k; }

nnq_status nnq_decoder_set_layer(nnq_decoder *d, int layer, const nnq_weight *q, const nnq_weight *k, const nnq_weight *v,
                                 const nnq_weight *o, const nnq_weight *gate, const nnq_weight *up, const nnq_weight *down,
                                 const float *in_norm, const float *post_norm, const float *q_norm, const float *k_norm) {
    if (!d) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = d->ctx;
    const nnq_decoder_config &c = d->cfg;
    if (layer < 0 || layer >= c.n_layers) return fail(ctx, NNQ_ERR_INVALID_ARG, "layer %d out of range", layer);
    if (!in_norm || !post_norm || !q_norm || !k_norm) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL norm weight");
    // with tensor parallelism: this rank's column shards of q / k / v / gate / up and row shards of o / down
    const int64_t qdim = (int64_t)d->lh * c.head_dim, kvdim = (int64_t)d->lkv * c.head_dim, lffn = c.ffn / c.tp_world;
    if (!shape_is(q, qdim, c.hidden) || !shape_is(k, kvdim, c.hidden) || !shape_is(v, kvdim, c.hidden) ||
        !shape_is(o, c.hidden, qdim) || !shape_is(gate, lffn, c.hidden) || !shape_is(up, lffn, c.hidden) ||
        !shape_is(down, c.hidden, lffn))
        return fail(ctx, NNQ_ERR_SHAPE_MISMATCH, "projection shapes of layer %d do not match the configuration", layer);
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    nnq_decoder::Layer &L = d->layers[layer];
    L.q = q; L.k = k; L.v = v; L.o = o; L.gate = gate; L.up = up; L.down = down;
    s = check_cuda(ctx, cudaMemcpy(L.in_norm, in_norm, (size_t)c.hidden * 4, cudaMemcpyDefault), "norm weight");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemcpy(L.post_norm, post_norm, (size_t)c.hidden * 4, cudaMemcpyDefault), "norm weight");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemcpy(L.q_norm, q_norm, (size_t)c.head_dim * 4, cudaMemcpyDefault), "norm weight");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemcpy(L.k_norm, k_norm, (size_t)c.head_dim * 4, cudaMemcpyDefault), "norm weight");
    return s;
}

nnq_status nnq_decoder_set_head(nnq_decoder *d, const void *embed_bf16_dev, const float *final_norm, const nnq_weight *lm_head) {
    if (!d) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = d->ctx;
    if (!embed_bf16_dev || !final_norm) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL tensor");
    // tensor parallel: either the whole [vocab, hidden] projection on every rank, or this rank's
    // rows [rank * vocab / world, (rank + 1) * vocab / world) of it (vocabulary parallel: the ranks
    // then agree on the greedy token through the communicator)
    const nnq_decoder_config &c = d->cfg;
    if (shape_is(lm_head, c.vocab, c.hidden)) {
        d->head_rows = c.vocab;
        d->head_row0 = 0;
    } else if (c.tp_world > 1 && c.vocab % c.tp_world == 0 && shape_is(lm_head, c.vocab / c.tp_world, c.hidden)) {
        d->head_rows = c.vocab / c.tp_world;
        d->head_row0 = c.tp_rank * d->head_rows;
    } else {
        return fail(ctx, NNQ_ERR_SHAPE_MISMATCH, "vocabulary projection must be [vocab, hidden] (or this rank's [vocab / world, hidden] rows)");
    }
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    d->d_embed = embed_bf16_dev;
    d->lm_head = lm_head;
    d->ready = 1;
    return check_cuda(ctx, cudaMemcpy(d->d_final_norm, final_norm, (size_t)d->cfg.hidden * 4, cudaMemcpyDefault), "final norm");
}

nnq_status nnq_decoder_set_comm(nnq_decoder *d, nnq_comm *comm) {
    if (!d) return NNQ_ERR_INVALID_ARG;
    if (d->cfg.tp_world > 1 && !comm) return fail(d->ctx, NNQ_ERR_INVALID_ARG, "a tensor-parallel decoder needs a communicator");
    d->comm = comm;
    return NNQ_OK;
}

nnq_status nnq_decoder_reset(nnq_decoder *d, int token, int pos, void *stream) {
    if (!d) return NNQ_ERR_INVALID_ARG;
    if (token < 0 || token >= d->cfg.vocab || pos < 0 || pos >= d->cfg.max_seq) return fail(d->ctx, NNQ_ERR_INVALID_ARG, "token or position out of range");
    cudaSetDevice(d->ctx->device);
    const int st[4] = {token, pos, 0, 0};
    d->host_pos = pos;
    nnq_status s = check_cuda(d->ctx, cudaMemcpyAsync(d->d_state, st, sizeof(st), cudaMemcpyHostToDevice, (cudaStream_t)stream), "decoder state");
    if (s == NNQ_OK) s = check_cuda(d->ctx, cudaStreamSynchronize((cudaStream_t)stream), "decoder state");   // st is on the stack
    return s;
}

nnq_status nnq_decoder_buffers(nnq_decoder *d, float **k_cache, float **v_cache, float **logits, int **tokens) {
    if (!d) return NNQ_ERR_INVALID_ARG;
    if (k_cache) *k_cache = d->d_kcache;
    if (v_cache) *v_cache = d->d_vcache;
    if (logits) *logits = d->d_logits;
    if (tokens) *tokens = d->d_tokens;
    return NNQ_OK;
}

// Vocabulary projection of the normed state in d_xn, greedy argmax (exchanged between the ranks
// when the projection is split by rows), commit of the token and advance of the position.
static nnq_status launch_head(nnq_decoder *d, bool vocab_parallel, const CommView &cv, cudaStream_t st) {
    nnq_ctx *ctx = d->ctx;
    const nnq_decoder_config &c = d->cfg;
    nnq_status s;
    // the logits of this rank's rows land at their global offsets in the [vocab] buffer
    float *logits = d->d_logits + d->head_row0;
    if ((s = nnq_linear(ctx, d->lm_head, d->d_xn, (nnq_dtype)d->act_dt, 1, nullptr, logits, NNQ_F32, st)) != NNQ_OK) return s;
    float *bv = reinterpret_cast<float *>(d->d_state + 4);
    int *bi = d->d_state + 4 + kArgmaxBlocks;
    launch_pdl(dec_argmax_stage1_kernel, dim3(kArgmaxBlocks), dim3(256), st, logits, d->head_rows, bv, bi);
    if (vocab_parallel)
        launch_pdl(dec_argmax_exchange_kernel, dim3(1), dim3(32), st, bv, bi, kArgmaxBlocks, d->head_row0, cv.peer_table, cv.rank, cv.world,
                   cv.slot_bytes, d->d_state, d->d_tokens, c.max_seq, ctx->d_status);
    else
        launch_pdl(dec_argmax_stage2_kernel, dim3(1), dim3(32), st, bv, bi, kArgmaxBlocks, d->d_state, d->d_tokens, c.max_seq, ctx->d_status);
    ctx->launches += 2;
    return check_cuda(ctx, cudaGetLastError(), "decoder head launch");
}

static nnq_status head_mode(nnq_decoder *d, bool *vocab_parallel, CommView *cv) {
    const nnq_decoder_config &c = d->cfg;
    *vocab_parallel = d->head_rows != c.vocab;
    *cv = CommView{};
    if (*vocab_parallel) {
        nnq_status sv = comm_view(d->comm, cv);
        if (sv != NNQ_OK) return sv;
        if (cv->slot_bytes < (size_t)8 * c.hidden + 16)
            return fail(d->ctx, NNQ_ERR_UNSUPPORTED, "a vocabulary-parallel head needs communicator slots of at least 8 * hidden + 16 bytes (have %zu)", cv->slot_bytes);
    }
    return NNQ_OK;
}

// Measurement aid (builds with -DNNQ_DIAG only): NNQ_DEC_SKIP is a bit mask of step parts that are
// not launched (1 norms, 2 rotation / cache append, 4 attention, 16 SwiGLU, 32 products), to read
// the cost of each part off the time of a replayed step. The results are meaningless with any bit set.
#ifdef NNQ_DIAG
static int dec_skip() {
    static const int v = getenv("NNQ_DEC_SKIP") ? atoi(getenv("NNQ_DEC_SKIP")) : 0;
    return v;
}
#define DEC_RUN(bit, ...) do { if (!(dec_skip() & (bit))) { __VA_ARGS__; } } while (0)
#else
#define DEC_RUN(bit, ...) do { __VA_ARGS__; } while (0)
#endif

nnq_status nnq_decoder_step(nnq_decoder *d, void *stream) {
    if (!d) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = d->ctx;
    if (!d->ready) return fail(ctx, NNQ_ERR_INVALID_ARG, "decoder head has not been set");
    const nnq_decoder_config &c = d->cfg;
    if (c.tp_world > 1 && !d->comm) return fail(ctx, NNQ_ERR_INVALID_ARG, "communicator has not been set");
    for (int l = 0; l < c.n_layers; l++)
        if (!d->layers[l].q) return fail(ctx, NNQ_ERR_INVALID_ARG, "layer %d has not been set", l);
    // The caches hold max_seq positions and never grow (the reference's KvCacheLayer::append doubles
    // its buffer instead): a step past the last position is refused here, and -- for captured graphs
    // that the host does not see being replayed -- by the device-side flag behind nnq_device_status.
    if (d->host_pos >= c.max_seq)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "the decoder's context is full (max_seq = %d positions): reset it", c.max_seq);
    if (d->host_pos >= 0) d->host_pos++;
    bool vocab_parallel = false;
    CommView cv = {};
    nnq_status s = head_mode(d, &vocab_parallel, &cv);
    if (s != NNQ_OK) return s;
    s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    const int hd = c.head_dim, group = c.n_heads / c.n_kv_heads, lh = d->lh, lkv = d->lkv, lffn = c.ffn / c.tp_world;
    const nnq_dtype adt = (nnq_dtype)d->act_dt;
    const size_t layer_cache = (size_t)lkv * c.max_seq * hd;
    const float scale = (float)(1.0 / sqrt((double)hd));
    const __nv_bfloat16 *embed = (const __nv_bfloat16 *)d->d_embed;
    for (int l = 0; l < c.n_layers; l++) {
        const nnq_decoder::Layer &L = d->layers[l];
        DEC_RUN(1, launch_pdl(dec_norm_kernel, dim3(1), dim3(1024), st, d->d_h, d->d_delta, l == 0 ? embed : nullptr, d->d_state, L.in_norm, c.rms_eps, d->d_xn, d->act_dt, c.hidden));
        const nnq_weight *w3[3] = {L.q, L.k, L.v};
        const void *x3[3] = {d->d_xn, d->d_xn, d->d_xn};
        void *y3[3] = {d->d_q, d->d_k, d->d_v};
        DEC_RUN(32, if ((s = nnq_linear_batch(ctx, 3, w3, x3, adt, 1, nullptr, y3, NNQ_F32, st)) != NNQ_OK) return s);
        DEC_RUN(2, launch_pdl(dec_qk_rope_kernel, dim3(lh + 2 * lkv), dim3(hd), st, d->d_q, d->d_k, d->d_v, L.q_norm, L.k_norm, d->d_cos, d->d_sin, d->d_state,
                              c.rms_eps, d->d_qrot, d->d_kcache + l * layer_cache, d->d_vcache + l * layer_cache, lh, lkv, hd, c.max_seq));
        DEC_RUN(4, {
            const dim3 ag(lkv, kAttnRanges), ab(kAttnWarps * 32);
            const float *kc = d->d_kcache + l * layer_cache, *vc = d->d_vcache + l * layer_cache;
            switch (group) {
                case 1: launch_pdl(dec_attn_kernel<1>, ag, ab, st, d->d_qrot, kc, vc, d->d_state, scale, d->d_part, d->d_arrived, d->d_attn, d->act_dt, hd, c.max_seq); break;
                case 2: launch_pdl(dec_attn_kernel<2>, ag, ab, st, d->d_qrot, kc, vc, d->d_state, scale, d->d_part, d->d_arrived, d->d_attn, d->act_dt, hd, c.max_seq); break;
                case 4: launch_pdl(dec_attn_kernel<4>, ag, ab, st, d->d_qrot, kc, vc, d->d_state, scale, d->d_part, d->d_arrived, d->d_attn, d->act_dt, hd, c.max_seq); break;
                case 8: launch_pdl(dec_attn_kernel<8>, ag, ab, st, d->d_qrot, kc, vc, d->d_state, scale, d->d_part, d->d_arrived, d->d_attn, d->act_dt, hd, c.max_seq); break;
                default: return fail(ctx, NNQ_ERR_UNSUPPORTED, "query heads per key/value head must be 1, 2, 4 or 8");
            }
        });
        // row-parallel products: with tensor parallelism the partial sums are exchanged inside the kernel
        DEC_RUN(32, s = d->comm ? nnq_comm_linear(d->comm, L.o, d->d_attn, adt, 1, nullptr, d->d_delta, NNQ_F32, st)
                                : nnq_linear(ctx, L.o, d->d_attn, adt, 1, nullptr, d->d_delta, NNQ_F32, st));
        if (s != NNQ_OK) return s;
        DEC_RUN(1, launch_pdl(dec_norm_kernel, dim3(1), dim3(1024), st, d->d_h, d->d_delta, nullptr, d->d_state, L.post_norm, c.rms_eps, d->d_xn, d->act_dt, c.hidden));
        const nnq_weight *w2[2] = {L.gate, L.up};
        const void *x2[2] = {d->d_xn, d->d_xn};
        void *y2[2] = {d->d_g, d->d_u};
        DEC_RUN(32, if ((s = nnq_linear_batch(ctx, 2, w2, x2, adt, 1, nullptr, y2, NNQ_F32, st)) != NNQ_OK) return s);
        DEC_RUN(16, launch_pdl(dec_silu_mul_kernel, dim3((lffn + 255) / 256), dim3(256), st, d->d_g, d->d_u, d->d_mid, d->act_dt, lffn));
        DEC_RUN(32, s = d->comm ? nnq_comm_linear(d->comm, L.down, d->d_mid, adt, 1, nullptr, d->d_delta, NNQ_F32, st)
                                : nnq_linear(ctx, L.down, d->d_mid, adt, 1, nullptr, d->d_delta, NNQ_F32, st));
        if (s != NNQ_OK) return s;
        ctx->launches += 5;
    }
    launch_pdl(dec_norm_kernel, dim3(1), dim3(1024), st, d->d_h, d->d_delta, nullptr, d->d_state, d->d_final_norm, c.rms_eps, d->d_xn, d->act_dt, c.hidden);
    ctx->launches++;
    return launch_head(d, vocab_parallel, cv, st);
}

nnq_status nnq_decoder_prefill(nnq_decoder *d, const int32_t *tokens_host, int count, int start_pos, void *stream) {
    if (!d) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = d->ctx;
    const nnq_decoder_config &c = d->cfg;
    if (!d->ready) return fail(ctx, NNQ_ERR_INVALID_ARG, "decoder head has not been set");
    if (c.tp_world > 1 && !d->comm) return fail(ctx, NNQ_ERR_INVALID_ARG, "communicator has not been set");
    for (int l = 0; l < c.n_layers; l++)
        if (!d->layers[l].q) return fail(ctx, NNQ_ERR_INVALID_ARG, "layer %d has not been set", l);
    if (!tokens_host || count < 1 || start_pos < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad prompt arguments");
    if ((long long)start_pos + count > c.max_seq)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "a prompt of %d tokens at position %d does not fit max_seq = %d", count, start_pos, c.max_seq);
    for (int i = 0; i < count; i++)
        if (tokens_host[i] < 0 || tokens_host[i] >= c.vocab) return fail(ctx, NNQ_ERR_INVALID_ARG, "prompt token %d out of range", i);
    bool vocab_parallel = false;
    CommView cv = {};
    nnq_status s = head_mode(d, &vocab_parallel, &cv);
    if (s != NNQ_OK) return s;
    if ((s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice")) != NNQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    const int hd = c.head_dim, group = c.n_heads / c.n_kv_heads, lh = d->lh, lkv = d->lkv, lffn = c.ffn / c.tp_world;
    const int qdim = lh * hd, kvdim = lkv * hd;
    const nnq_dtype adt = (nnq_dtype)d->act_dt;
    const size_t es = adt == NNQ_F32 ? 4 : 2;
    // rows per pass: bounded by the scratch below and, with tensor parallelism, by what one exchange carries
    int rows_max = kPrefillRows;
    if (d->comm) {
        CommView v;
        if ((s = comm_view(d->comm, &v)) != NNQ_OK) return s;
        const size_t fit = v.slot_bytes / ((size_t)c.hidden * 4);
        if (fit < 1) return fail(ctx, NNQ_ERR_UNSUPPORTED, "communicator slots are smaller than one row of the hidden state");
        if ((size_t)rows_max > fit) rows_max = (int)fit;
    }
    if (!d->pf_h) {
        d->pf_rows = kPrefillRows;
        const size_t R = kPrefillRows;
        s = dev_alloc(ctx, (void **)&d->pf_h, R * c.hidden * 4, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->pf_delta, R * c.hidden * 4, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->pf_q, R * qdim * 4, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->pf_k, R * kvdim * 4, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->pf_v, R * kvdim * 4, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->pf_qrot, R * qdim * 4, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->pf_g, R * lffn * 4, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->pf_u, R * lffn * 4, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, &d->pf_xn, R * c.hidden * es, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, &d->pf_attn, R * qdim * es, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, &d->pf_mid, R * lffn * es, "prompt buffer");
        if (s == NNQ_OK) s = dev_alloc(ctx, (void **)&d->pf_tokens, R * 4, "prompt buffer");
        if (s != NNQ_OK) return s;
    }
    const size_t layer_cache = (size_t)lkv * c.max_seq * hd;
    const float scale = (float)(1.0 / sqrt((double)hd));
    const __nv_bfloat16 *embed = (const __nv_bfloat16 *)d->d_embed;
    int n = 0;
    for (int c0 = 0; c0 < count; c0 += n) {
        n = count - c0 < rows_max ? count - c0 : rows_max;
        const int pos0 = start_pos + c0;
        if ((s = check_cuda(ctx, cudaMemcpyAsync(d->pf_tokens, tokens_host + c0, (size_t)n * 4, cudaMemcpyHostToDevice, st), "prompt tokens")) != NNQ_OK) return s;
        for (int l = 0; l < c.n_layers; l++) {
            const nnq_decoder::Layer &L = d->layers[l];
            float *kc = d->d_kcache + l * layer_cache, *vc = d->d_vcache + l * layer_cache;
            dec_norm_rows_kernel<<<n, 256, 0, st>>>(d->pf_h, l == 0 ? nullptr : d->pf_delta, l == 0 ? embed : nullptr, d->pf_tokens, L.in_norm,
                                                    c.rms_eps, d->pf_xn, d->act_dt, c.hidden);
            const nnq_weight *w3[3] = {L.q, L.k, L.v};
            const void *x3[3] = {d->pf_xn, d->pf_xn, d->pf_xn};
            void *y3[3] = {d->pf_q, d->pf_k, d->pf_v};
            if ((s = nnq_linear_batch(ctx, 3, w3, x3, adt, n, nullptr, y3, NNQ_F32, st)) != NNQ_OK) return s;
            dec_qk_rope_rows_kernel<<<dim3(lh + 2 * lkv, n), hd, 0, st>>>(d->pf_q, d->pf_k, d->pf_v, L.q_norm, L.k_norm, d->d_cos, d->d_sin, pos0,
                                                                         c.rms_eps, d->pf_qrot, kc, vc, lh, lkv, hd, c.max_seq);
            // 16 query vectors per warp: R = 16 / G rows share each key / value row
            switch (group) {
                case 1: dec_attn_rows_kernel<1, 16><<<dim3(lkv, (n + 15) / 16), 32, 0, st>>>(d->pf_qrot, kc, vc, pos0, n, scale, d->pf_attn, d->act_dt, lh, hd, c.max_seq); break;
                case 2: dec_attn_rows_kernel<2, 8><<<dim3(lkv, (n + 7) / 8), 32, 0, st>>>(d->pf_qrot, kc, vc, pos0, n, scale, d->pf_attn, d->act_dt, lh, hd, c.max_seq); break;
                case 4: dec_attn_rows_kernel<4, 4><<<dim3(lkv, (n + 3) / 4), 32, 0, st>>>(d->pf_qrot, kc, vc, pos0, n, scale, d->pf_attn, d->act_dt, lh, hd, c.max_seq); break;
                case 8: dec_attn_rows_kernel<8, 2><<<dim3(lkv, (n + 1) / 2), 32, 0, st>>>(d->pf_qrot, kc, vc, pos0, n, scale, d->pf_attn, d->act_dt, lh, hd, c.max_seq); break;
                default: return fail(ctx, NNQ_ERR_UNSUPPORTED, "query heads per key/value head must be 1, 2, 4 or 8");
            }
            s = d->comm ? nnq_comm_linear(d->comm, L.o, d->pf_attn, adt, n, nullptr, d->pf_delta, NNQ_F32, st)
                        : nnq_linear(ctx, L.o, d->pf_attn, adt, n, nullptr, d->pf_delta, NNQ_F32, st);
            if (s != NNQ_OK) return s;
            dec_norm_rows_kernel<<<n, 256, 0, st>>>(d->pf_h, d->pf_delta, nullptr, d->pf_tokens, L.post_norm, c.rms_eps, d->pf_xn, d->act_dt, c.hidden);
            const nnq_weight *w2[2] = {L.gate, L.up};
            const void *x2[2] = {d->pf_xn, d->pf_xn};
            void *y2[2] = {d->pf_g, d->pf_u};
            if ((s = nnq_linear_batch(ctx, 2, w2, x2, adt, n, nullptr, y2, NNQ_F32, st)) != NNQ_OK) return s;
            const int total = n * lffn;
            dec_silu_mul_kernel<<<(total + 255) / 256, 256, 0, st>>>(d->pf_g, d->pf_u, d->pf_mid, d->act_dt, total);
            s = d->comm ? nnq_comm_linear(d->comm, L.down, d->pf_mid, adt, n, nullptr, d->pf_delta, NNQ_F32, st)
                        : nnq_linear(ctx, L.down, d->pf_mid, adt, n, nullptr, d->pf_delta, NNQ_F32, st);
            if (s != NNQ_OK) return s;
            ctx->launches += 5;
        }
    }
    // the last prompt token's state: final norm, vocabulary projection, greedy successor
    const size_t last = (size_t)(n - 1) * c.hidden;
    const int st4[4] = {tokens_host[count - 1], start_pos + count - 1, 0, 0};
    if ((s = check_cuda(ctx, cudaMemcpyAsync(d->d_state, st4, sizeof(st4), cudaMemcpyHostToDevice, st), "decoder state")) != NNQ_OK) return s;
    launch_pdl(dec_norm_kernel, dim3(1), dim3(1024), st, d->pf_h + last, d->pf_delta + last, nullptr, d->d_state, d->d_final_norm, c.rms_eps, d->d_xn, d->act_dt, c.hidden);
    ctx->launches++;
    if ((s = launch_head(d, vocab_parallel, cv, st)) != NNQ_OK) return s;
    d->host_pos = (long long)start_pos + count;
    return check_cuda(ctx, cudaStreamSynchronize(st), "prompt pass");   // tokens_host and st4 are the caller's / the stack's
}

nnq_status nnq_decoder_state(nnq_decoder *d, int *token, int *pos, int *steps, void *stream) {
    if (!d) return NNQ_ERR_INVALID_ARG;
    cudaSetDevice(d->ctx->device);
    int st[4] = {0, 0, 0, 0};
    nnq_status s = check_cuda(d->ctx, cudaMemcpyAsync(st, d->d_state, sizeof(st), cudaMemcpyDeviceToHost, (cudaStream_t)stream), "decoder state");
    if (s == NNQ_OK) s = check_cuda(d->ctx, cudaStreamSynchronize((cudaStream_t)stream), "decoder state");
    if (token) *token = st[0];
    if (pos) *pos = st[1];
    if (steps) *steps = st[2];
    return s;
}

void nnq_decoder_destroy(nnq_decoder *d) {
    if (!d) return;
    cudaSetDevice(d->ctx->device);
    cudaDeviceSynchronize();
    if (d->layers) {
        for (int l = 0; l < d->cfg.n_layers; l++) {
            cudaFree(d->layers[l].in_norm); cudaFree(d->layers[l].post_norm);
            cudaFree(d->layers[l].q_norm); cudaFree(d->layers[l].k_norm);
        }
        delete[] d->layers;
    }
    cudaFree(d->d_final_norm); cudaFree(d->d_cos); cudaFree(d->d_sin); cudaFree(d->d_kcache); cudaFree(d->d_vcache);
    cudaFree(d->d_h); cudaFree(d->d_delta); cudaFree(d->d_q); cudaFree(d->d_k); cudaFree(d->d_v); cudaFree(d->d_qrot);
    cudaFree(d->d_g); cudaFree(d->d_u); cudaFree(d->d_logits); cudaFree(d->d_part); cudaFree(d->d_arrived); cudaFree(d->d_xn); cudaFree(d->d_attn);
    cudaFree(d->d_mid); cudaFree(d->d_state); cudaFree(d->d_tokens);
    cudaFree(d->pf_h); cudaFree(d->pf_delta); cudaFree(d->pf_q); cudaFree(d->pf_k); cudaFree(d->pf_v); cudaFree(d->pf_qrot);
    cudaFree(d->pf_g); cudaFree(d->pf_u); cudaFree(d->pf_xn); cudaFree(d->pf_attn); cudaFree(d->pf_mid); cudaFree(d->pf_tokens);
    cudaGetLastError();
    delete d;
}

}  // extern "C"
