// Skinny (decode, M <= 16) streaming kernels for Q4_K weights on the tiled "T16" layout.
//
// Why tensor cores for a GEMV: at HBM speed an SM receives about 50 four-bit weights per
// clock, so there are fewer than three issue slots per weight for unpacking, converting,
// multiplying and adding. The kernel therefore builds fp16 operand registers straight
// from the packed nibbles with one logic op per two weights ((w & mask) | magic gives
// 1024+q or 64+q as fp16), lets mma.sync.m16n8k16 form the dot products with f32
// accumulation, and removes the constant offsets afterwards with per-sub-block sums of
// the activations. The products (q <= 15, x bf16 -> fp16) are exact; only the f32
// accumulation order differs from the CPU oracle.
//
// Sub-block scales: the eight n-columns of the MMA are used as eight *sub-blocks* of one
// 256-weight super-block. The activation operand is zero except in the column of the
// sub-block a k-slot belongs to, so after 16 MMAs the accumulator tile holds the 8
// per-sub-block dot products of 16 rows, and the 6-bit scales / mins are applied once
// per super-block, two sub-blocks per lane.
//
// Tiled layout (built once at weight creation, same byte count as the raw blocks):
//   tile(rt, kb) = 16 rows x one super-block = 2304 bytes at ((rt * KB + kb) * 2304)
//   [0, 256)     header: row r, word t (r*16 + t*4):
//                sc[2t] | sc[2t+1]<<6 | mn[2t]<<12 | mn[2t+1]<<18 | byte t of (d | dmin<<16) << 24
//   [256, 2304)  quants: region p (sub-blocks 2p, 2p+1), lane l = 4g + t, 16 bytes at
//                256 + 512p + 16l = words {(row g, sb 2p), (row g+8, sb 2p), (row g, sb 2p+1),
//                (row g+8, sb 2p+1)}, each word = elements 8t..8t+7 of that sub-block with
//                nibbles placed so that four logic ops yield the element pairs (0,1)..(6,7):
//                byte0 = e0 | e2<<4, byte1 = e4 | e6<<4, byte2 = e1 | e3<<4, byte3 = e5 | e7<<4
// Every global load of the main loop is a fully coalesced 512-byte warp access.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#include "decode.cuh"
#include "skinny.h"
#include "sync.cuh"

namespace nnq {

constexpr int kTileBytes = 2304;
constexpr int kWarps = 8;          // compute warps per CTA; they split K of one row tile
constexpr int kMaxStages = 4;      // bulk-copy ring depth per warp (tiles in flight)
constexpr int kSmemMax = 227 * 1024;         // one CTA per SM
constexpr int kMoeMaxExperts = 64;

struct SkinnyJobDev {
    const uint8_t *tiled;
    const float *bias;
    void *y;
    int n;              // real rows
    int row_tiles;      // ceil(n / 16)
    int tile_begin;     // first row tile of this job in the launch-wide numbering
};

struct SkinnyParams {
    SkinnyJobDev job[kSkinnyMaxJobs];
    const void *x;      // activations shared by all jobs, [K]
    int njobs;
    int m;              // tokens (1 for the M = 1 kernel, 2..16 for the token-column kernel)
    int y_dt;
    int kblocks;        // tiles along K (K / 256; K / 192 for six-block MXFP4 tiles)
    int total_tiles;    // row tiles of all jobs
    int stages;         // ring depth per warp
    int diag;           // diagnostics (NNQ_SKINNY_DIAG): bit 0 = skip the arithmetic (stream only),
                        // bit 1 = do not wait for the previous kernel; 4 = plain streaming read
    int l2_prefetch;    // 1 = ask L2 for the warp's whole weight stream at kernel start
    int *status;
    FusedReduce fr;     // row-parallel product + all-reduce in one kernel (M = 1 kernel, one job)
};

// ---------------------------------------------------------------------------------
// repack: raw Q4_K blocks (either element order) -> tiled layout
// ---------------------------------------------------------------------------------

template <bool GGML>
__global__ void repack_q4k_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ tiled, int n,
                                  int kblocks) {
    // one thread per (row, super-block, sub-block); sub-block 0's thread also writes the header
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)n * kblocks * 8;
    if (idx >= total) return;
    int sb = (int)(idx & 7);
    int64_t blk = idx >> 3;
    int kb = (int)(blk % kblocks);
    int row = (int)(blk / kblocks);
    const uint8_t *b = raw + blk * 144;
    uint8_t *tile = tiled + ((int64_t)(row >> 4) * kblocks + kb) * kTileBytes;
    int r16 = row & 15, g = row & 7, upper = (row >> 3) & 1;

    // the 32 four-bit codes of this sub-block in element order
    uint32_t e[32];
    if (!GGML) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            uint32_t q = b[16 + 16 * sb + i];
            e[2 * i] = q & 15u;
            e[2 * i + 1] = q >> 4;
        }
    } else {
        int sh = 4 * (sb & 1);
#pragma unroll
        for (int i = 0; i < 32; i++) e[i] = (b[16 + 32 * (sb >> 1) + i] >> sh) & 15u;
    }
    int p = sb >> 1, comp = (sb & 1) * 2 + upper;
#pragma unroll
    for (int v = 0; v < 4; v++) {
        const uint32_t *q = e + 8 * v;
        uint32_t word = (q[0] | (q[2] << 4)) | ((q[4] | (q[6] << 4)) << 8) | ((q[1] | (q[3] << 4)) << 16) |
                        ((q[5] | (q[7] << 4)) << 24);
        int lane = 4 * g + v;
        *reinterpret_cast<uint32_t *>(tile + 256 + 512 * p + 16 * lane + 4 * comp) = word;
    }
    if (sb < 4) {
        // header word t = sb: scales / mins of sub-blocks 2t, 2t+1 and byte t of (d, dmin)
        int t = sb;
        const uint8_t *S = b + 4;
        uint32_t sc[2], mn[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int j = 2 * t + h;
            if (!GGML) {
                sc[h] = ((S[j / 2] >> (4 * (j % 2))) & 15u) | (((S[8 + j / 4] >> (2 * (j % 4))) & 3u) << 4);
                mn[h] = ((S[4 + j / 2] >> (4 * (j % 2))) & 15u) | (((S[10 + j / 4] >> (2 * (j % 4))) & 3u) << 4);
            } else if (j < 4) {
                sc[h] = S[j] & 63u;
                mn[h] = S[j + 4] & 63u;
            } else {
                sc[h] = (S[j + 4] & 15u) | ((uint32_t)(S[j - 4] >> 6) << 4);
                mn[h] = (S[j + 4] >> 4) | ((uint32_t)(S[j] >> 6) << 4);
            }
        }
        uint32_t word = sc[0] | (sc[1] << 6) | (mn[0] << 12) | (mn[1] << 18) | ((uint32_t)b[t] << 24);
        *reinterpret_cast<uint32_t *>(tile + 16 * r16 + 4 * t) = word;
    }
}

// ---------------------------------------------------------------------------------
// M = 1 kernel
// ---------------------------------------------------------------------------------

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint2 b) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
}

// (a & b) | c in one LOP3 with all three operands in registers. The masks and magic
// numbers are kept in registers (see Consts) so that the instruction is never split.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

struct Consts {
    uint32_t mlo, mhi, k1024, k64;
    __device__ __forceinline__ void init() {
        // opaque moves: the values live in registers for the whole kernel
        asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(mlo));
        asm volatile("mov.b32 %0, 0x00F000F0;" : "=r"(mhi));
        asm volatile("mov.b32 %0, 0x64006400;" : "=r"(k1024));
        asm volatile("mov.b32 %0, 0x54005400;" : "=r"(k64));
    }
};

__device__ __forceinline__ uint32_t sel4(const uint4 &v, int t) {
    uint32_t lo = t & 1 ? v.y : v.x;
    uint32_t hi = t & 1 ? v.w : v.z;
    return t & 2 ? hi : lo;
}

// Shared memory of one CTA.
//   img: for every super-block of the k-chunk, the activation operand of its 16 MMAs exactly as
//        the lanes consume it: img[kb][mma = 4p + e][lane][2] (8 bytes per lane, LDS.64).
//        Word h of lane (g, t) in MMA (p, e) is the fp16 pair (2e, 2e+1) of word t of sub-block g
//        when g == 2p + h, and zero otherwise, so that column g of the accumulator tile
//        receives only sub-block g. The zero pattern is written once per CTA.
//   tab: per super-block and t a float4 (Ox[2t], Ox[2t+1], Sx[2t], Sx[2t+1]); Ox = sum of
//        offset * x over the sub-block (offset 1024 or 64 by element), Sx = sum of x.
// Shared memory of one CTA (dynamic):
//   ring   kWarps x stages x 2304 B      per-warp ring of weight tiles filled by bulk copies
//   xs     K x 4 B (x 2 for f32 inputs)  activations as the MMA operand, "half expanded":
//          for super-block kb, sub-block sb, word t (32 B at kb*1024 + (4 sb + t)*32):
//          8 words {b0,b1} x 4 element pairs, b_h = fp16 pair when h == sb & 1, else 0
//   tab    K/256 x 4 x float4            (Ox[2t], Ox[2t+1], Sx[2t], Sx[2t+1]) per super-block, t
//   xinv   K/256 floats                  1 / prescale of each super-block's activations
//   part   2 x kWarps x 16 floats        per-warp partial sums of a row tile, double buffered
//   bars: kWarps x stages ring barriers + full[2] + empty[2]
struct SmemPlan {
    int ring_off, xs_off, xs_lo_off, tab_off, xinv_off, part_off, bar_off, total;
};

__host__ __device__ inline SmemPlan smem_plan(int kblocks, int stages, bool f32x) {
    SmemPlan p;
    p.ring_off = 0;
    p.xs_off = kWarps * stages * kTileBytes;
    p.xs_lo_off = p.xs_off + kblocks * 1024;
    p.tab_off = p.xs_lo_off + (f32x ? kblocks * 1024 : 0);
    p.xinv_off = p.tab_off + kblocks * 64;
    p.part_off = (p.xinv_off + kblocks * 4 + 15) & ~15;
    p.bar_off = p.part_off + 2 * kWarps * 16 * 4;
    p.total = p.bar_off + (kWarps * kMaxStages + 4) * 8;
    return p;
}

// predicated 32-byte shared load (two 16-byte halves): the registers keep their value where the
// predicate is false
__device__ __forceinline__ void lds256_if(uint4 &a, uint4 &b, uint32_t addr, int pred) {
    asm volatile(
        "{\n .reg .pred q;\n setp.ne.s32 q, %8, 0;\n @q ld.shared.v4.u32 {%0,%1,%2,%3}, [%9];\n"
        " @q ld.shared.v4.u32 {%4,%5,%6,%7}, [%9+16];\n}"
        : "+r"(a.x), "+r"(a.y), "+r"(a.z), "+r"(a.w), "+r"(b.x), "+r"(b.y), "+r"(b.z), "+r"(b.w)
        : "r"(pred), "r"(addr));
}

struct BRegs {
    uint4 v[4][2];  // [p][pairs 0-1 | pairs 2-3] = {b0, b1, b0', b1'}: non-zero only for p == g / 2
};

template <bool F32X>
__device__ __forceinline__ void tile_mac(const uint8_t *stage, uint32_t xs_s, uint32_t xs_lo_s, const float *tab,
                                         float inv, int lane, int g, int t, const Consts &K, BRegs &B, BRegs &BL,
                                         float &yg, float &yg8) {
    const uint4 *st = reinterpret_cast<const uint4 *>(stage);
    // activation operand of this super-block: only the lanes whose column g is a sub-block of
    // pair p load data for p; every other register of B stays zero for the whole kernel
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const int mine = (g >> 1) == p;
        lds256_if(B.v[p][0], B.v[p][1], xs_s, mine);
        if (F32X) lds256_if(BL.v[p][0], BL.v[p][1], xs_lo_s, mine);
    }
    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float c2[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // second accumulator chain: halves the MMA dependency depth
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const uint4 q = st[16 + 32 * p + lane];
        const uint32_t w0 = q.x, w1 = q.y, w2 = q.z, w3 = q.w;
        const uint32_t v0 = w0 >> 8, v1 = w1 >> 8, v2 = w2 >> 8, v3 = w3 >> 8;
        mma_f16(c, and_or(w0, K.mlo, K.k1024), and_or(w1, K.mlo, K.k1024), and_or(w2, K.mlo, K.k1024),
                and_or(w3, K.mlo, K.k1024), make_uint2(B.v[p][0].x, B.v[p][0].y));
        mma_f16(c2, and_or(w0, K.mhi, K.k64), and_or(w1, K.mhi, K.k64), and_or(w2, K.mhi, K.k64),
                and_or(w3, K.mhi, K.k64), make_uint2(B.v[p][0].z, B.v[p][0].w));
        mma_f16(c, and_or(v0, K.mlo, K.k1024), and_or(v1, K.mlo, K.k1024), and_or(v2, K.mlo, K.k1024),
                and_or(v3, K.mlo, K.k1024), make_uint2(B.v[p][1].x, B.v[p][1].y));
        mma_f16(c2, and_or(v0, K.mhi, K.k64), and_or(v1, K.mhi, K.k64), and_or(v2, K.mhi, K.k64),
                and_or(v3, K.mhi, K.k64), make_uint2(B.v[p][1].z, B.v[p][1].w));
        if (F32X) {
            mma_f16(c, and_or(w0, K.mlo, K.k1024), and_or(w1, K.mlo, K.k1024), and_or(w2, K.mlo, K.k1024),
                    and_or(w3, K.mlo, K.k1024), make_uint2(BL.v[p][0].x, BL.v[p][0].y));
            mma_f16(c2, and_or(w0, K.mhi, K.k64), and_or(w1, K.mhi, K.k64), and_or(w2, K.mhi, K.k64),
                    and_or(w3, K.mhi, K.k64), make_uint2(BL.v[p][0].z, BL.v[p][0].w));
            mma_f16(c, and_or(v0, K.mlo, K.k1024), and_or(v1, K.mlo, K.k1024), and_or(v2, K.mlo, K.k1024),
                    and_or(v3, K.mlo, K.k1024), make_uint2(BL.v[p][1].x, BL.v[p][1].y));
            mma_f16(c2, and_or(v0, K.mhi, K.k64), and_or(v1, K.mhi, K.k64), and_or(v2, K.mhi, K.k64),
                    and_or(v3, K.mhi, K.k64), make_uint2(BL.v[p][1].z, BL.v[p][1].w));
        }
    }
    // c[0], c[1]: row g, sub-blocks 2t, 2t+1; c[2], c[3]: row g+8
    const float4 tb = *reinterpret_cast<const float4 *>(tab + t * 4);
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint4 hd = st[8 * h + g];
        uint32_t p01 = __byte_perm(hd.x, hd.y, 0x0073);
        uint32_t p23 = __byte_perm(hd.z, hd.w, 0x0073);
        uint32_t dd = __byte_perm(p01, p23, 0x5410);
        float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&dd));
        uint32_t o = reinterpret_cast<const uint32_t *>(stage)[(8 * h + g) * 4 + t];
        float sc0 = (float)(o & 63u), sc1 = (float)((o >> 6) & 63u);
        float mn0 = (float)((o >> 12) & 63u), mn1 = (float)((o >> 18) & 63u);
        float dot = sc0 * ((c[2 * h] + c2[2 * h]) - tb.x) + sc1 * ((c[2 * h + 1] + c2[2 * h + 1]) - tb.y);
        float mins = mn0 * tb.z + mn1 * tb.w;
        float v = dm.x * dot - dm.y * mins;
        if (h) yg8 = fmaf(v, inv, yg8); else yg = fmaf(v, inv, yg);
    }
}

// Stage the activations of super-blocks kb_begin, kb_begin + kb_step, ... < kb_end; one warp per
// super-block, 8 consecutive elements (one word of one sub-block) per lane. Every super-block gets
// its own power-of-two prescale to fp16 (its largest |x| lands in [1, 2): exact, and fp16 stays in
// range whatever the magnitude of x), so that a warp can stage its own part of K without waiting
// for the rest of the CTA. Writes the half-expanded operand, the per-sub-block offset sums and
// 1 / prescale.
template <bool F32X>
__device__ __forceinline__ void stage_x_warp(const void *x, int kb_begin, int kb_end, int kb_step, uint8_t *xs,
                                             uint8_t *xs_lo, float *tab, float *xinv, int lane) {
    const int sb8 = lane >> 2;
    const bool odd = sb8 & 1;
#pragma unroll 2
    for (int kb = kb_begin; kb < kb_end; kb += kb_step) {
        float xv[8];
        const int i = kb * 256 + lane * 8;
        if (F32X) {
            const float4 *px = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + i);
            float4 a = __ldg(px), b = __ldg(px + 1);
            xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w;
            xv[4] = b.x; xv[5] = b.y; xv[6] = b.z; xv[7] = b.w;
        } else {
            uint4 v = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(x) + i));
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                xv[2 * k] = __uint_as_float(u[k] << 16);
                xv[2 * k + 1] = __uint_as_float(u[k] & 0xFFFF0000u);
            }
        }
        float amax = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; k++) amax = fmaxf(amax, fabsf(xv[k]));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
        uint32_t ex = (__float_as_uint(amax) >> 23) & 0xFFu;
        ex = amax > 0.0f && ex < 255u ? min(max(ex, 1u), 253u) : 127u;
        const float scale = __uint_as_float((254u - ex) << 23);
        uint32_t ph[4], pl[4];
        float xr[8];  // the values the MMAs will see
#pragma unroll
        for (int k = 0; k < 4; k++) {
            float s0 = xv[2 * k] * scale, s1 = xv[2 * k + 1] * scale;
            __half h0 = __float2half_rn(s0), h1 = __float2half_rn(s1);
            xr[2 * k] = __half2float(h0);
            xr[2 * k + 1] = __half2float(h1);
            ph[k] = __half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
            if (F32X) {
                __half l0 = __float2half_rn(s0 - xr[2 * k]), l1 = __float2half_rn(s1 - xr[2 * k + 1]);
                xr[2 * k] += __half2float(l0);
                xr[2 * k + 1] += __half2float(l1);
                pl[k] = __half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
            }
        }
        // lane = 4 * sub-block + word: its 32 bytes of the operand image are contiguous
        uint4 *dst = reinterpret_cast<uint4 *>(xs + kb * 1024 + lane * 32);
        dst[0] = odd ? make_uint4(0, ph[0], 0, ph[1]) : make_uint4(ph[0], 0, ph[1], 0);
        dst[1] = odd ? make_uint4(0, ph[2], 0, ph[3]) : make_uint4(ph[2], 0, ph[3], 0);
        if (F32X) {
            uint4 *dl = reinterpret_cast<uint4 *>(xs_lo + kb * 1024 + lane * 32);
            dl[0] = odd ? make_uint4(0, pl[0], 0, pl[1]) : make_uint4(pl[0], 0, pl[1], 0);
            dl[1] = odd ? make_uint4(0, pl[2], 0, pl[3]) : make_uint4(pl[2], 0, pl[3], 0);
        }
        // within a word (8 elements), elements 0,1,4,5 carry offset 1024 and 2,3,6,7 offset 64
        float sa = (xr[0] + xr[1]) + (xr[4] + xr[5]), sb = (xr[2] + xr[3]) + (xr[6] + xr[7]);
        float ox = 1024.0f * sa + 64.0f * sb;
        float sx = sa + sb;
#pragma unroll
        for (int o2 = 1; o2 < 4; o2 <<= 1) {  // the 4 lanes of one sub-block are consecutive
            ox += __shfl_xor_sync(0xFFFFFFFFu, ox, o2);
            sx += __shfl_xor_sync(0xFFFFFFFFu, sx, o2);
        }
        if ((lane & 3) == 0) {
            float *e = tab + (kb * 4 + (sb8 >> 1)) * 4 + (sb8 & 1);
            e[0] = ox;
            e[2] = sx;
        }
        if (lane == 0) xinv[kb] = __uint_as_float(ex << 23);
    }
}

// expect-tx + bulk copy issued by the lanes whose predicate is set (lane 0), without a branch
__device__ __forceinline__ void issue_tile(uint32_t dst, const void *src, uint32_t bar, int pred) {
    asm volatile(
        "{\n .reg .pred q;\n setp.ne.s32 q, %3, 0;\n"
        " @q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%2], 2304;\n"
        " @q cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 2304, [%2];\n}"
        ::"r"(dst), "l"(src), "r"(bar), "r"(pred) : "memory");
}

// Persistent kernel. A unit is RG = 8 / KS consecutive row tiles; CTA c handles units c, c + grid,
// ... (row tiles numbered across all jobs of the launch). Warp w works on row tile w / KS of the
// unit and on the (w % KS)-th part of K, streaming its tiles through a private ring of bulk
// copies; with KS > 1 the partial sums of a row tile meet in shared memory and one of the KS
// warps (in turn) writes the 16 outputs while the others already work on the next unit.
template <bool F32X, int KS, bool FUSED = false>
__global__ void __launch_bounds__(kWarps * 32, 2)
skinny_q4k_m1_kernel(const __grid_constant__ SkinnyParams P) {
    constexpr int RG = kWarps / KS;
    extern __shared__ __align__(128) uint8_t smem[];
    const SmemPlan L = smem_plan(P.kblocks, P.stages, F32X);
    uint8_t *xs = smem + L.xs_off;
    uint8_t *xs_lo = smem + L.xs_lo_off;
    float *tab = reinterpret_cast<float *>(smem + L.tab_off);
    float *xinv = reinterpret_cast<float *>(smem + L.xinv_off);
    float *part = reinterpret_cast<float *>(smem + L.part_off);

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);   // tells the compiler it is warp-uniform
    const int g = lane >> 2, t = lane & 3;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int stages = P.stages;
    const int ks = warp % KS, rsub = warp / KS;
    uint8_t *ring = smem + warp * stages * kTileBytes;
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t bars_s = smem_u32(smem + L.bar_off);
    const uint32_t bar_s = bars_s + warp * kMaxStages * 8;
    const uint32_t full_s = bars_s + kWarps * kMaxStages * 8;   // full[2], then empty[2]
    const uint32_t empty_s = full_s + 16;

    if (tid == 0) {
        mbar_init(full_s, kWarps);
        mbar_init(full_s + 8, kWarps);
        mbar_init(empty_s, RG);
        mbar_init(empty_s + 8, RG);
    }
    if (lane == 0) {
        for (int d = 0; d < stages; d++) mbar_init(bar_s + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // this warp's share of K and of the units
    const int kb_lo = (ks * P.kblocks) / KS, kb_hi = ((ks + 1) * P.kblocks) / KS;
    const int nkb = kb_hi - kb_lo;
    const int total_units = (P.total_tiles + RG - 1) / RG;
    const int n_units = cta < total_units ? (total_units - cta + grid - 1) / grid : 0;

    // job and row tile of this warp in a unit; j < 0 when the unit has no row tile for the warp
    auto locate = [&](int unit, int &j, int &rt) {
        int gt = (cta + unit * grid) * RG + rsub;
        j = -1;
        rt = 0;
        if (gt < P.total_tiles) {
            j = 0;
#pragma unroll
            for (int i = 1; i < kSkinnyMaxJobs; i++)
                if (i < P.njobs && gt >= P.job[i].tile_begin) j = i;
            rt = gt - P.job[j].tile_begin;
        }
    };

    // ---- weights first: they do not depend on anything an earlier kernel produced ----
    int pf_unit = -1, pf_k = 0, pf_slot = 0;
    unsigned issued = 0;
    const uint8_t *pf_src = nullptr;
    bool pf_done = nkb == 0;
    auto pf_advance_unit = [&]() {   // next unit in which this warp has a row tile
        for (;;) {
            if (++pf_unit >= n_units) {
                pf_done = true;
                return;
            }
            int j, rt;
            locate(pf_unit, j, rt);
            if (j >= 0) {
                pf_src = P.job[j].tiled + ((size_t)rt * P.kblocks + kb_lo) * kTileBytes;
                pf_k = 0;
                return;
            }
        }
    };
    // Ask L2 for this warp's whole weight stream right away: HBM then runs ahead of the ring and
    // keeps streaming while the CTA waits for its activations and for the previous kernel to drain.
    if (P.l2_prefetch && nkb > 0 && lane == 0) {
        for (int u = 0; u < n_units; u++) {
            int j, rt;
            locate(u, j, rt);
            if (j >= 0) {
                const uint8_t *src = P.job[j].tiled + ((size_t)rt * P.kblocks + kb_lo) * kTileBytes;
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(nkb * kTileBytes) : "memory");
            }
        }
    }
    if (!pf_done) pf_advance_unit();
    const int is_lane0 = lane == 0;
    auto issue = [&]() {
        if (!pf_done) {
            issue_tile(ring_s + pf_slot * kTileBytes, pf_src, bar_s + 8 * pf_slot, is_lane0);
            issued++;
            pf_slot = pf_slot + 1 == stages ? 0 : pf_slot + 1;
            pf_src += kTileBytes;
            if (++pf_k == nkb) pf_advance_unit();
        }
    };
    for (int d = 0; d < stages; d++) issue();

    // let the next kernel in the stream start its own weight prefetch; wait for the previous
    // one before touching activations
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!(P.diag & 2)) asm volatile("griddepcontrol.wait;" ::: "memory");
    // fused all-reduce: the exchange this launch takes part in (the epoch word is written by the
    // previous exchange, which the wait above has seen complete)
    unsigned ar_seq = 0;
    if (FUSED) ar_seq = *reinterpret_cast<volatile unsigned *>(P.fr.peers[P.fr.rank]) + 1u;

    if (KS == kWarps) {
        // the warp owns its part of K: no other warp reads what it stages
        stage_x_warp<F32X>(P.x, kb_lo, kb_hi, 1, xs, xs_lo, tab, xinv, lane);
        __syncwarp();
    } else {
        stage_x_warp<F32X>(P.x, warp, P.kblocks, kWarps, xs, xs_lo, tab, xinv, lane);
        __syncthreads();
    }
    const uint32_t xs_s = smem_u32(xs) + lane * 32, xs_lo_s = smem_u32(xs_lo) + lane * 32;

    Consts K;
    K.init();
    BRegs B, BL;
#pragma unroll
    for (int p = 0; p < 4; p++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            B.v[p][h] = make_uint4(0, 0, 0, 0);
            BL.v[p][h] = make_uint4(0, 0, 0, 0);
        }
    unsigned consumed = 0;
    int slot = 0;
    uint32_t phase = 0;
    bool failed = false;

    auto store16 = [&](int j, int rt, float v) {   // lanes 0..15 hold the 16 outputs of a row tile
        const SkinnyJobDev &J = P.job[j];
        int row = rt * 16 + lane;
        if (FUSED) {
            // Exchange without fences: every partial sum travels as one 8-byte store (value, sequence
            // number) into this rank's slot on each peer; the same lane then waits (bounded) for the
            // peers' pairs of this row and adds them in rank order, so every rank gets the same bits.
            if (lane < 16 && row < J.n) {
                const int par = (int)(ar_seq & 1u);
                const size_t mine = comm_data_offset(par, P.fr.rank, P.fr.world, P.fr.slot_bytes) + (size_t)row * 8;
                for (int p = 0; p < P.fr.world; p++)
                    if (p != P.fr.rank)
                        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(P.fr.peers[p] + mine),
                                     "r"(__float_as_uint(v)), "r"(ar_seq) : "memory");
                const uint8_t *local = P.fr.peers[P.fr.rank];
                float acc = 0.0f;
                bool ok = true;
                for (int r = 0; r < P.fr.world; r++) {
                    if (r == P.fr.rank) {
                        acc += v;
                        continue;
                    }
                    const uint8_t *src = local + comm_data_offset(par, r, P.fr.world, P.fr.slot_bytes) + (size_t)row * 8;
                    uint32_t bits = 0, tag = 0;
                    unsigned spins = 0;
                    do {
                        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(bits), "=r"(tag) : "l"(src) : "memory");
                    } while (tag != ar_seq && ++spins <= kCommSpins);
                    ok = ok && tag == ar_seq;
                    acc += __uint_as_float(bits);
                }
                if (!ok) atomicExch(P.status, 1);
                if (J.bias) acc += __ldg(J.bias + row);
                if (P.y_dt == NNQ_F32) reinterpret_cast<float *>(J.y)[row] = acc;
                else reinterpret_cast<__nv_bfloat16 *>(J.y)[row] = __float2bfloat16_rn(acc);
            }
            return;
        }
        if (lane < 16 && row < J.n) {
            if (J.bias) v += __ldg(J.bias + row);
            if (P.y_dt == NNQ_F32) reinterpret_cast<float *>(J.y)[row] = v;
            else reinterpret_cast<__nv_bfloat16 *>(J.y)[row] = __float2bfloat16_rn(v);
        }
    };

    // KS > 1: the warp whose turn it is adds the KS partial sums of its row tile and writes it out
    auto finish = [&](int unit) {
        const int b = unit & 1;
        if (!mbar_wait_fast(full_s + 8 * b, (unit >> 1) & 1u)) {
            failed = true;
            return;
        }
        int j, rt;
        locate(unit, j, rt);
        if (j >= 0) {
            float v = 0.0f;
            if (lane < 16) {
#pragma unroll
                for (int w = 0; w < KS; w++) v += part[(b * kWarps + rsub * KS + w) * 16 + lane];
            }
            store16(j, rt, v);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_s + 8 * b);
    };

#pragma unroll 1
    for (int unit = 0; unit < n_units && !failed; unit++) {
        int j, rt;
        locate(unit, j, rt);
        float yg = 0.0f, yg8 = 0.0f;
        if (j >= 0) {
            bool ok = true;
#pragma unroll 1
            for (int k = 0; k < nkb; k++) {
                ok &= mbar_wait_fast(bar_s + 8 * slot, phase);
                if (!(P.diag & 1))
                    tile_mac<F32X>(ring + slot * kTileBytes, xs_s + (kb_lo + k) * 1024, xs_lo_s + (kb_lo + k) * 1024,
                                   tab + (kb_lo + k) * 16, xinv[kb_lo + k], lane, g, t, K, B, BL, yg, yg8);
                consumed++;
                if (++slot == stages) {
                    slot = 0;
                    phase ^= 1u;
                }
                __syncwarp();  // all lanes have read the slot before it is refilled
                issue();
            }
            if (!ok) {   // a wait ran out: the sums are meaningless, stop here
                failed = true;
                break;
            }
            yg += __shfl_xor_sync(0xFFFFFFFFu, yg, 1);
            yg8 += __shfl_xor_sync(0xFFFFFFFFu, yg8, 1);
            yg += __shfl_xor_sync(0xFFFFFFFFu, yg, 2);
            yg8 += __shfl_xor_sync(0xFFFFFFFFu, yg8, 2);
        }
        if (KS == 1) {
            // no K split: lanes with t == 0 hold finished rows g and g + 8; gather them into lanes 0..15
            if (j >= 0) {
                float lo = __shfl_sync(0xFFFFFFFFu, yg, (lane & 7) * 4);
                float hi = __shfl_sync(0xFFFFFFFFu, yg8, (lane & 7) * 4);
                store16(j, rt, lane < 8 ? lo : hi);
            }
            continue;
        }
        const int b = unit & 1;
        // the partial-sum slot is free once the unit two back has been written out
        if (unit >= 2 && !mbar_wait_fast(empty_s + 8 * b, ((unit >> 1) - 1) & 1u)) {
            failed = true;
            break;
        }
        if (t == 0) {
            part[(b * kWarps + warp) * 16 + g] = yg;
            part[(b * kWarps + warp) * 16 + 8 + g] = yg8;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(full_s + 8 * b);
        // the previous unit's partial sums are long complete: write it out (one warp per row tile)
        if (unit >= 1 && ks == (unit - 1) % KS) finish(unit - 1);
    }
    if (KS > 1 && !failed && n_units >= 1 && ks == (n_units - 1) % KS) finish(n_units - 1);
    if (failed) {
        // record the failure, then give this warp's copies still in flight a bounded chance to
        // land before the CTA's shared memory goes away
        if (lane == 0) atomicExch(P.status, 1);
        for (unsigned n = consumed; n < issued; n++) {
            mbar_wait(bar_s + 8 * slot, phase);
            if (++slot == stages) {
                slot = 0;
                phase ^= 1u;
            }
        }
    }
    if (FUSED) {
        // the last CTA of this launch to finish advances the communicator's sequence number
        __syncthreads();
        if (tid == 0) {
            uint8_t *local = P.fr.peers[P.fr.rank];
            unsigned *arrived = reinterpret_cast<unsigned *>(local + 128);
            if (atomicAdd(arrived, 1u) == gridDim.x - 1) {
                *arrived = 0;
                *reinterpret_cast<volatile unsigned *>(local) = ar_seq;
            }
        }
    }
}

// ---------------------------------------------------------------------------------
// Token-column kernel: 1 <= M <= 16, the n-columns of the MMA are tokens
// ---------------------------------------------------------------------------------
//
// Same kind of tiles (16 rows x 256 weights, one bulk copy each), per-warp rings and K split over
// the 8 warps of a CTA as the M = 1 kernel, but the eight MMA columns are eight tokens (NT = 2:
// sixteen) and the activations are used as they are: bf16 pairs loaded straight from global
// memory (L1 / L2 resident) as the B operand (f32 activations are split into two bf16 terms on
// the fly and cost a second MMA). The weights enter as exact bf16 codes built with one logic op
// per two weights:
//   four-bit plane   (w & 0x000F000F) | 0x4300 = 128 + nibble
//   upper plane      (w & mask)       | 0x4500 = 2048 + 16 * field   (same accumulator)
// and a second MMA with an all-ones A operand yields the activation sum s of the group, which
// removes the constant offsets (and carries the Q4_K min term). Scales are applied per scale
// group on the f32 accumulators:
//   Q4_K  y += (d sc) * c - (128 d sc + dmin m) * s        group = sub-block of 32
//   Q8_0  y += d * (c - 2304 s)                            group = block of 32, code = q + 128
//   Q6_K  y += (d sc) * (c - 2208 s)                       group = 16 weights, code = q6
// Tiled layouts of Q8_0 and Q6_K (same byte count as the raw blocks; lane l = 4g + t owns rows g
// and g + 8 of the tile; a "T16 word" packs eight four-bit fields e0..e7 as byte0 = e0 | e2<<4,
// byte1 = e4 | e6<<4, byte2 = e1 | e3<<4, byte3 = e5 | e7<<4, so that (w >> 4i) & 0x000F000F is
// the pair (e_2i, e_2i+1)):
//   Q8_0, 4352 B: [0,256) fp16 d[row][block]; then per block b 512 B, lane l 16 B =
//         {low nibbles row g, high nibbles row g, low row g+8, high row g+8} of elements 8t..8t+7
//   Q6_K, 3360 B: [0,256) int8 sc[row][16]; [256,288) fp16 d[row]; then per sub-block 384 B =
//         128 B low-nibble words row g | 128 B row g+8 | 128 B two-bit words, one word per lane.
//         Lane t owns elements 4t..4t+3 (scale group 2sb) and 16+4t..16+4t+3 (group 2sb+1) as
//         e0..e7; two-bit word: row g pair i at bits 2i (e_2i) and 16+2i (e_2i+1), row g+8 at
//         bits 8+2i and 24+2i.

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// eight activations of one token as four bf16 pairs (and the bf16 remainder when they are f32)
template <bool F32X>
struct XB {
    uint4 hi, lo;
};

__device__ __forceinline__ void split_bf16(float a, float b, uint32_t &hi, uint32_t &lo) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    float2 hf = __bfloat1622float2(h);
    __nv_bfloat162 l = __floats2bfloat162_rn(a - hf.x, b - hf.y);
    hi = *reinterpret_cast<uint32_t *>(&h);
    lo = *reinterpret_cast<uint32_t *>(&l);
}

// elements [e0, e0+4) and [e1, e1+4) of the token row x (element offsets)
template <bool F32X>
__device__ __forceinline__ XB<F32X> load_xb(const void *x, int e0, int e1) {
    XB<F32X> r;
    if (F32X) {
        const float *p = reinterpret_cast<const float *>(x);
        const float4 u = __ldg(reinterpret_cast<const float4 *>(p + e0));
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p + e1));
        split_bf16(u.x, u.y, r.hi.x, r.lo.x);
        split_bf16(u.z, u.w, r.hi.y, r.lo.y);
        split_bf16(v.x, v.y, r.hi.z, r.lo.z);
        split_bf16(v.z, v.w, r.hi.w, r.lo.w);
    } else {
        const __nv_bfloat16 *p = reinterpret_cast<const __nv_bfloat16 *>(x);
        if (e1 == e0 + 4) {
            r.hi = __ldg(reinterpret_cast<const uint4 *>(p + e0));
        } else {
            const uint2 u = __ldg(reinterpret_cast<const uint2 *>(p + e0));
            const uint2 v = __ldg(reinterpret_cast<const uint2 *>(p + e1));
            r.hi = make_uint4(u.x, u.y, v.x, v.y);
        }
        r.lo = make_uint4(0, 0, 0, 0);
    }
    return r;
}

// d = A * B(pairs 2h, 2h+1 of xb) + c, with the remainder term of f32 activations
template <bool F32X>
__device__ __forceinline__ void mma_x(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                      const XB<F32X> &xb, int h, const float (&c)[4]) {
    mma_bf16(d, a0, a1, a2, a3, h ? xb.hi.z : xb.hi.x, h ? xb.hi.w : xb.hi.y, c);
    if (F32X) mma_bf16(d, a0, a1, a2, a3, h ? xb.lo.z : xb.lo.x, h ? xb.lo.w : xb.lo.y, d);
}

struct MnConsts {
    uint32_t m4, m2, k128, k2048, ones;
    uint32_t tl0, tl1, th0, th1;   // E2M1 magnitude -> bf16 low / high byte tables
    __device__ __forceinline__ void init() {
        asm volatile("mov.b32 %0, 0xC0800000;" : "=r"(tl0));
        asm volatile("mov.b32 %0, 0xC0804000;" : "=r"(tl1));
        asm volatile("mov.b32 %0, 0x3F3F3F00;" : "=r"(th0));
        asm volatile("mov.b32 %0, 0x40404040;" : "=r"(th1));
        asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(m4));
        asm volatile("mov.b32 %0, 0x00030003;" : "=r"(m2));
        asm volatile("mov.b32 %0, 0x43004300;" : "=r"(k128));
        asm volatile("mov.b32 %0, 0x45004500;" : "=r"(k2048));
        asm volatile("mov.b32 %0, 0x3F803F80;" : "=r"(ones));
    }
};

template <int FMT, int SB = 8>
struct TileFmt;   // SB = sub-blocks of 32 weights per tile row

// ---- Q4_K (both element orders share the tiled layout) ----
template <>
struct TileFmt<NNQ_Q4_K, 8> {
    static constexpr int kBytes = 2304;
    static constexpr int kElems = 256;
    template <int NT, bool F32X>
    static __device__ __forceinline__ void tile(const uint8_t *stage, float4 *sct4, const uint8_t *const (&xrow)[NT],
                                                int koff, int lane, int g, int t, const MnConsts &K,
                                                float (&y)[NT][4]) {
        constexpr int ES = F32X ? 4 : 2;
        const uint4 *st = reinterpret_cast<const uint4 *>(stage);
        const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        // (d sc, 128 d sc + dmin m) of the tile: this lane's share (rows g, g+8; sub-blocks 2t, 2t+1)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint4 hd = st[8 * h + g];
            uint32_t p01 = __byte_perm(hd.x, hd.y, 0x0073);
            uint32_t p23 = __byte_perm(hd.z, hd.w, 0x0073);
            uint32_t dd = __byte_perm(p01, p23, 0x5410);
            float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&dd));
            uint32_t o = reinterpret_cast<const uint32_t *>(stage)[(8 * h + g) * 4 + t];
            float sc0 = (float)(o & 63u), sc1 = (float)((o >> 6) & 63u);
            float mn0 = (float)((o >> 12) & 63u), mn1 = (float)((o >> 18) & 63u);
            float a0 = dm.x * sc0, a1 = dm.x * sc1;
            sct4[(8 * h + g) * 4 + t] = make_float4(a0, fmaf(128.0f, a0, dm.y * mn0), a1, fmaf(128.0f, a1, dm.y * mn1));
        }
        __syncwarp();
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const uint4 q = st[16 + 32 * p + lane];
            const float4 sg = sct4[g * 4 + p], sg8 = sct4[(g + 8) * 4 + p];
#pragma unroll
            for (int s2 = 0; s2 < 2; s2++) {
                const uint32_t wa = s2 ? q.z : q.x, wb = s2 ? q.w : q.y;
                const uint32_t a0 = and_or(wa, K.m4, K.k128), a1 = and_or(wb, K.m4, K.k128);
                const uint32_t a2 = and_or(wa >> 4, K.m4, K.k128), a3 = and_or(wb >> 4, K.m4, K.k128);
                const uint32_t a4 = and_or(wa >> 8, K.m4, K.k128), a5 = and_or(wb >> 8, K.m4, K.k128);
                const uint32_t a6 = and_or(wa >> 12, K.m4, K.k128), a7 = and_or(wb >> 12, K.m4, K.k128);
                const float dsc = s2 ? sg.z : sg.x, e = s2 ? sg.w : sg.y;
                const float dsc8 = s2 ? sg8.z : sg8.x, e8 = s2 ? sg8.w : sg8.y;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int e0 = koff + (2 * p + s2) * 32 + 8 * t;
                    const XB<F32X> xb = load_xb<F32X>(xrow[nt], e0, e0 + 4);
                    float c[4], sx[4];
                    mma_x<F32X>(c, a0, a1, a2, a3, xb, 0, zero);
                    mma_x<F32X>(c, a4, a5, a6, a7, xb, 1, c);
                    mma_x<F32X>(sx, K.ones, K.ones, K.ones, K.ones, xb, 0, zero);
                    mma_x<F32X>(sx, K.ones, K.ones, K.ones, K.ones, xb, 1, sx);
                    y[nt][0] = fmaf(dsc, c[0], fmaf(-e, sx[0], y[nt][0]));
                    y[nt][1] = fmaf(dsc, c[1], fmaf(-e, sx[1], y[nt][1]));
                    y[nt][2] = fmaf(dsc8, c[2], fmaf(-e8, sx[2], y[nt][2]));
                    y[nt][3] = fmaf(dsc8, c[3], fmaf(-e8, sx[3], y[nt][3]));
                }
            }
        }
        (void)ES;
    }
};

// ---- Q8_0 ----
template <>
struct TileFmt<NNQ_Q8_0, 8> {
    static constexpr int kBytes = 4352;
    static constexpr int kElems = 256;
    template <int NT, bool F32X>
    static __device__ __forceinline__ void tile(const uint8_t *stage, float4 *, const uint8_t *const (&xrow)[NT],
                                                int koff, int lane, int g, int t, const MnConsts &K,
                                                float (&y)[NT][4]) {
        const uint4 *st = reinterpret_cast<const uint4 *>(stage);
        const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint4 dg = st[g], dg8 = st[8 + g];   // the eight block scales of rows g and g + 8
        const uint32_t dgw[4] = {dg.x, dg.y, dg.z, dg.w}, dg8w[4] = {dg8.x, dg8.y, dg8.z, dg8.w};
#pragma unroll
        for (int sb = 0; sb < 8; sb++) {
            const uint4 q = st[16 + 32 * sb + lane];   // {low g, high g, low g+8, high g+8}
            const float2 d2 = __half22float2(*reinterpret_cast<const __half2 *>(&dgw[sb >> 1]));
            const float2 d28 = __half22float2(*reinterpret_cast<const __half2 *>(&dg8w[sb >> 1]));
            const float d = sb & 1 ? d2.y : d2.x, d8 = sb & 1 ? d28.y : d28.x;
            uint32_t L[4], L8[4], H[4], H8[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                L[i] = and_or(q.x >> (4 * i), K.m4, K.k128);
                H[i] = and_or(q.y >> (4 * i), K.m4, K.k2048);
                L8[i] = and_or(q.z >> (4 * i), K.m4, K.k128);
                H8[i] = and_or(q.w >> (4 * i), K.m4, K.k2048);
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int e0 = koff + sb * 32 + 8 * t;
                const XB<F32X> xb = load_xb<F32X>(xrow[nt], e0, e0 + 4);
                float c[4], sx[4];
                mma_x<F32X>(c, L[0], L8[0], L[1], L8[1], xb, 0, zero);
                mma_x<F32X>(c, L[2], L8[2], L[3], L8[3], xb, 1, c);
                mma_x<F32X>(c, H[0], H8[0], H[1], H8[1], xb, 0, c);
                mma_x<F32X>(c, H[2], H8[2], H[3], H8[3], xb, 1, c);
                mma_x<F32X>(sx, K.ones, K.ones, K.ones, K.ones, xb, 0, zero);
                mma_x<F32X>(sx, K.ones, K.ones, K.ones, K.ones, xb, 1, sx);
                y[nt][0] = fmaf(d, fmaf(-2304.0f, sx[0], c[0]), y[nt][0]);
                y[nt][1] = fmaf(d, fmaf(-2304.0f, sx[1], c[1]), y[nt][1]);
                y[nt][2] = fmaf(d8, fmaf(-2304.0f, sx[2], c[2]), y[nt][2]);
                y[nt][3] = fmaf(d8, fmaf(-2304.0f, sx[3], c[3]), y[nt][3]);
            }
        }
    }
};

// ---- Q6_K ----
template <>
struct TileFmt<NNQ_Q6_K, 8> {
    static constexpr int kBytes = 3360;
    static constexpr int kElems = 256;
    template <int NT, bool F32X>
    static __device__ __forceinline__ void tile(const uint8_t *stage, float4 *sct4, const uint8_t *const (&xrow)[NT],
                                                int koff, int lane, int g, int t, const MnConsts &K,
                                                float (&y)[NT][4]) {
        const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint32_t *sw = reinterpret_cast<const uint32_t *>(stage);
        // d * sc of the tile: this lane's share (rows g, g+8; scale groups 4t .. 4t+3)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int r = 8 * h + g;
            const float d = __half2float(reinterpret_cast<const __half *>(stage + 256)[r]);
            const uint32_t w = sw[r * 4 + t];
            sct4[r * 4 + t] = make_float4(d * (float)(int8_t)(w & 0xFFu), d * (float)(int8_t)((w >> 8) & 0xFFu),
                                          d * (float)(int8_t)((w >> 16) & 0xFFu), d * (float)(int8_t)(w >> 24));
        }
        __syncwarp();
        const float2 *sct2 = reinterpret_cast<const float2 *>(sct4);
#pragma unroll
        for (int sb = 0; sb < 8; sb++) {
            const uint32_t *cw = sw + 72 + sb * 96;   // byte 288 + 384 sb
            const uint32_t lo = cw[lane], lo8 = cw[32 + lane], hw = cw[64 + lane];
            const float2 sg = sct2[g * 8 + sb], sg8 = sct2[(g + 8) * 8 + sb];   // groups 2sb, 2sb+1
            uint32_t L[4], L8[4], H[4], H8[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                L[i] = and_or(lo >> (4 * i), K.m4, K.k128);
                L8[i] = and_or(lo8 >> (4 * i), K.m4, K.k128);
                H[i] = and_or(hw >> (2 * i), K.m2, K.k2048);
                H8[i] = and_or(hw >> (8 + 2 * i), K.m2, K.k2048);
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int e0 = koff + sb * 32 + 4 * t;
                const XB<F32X> xb = load_xb<F32X>(xrow[nt], e0, e0 + 16);
                float ca[4], cb[4], sa[4], sb4[4];
                mma_x<F32X>(ca, L[0], L8[0], L[1], L8[1], xb, 0, zero);
                mma_x<F32X>(ca, H[0], H8[0], H[1], H8[1], xb, 0, ca);
                mma_x<F32X>(sa, K.ones, K.ones, K.ones, K.ones, xb, 0, zero);
                mma_x<F32X>(cb, L[2], L8[2], L[3], L8[3], xb, 1, zero);
                mma_x<F32X>(cb, H[2], H8[2], H[3], H8[3], xb, 1, cb);
                mma_x<F32X>(sb4, K.ones, K.ones, K.ones, K.ones, xb, 1, zero);
                y[nt][0] = fmaf(sg.x, fmaf(-2208.0f, sa[0], ca[0]), fmaf(sg.y, fmaf(-2208.0f, sb4[0], cb[0]), y[nt][0]));
                y[nt][1] = fmaf(sg.x, fmaf(-2208.0f, sa[1], ca[1]), fmaf(sg.y, fmaf(-2208.0f, sb4[1], cb[1]), y[nt][1]));
                y[nt][2] = fmaf(sg8.x, fmaf(-2208.0f, sa[2], ca[2]), fmaf(sg8.y, fmaf(-2208.0f, sb4[2], cb[2]), y[nt][2]));
                y[nt][3] = fmaf(sg8.x, fmaf(-2208.0f, sa[3], ca[3]), fmaf(sg8.y, fmaf(-2208.0f, sb4[3], cb[3]), y[nt][3]));
            }
        }
    }
};

// ---- Q4_0 / Q4_1: 32-blocks with an fp16 scale (and an fp16 minimum) ----
// Tile: [0,256) fp16 d[row][block] (Q4_1: then 256 B fp16 m[row][block]); then per block 256 B,
// lane l = 4g + t 8 B = {T16 word row g, T16 word row g+8} of elements 8t..8t+7.
//   Q4_0  y += d * (c - 136 s)      (code q, value d (q - 8))
//   Q4_1  y += d * (c - 128 s) + m * s
template <int FMT>
struct TileQ4x {
    static constexpr bool kMin = FMT == NNQ_Q4_1;
    static constexpr int kBytes = (kMin ? 512 : 256) + 2048;
    static constexpr int kElems = 256;
    template <int NT, bool F32X>
    static __device__ __forceinline__ void tile(const uint8_t *stage, float4 *, const uint8_t *const (&xrow)[NT],
                                                int koff, int lane, int g, int t, const MnConsts &K,
                                                float (&y)[NT][4]) {
        const uint4 *st = reinterpret_cast<const uint4 *>(stage);
        const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint4 dg = st[g], dg8 = st[8 + g];
        const uint32_t dgw[4] = {dg.x, dg.y, dg.z, dg.w}, dg8w[4] = {dg8.x, dg8.y, dg8.z, dg8.w};
        uint32_t mgw[4] = {0, 0, 0, 0}, mg8w[4] = {0, 0, 0, 0};
        if (kMin) {
            const uint4 mg = st[16 + g], mg8 = st[24 + g];
            mgw[0] = mg.x; mgw[1] = mg.y; mgw[2] = mg.z; mgw[3] = mg.w;
            mg8w[0] = mg8.x; mg8w[1] = mg8.y; mg8w[2] = mg8.z; mg8w[3] = mg8.w;
        }
        const uint2 *cw = reinterpret_cast<const uint2 *>(stage + (kMin ? 512 : 256));
#pragma unroll
        for (int sb = 0; sb < 8; sb++) {
            const uint2 q = cw[sb * 32 + lane];
            const float2 d2 = __half22float2(*reinterpret_cast<const __half2 *>(&dgw[sb >> 1]));
            const float2 d28 = __half22float2(*reinterpret_cast<const __half2 *>(&dg8w[sb >> 1]));
            const float d = sb & 1 ? d2.y : d2.x, d8 = sb & 1 ? d28.y : d28.x;
            float mn = 0.0f, mn8 = 0.0f;
            if (kMin) {
                const float2 m2 = __half22float2(*reinterpret_cast<const __half2 *>(&mgw[sb >> 1]));
                const float2 m28 = __half22float2(*reinterpret_cast<const __half2 *>(&mg8w[sb >> 1]));
                mn = sb & 1 ? m2.y : m2.x;
                mn8 = sb & 1 ? m28.y : m28.x;
            }
            uint32_t L[4], L8[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                L[i] = and_or(q.x >> (4 * i), K.m4, K.k128);
                L8[i] = and_or(q.y >> (4 * i), K.m4, K.k128);
            }
            // per unit of the activation sum: -136 d (Q4_0), -128 d + m (Q4_1)
            const float e = kMin ? fmaf(-128.0f, d, mn) : -136.0f * d, e8 = kMin ? fmaf(-128.0f, d8, mn8) : -136.0f * d8;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int e0 = koff + sb * 32 + 8 * t;
                const XB<F32X> xb = load_xb<F32X>(xrow[nt], e0, e0 + 4);
                float c[4], sx[4];
                mma_x<F32X>(c, L[0], L8[0], L[1], L8[1], xb, 0, zero);
                mma_x<F32X>(c, L[2], L8[2], L[3], L8[3], xb, 1, c);
                mma_x<F32X>(sx, K.ones, K.ones, K.ones, K.ones, xb, 0, zero);
                mma_x<F32X>(sx, K.ones, K.ones, K.ones, K.ones, xb, 1, sx);
                y[nt][0] = fmaf(d, c[0], fmaf(e, sx[0], y[nt][0]));
                y[nt][1] = fmaf(d, c[1], fmaf(e, sx[1], y[nt][1]));
                y[nt][2] = fmaf(d8, c[2], fmaf(e8, sx[2], y[nt][2]));
                y[nt][3] = fmaf(d8, c[3], fmaf(e8, sx[3], y[nt][3]));
            }
        }
    }
};
template <>
struct TileFmt<NNQ_Q4_0, 8> : TileQ4x<NNQ_Q4_0> {};
template <>
struct TileFmt<NNQ_Q4_1, 8> : TileQ4x<NNQ_Q4_1> {};

// ---- MXFP4 (K-blocked layouts: 17-byte blocks, or codes [N, K/2] + scales [N, K/32]) ----
// Tile = 16 rows x SB blocks of 32 (SB = 8, or 6 when K is a multiple of 192 but not of 256, as
// the 2880-wide gpt-oss experts): [0,128) E8M0 scale bytes, row r at 8r; then per block 256 B,
// lane l = 4g + t 8 B = {word row g, word row g+8} for elements 8t..8t+7. A word keeps the
// eight E2M1 magnitudes (3 bits) in nibble order and the sign of pair i = (e_2i, e_2i+1) at
// bits 4i+3 and 4i+19. Magnitudes become bf16 through two 8-entry byte tables (PRMT), the signs
// are shifted onto bits 15 / 31: exact values, no offset, one scale per block applied on the
// f32 accumulators.
template <int SB>
struct TileFmt<NNQ_MXFP4_SPLIT, SB> {
    static constexpr int kBytes = 128 + 256 * SB;
    static constexpr int kElems = 32 * SB;
    static __device__ __forceinline__ void pairs(uint32_t w, const MnConsts &K, uint32_t (&a)[4]) {
        const uint32_t sel = w & 0x77777777u;
        const uint32_t lo_e = __byte_perm(K.tl0, K.tl1, sel), hi_e = __byte_perm(K.th0, K.th1, sel);
        const uint32_t lo_o = __byte_perm(K.tl0, K.tl1, sel >> 16), hi_o = __byte_perm(K.th0, K.th1, sel >> 16);
        a[0] = __byte_perm(lo_e, hi_e, 0x5140) | ((w << 12) & 0x80008000u);
        a[1] = __byte_perm(lo_e, hi_e, 0x7362) | ((w << 8) & 0x80008000u);
        a[2] = __byte_perm(lo_o, hi_o, 0x5140) | ((w << 4) & 0x80008000u);
        a[3] = __byte_perm(lo_o, hi_o, 0x7362) | (w & 0x80008000u);
    }
    static __device__ __forceinline__ float scale_of(uint2 s, int sb) {   // 2^(e-127); e = 0 -> 2^-127
        const uint32_t w = sb < 4 ? s.x : s.y;
        const int i = sb & 3;
        const uint32_t bits = (i < 3 ? w << (23 - 8 * i) : w >> 1) & 0x7F800000u;
        return __uint_as_float(max(bits, 0x00400000u));
    }
    template <int NT, bool F32X>
    static __device__ __forceinline__ void tile(const uint8_t *stage, float4 *, const uint8_t *const (&xrow)[NT],
                                                int koff, int lane, int g, int t, const MnConsts &K,
                                                float (&y)[NT][4]) {
        const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint2 sg = reinterpret_cast<const uint2 *>(stage)[g], sg8 = reinterpret_cast<const uint2 *>(stage)[g + 8];
        const uint2 *cw = reinterpret_cast<const uint2 *>(stage + 128);
#pragma unroll
        for (int sb = 0; sb < SB; sb++) {
            const uint2 q = cw[sb * 32 + lane];
            uint32_t A[4], A8[4];
            pairs(q.x, K, A);
            pairs(q.y, K, A8);
            const float d = scale_of(sg, sb), d8 = scale_of(sg8, sb);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int e0 = koff + sb * 32 + 8 * t;
                const XB<F32X> xb = load_xb<F32X>(xrow[nt], e0, e0 + 4);
                float c[4];
                mma_x<F32X>(c, A[0], A8[0], A[1], A8[1], xb, 0, zero);
                mma_x<F32X>(c, A[2], A8[2], A[3], A8[3], xb, 1, c);
                y[nt][0] = fmaf(d, c[0], y[nt][0]);
                y[nt][1] = fmaf(d, c[1], y[nt][1]);
                y[nt][2] = fmaf(d8, c[2], y[nt][2]);
                y[nt][3] = fmaf(d8, c[3], y[nt][3]);
            }
        }
    }
};

// ---- MXFP4, nn-gptoss [K, N] layout (blocks of 32 along N, i.e. across the rows of a tile) ----
// A tile (16 rows n x SB*32 k) lies inside one 32-wide block of n, so its scales depend on k only:
// [0, 32 SB) E8M0 scale per k; then the code words as in the K-blocked MXFP4 tile. The scales are
// applied to the activations (an exact power-of-two multiply of the bf16 pairs, e = 0 -> 2^-126),
// the accumulators need no further scaling.
template <int SB>
struct TileFmt<NNQ_MXFP4_GPTOSS, SB> {
    static constexpr int kBytes = 32 * SB + 256 * SB;
    static constexpr int kElems = 32 * SB;
    static __device__ __forceinline__ uint32_t scale_pair(uint32_t w, uint32_t sel) {   // two bytes -> bf16x2 2^(e-127)
        return __vmaxu2(__byte_perm(w, 0u, sel) << 7, 0x00800080u);
    }
    static __device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
        __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    }
    template <int NT, bool F32X>
    static __device__ __forceinline__ void tile(const uint8_t *stage, float4 *, const uint8_t *const (&xrow)[NT],
                                                int koff, int lane, int g, int t, const MnConsts &K,
                                                float (&y)[NT][4]) {
        const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint2 *cw = reinterpret_cast<const uint2 *>(stage + 32 * SB);
#pragma unroll
        for (int sb = 0; sb < SB; sb++) {
            const uint2 q = cw[sb * 32 + lane];
            const uint2 e8 = *reinterpret_cast<const uint2 *>(stage + sb * 32 + 8 * t);   // scales of k = 8t .. 8t+7
            uint32_t A[4], A8[4];
            TileFmt<NNQ_MXFP4_SPLIT, SB>::pairs(q.x, K, A);
            TileFmt<NNQ_MXFP4_SPLIT, SB>::pairs(q.y, K, A8);
            const uint32_t s0 = scale_pair(e8.x, 0x4140), s1 = scale_pair(e8.x, 0x4342);
            const uint32_t s2 = scale_pair(e8.y, 0x4140), s3 = scale_pair(e8.y, 0x4342);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int e0 = koff + sb * 32 + 8 * t;
                XB<F32X> xb = load_xb<F32X>(xrow[nt], e0, e0 + 4);
                xb.hi = make_uint4(mul2(xb.hi.x, s0), mul2(xb.hi.y, s1), mul2(xb.hi.z, s2), mul2(xb.hi.w, s3));
                if (F32X) xb.lo = make_uint4(mul2(xb.lo.x, s0), mul2(xb.lo.y, s1), mul2(xb.lo.z, s2), mul2(xb.lo.w, s3));
                float c[4];
                mma_x<F32X>(c, A[0], A8[0], A[1], A8[1], xb, 0, zero);
                mma_x<F32X>(c, A[2], A8[2], A[3], A8[3], xb, 1, c);
                y[nt][0] += c[0];
                y[nt][1] += c[1];
                y[nt][2] += c[2];
                y[nt][3] += c[3];
            }
        }
    }
};

template <int BYTES>
__device__ __forceinline__ void issue_tile_n(uint32_t dst, const void *src, uint32_t bar, int pred) {
    asm volatile(
        "{\n .reg .pred q;\n setp.ne.s32 q, %3, 0;\n"
        " @q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%2], %4;\n"
        " @q cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %4, [%2];\n}"
        ::"r"(dst), "l"(src), "r"(bar), "r"(pred), "n"(BYTES) : "memory");
}

struct MnPlan {
    int ring_off, sct_off, part_off, bar_off, total;
};

__host__ __device__ inline MnPlan mn_plan(int tile_bytes, int stages, int nt) {
    MnPlan p;
    p.ring_off = 0;
    p.sct_off = kWarps * stages * tile_bytes;
    p.part_off = p.sct_off + kWarps * 1024;
    p.bar_off = p.part_off + 2 * kWarps * nt * 32 * 16;
    p.total = p.bar_off + (kWarps * kMaxStages + 4) * 8;
    return p;
}

template <int FMT, int SB, int NT, bool F32X>
__global__ void __launch_bounds__(kWarps * 32, 2)
skinny_mn_kernel(const __grid_constant__ SkinnyParams P) {
    using TF = TileFmt<FMT, SB>;
    constexpr int TB = TF::kBytes;
    constexpr int TE = TF::kElems;   // weights per tile row
    extern __shared__ __align__(128) uint8_t smem[];
    const MnPlan L = mn_plan(TB, P.stages, NT);
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
    const int g = lane >> 2, t = lane & 3;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int stages = P.stages;
    uint8_t *ring = smem + warp * stages * TB;
    float4 *sct4 = reinterpret_cast<float4 *>(smem + L.sct_off + warp * 1024);
    float4 *part4 = reinterpret_cast<float4 *>(smem + L.part_off);
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t bars_s = smem_u32(smem + L.bar_off);
    const uint32_t bar_s = bars_s + warp * kMaxStages * 8;
    const uint32_t full_s = bars_s + kWarps * kMaxStages * 8;   // full[2], then empty[2]
    const uint32_t empty_s = full_s + 16;

    if (tid == 0) {
        mbar_init(full_s, kWarps);
        mbar_init(full_s + 8, kWarps);
        mbar_init(empty_s, 1);
        mbar_init(empty_s + 8, 1);
    }
    if (lane == 0) {
        for (int d = 0; d < stages; d++) mbar_init(bar_s + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // this warp's share of K; a unit is one row tile, CTA c handles units c, c + grid, ...
    const int kb_lo = (warp * P.kblocks) / kWarps, kb_hi = ((warp + 1) * P.kblocks) / kWarps;
    const int nkb = kb_hi - kb_lo;
    const int n_units = cta < P.total_tiles ? (P.total_tiles - cta + grid - 1) / grid : 0;
    auto locate = [&](int unit, int &j, int &rt) {
        const int gt = cta + unit * grid;
        j = 0;
#pragma unroll
        for (int i = 1; i < kSkinnyMaxJobs; i++)
            if (i < P.njobs && gt >= P.job[i].tile_begin) j = i;
        rt = gt - P.job[j].tile_begin;
    };

    // ---- weights first: they do not depend on anything an earlier kernel produced ----
    int pf_unit = -1, pf_k = 0, pf_slot = 0;
    unsigned issued = 0;
    const uint8_t *pf_src = nullptr;
    bool pf_done = nkb == 0 || n_units == 0;
    auto pf_advance_unit = [&]() {
        if (++pf_unit >= n_units) {
            pf_done = true;
            return;
        }
        int j, rt;
        locate(pf_unit, j, rt);
        pf_src = P.job[j].tiled + ((size_t)rt * P.kblocks + kb_lo) * TB;
        pf_k = 0;
    };
    if (!pf_done) pf_advance_unit();
    const int is_lane0 = lane == 0;
    auto issue = [&]() {
        if (!pf_done) {
            issue_tile_n<TB>(ring_s + pf_slot * TB, pf_src, bar_s + 8 * pf_slot, is_lane0);
            issued++;
            pf_slot = pf_slot + 1 == stages ? 0 : pf_slot + 1;
            pf_src += TB;
            if (++pf_k == nkb) pf_advance_unit();
        }
    };
    for (int d = 0; d < stages; d++) issue();

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // activations of this lane's token column(s); a column beyond M reads token 0 and is never stored
    const uint8_t *xrow[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int tok = nt * 8 + g;
        xrow[nt] = reinterpret_cast<const uint8_t *>(P.x) + (size_t)(tok < P.m ? tok : 0) * P.kblocks * TE * (F32X ? 4 : 2);
    }
    MnConsts K;
    K.init();

    unsigned consumed = 0;
    int slot = 0;
    uint32_t phase = 0;
    bool failed = false;

    auto put = [&](const SkinnyJobDev &J, int tok, int row, float v) {
        if (tok < P.m && row < J.n) {
            if (J.bias) v += __ldg(J.bias + row);
            const size_t at = (size_t)tok * J.n + row;
            if (P.y_dt == NNQ_F32) reinterpret_cast<float *>(J.y)[at] = v;
            else reinterpret_cast<__nv_bfloat16 *>(J.y)[at] = __float2bfloat16_rn(v);
        }
    };
    // the warp whose turn it is adds the 8 partial tiles of the unit and writes the outputs
    auto finish = [&](int unit) {
        const int b = unit & 1;
        if (!mbar_wait_fast(full_s + 8 * b, (unit >> 1) & 1u)) {
            failed = true;
            return;
        }
        int j, rt;
        locate(unit, j, rt);
        const SkinnyJobDev &J = P.job[j];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int w = 0; w < kWarps; w++) {
                const float4 a = part4[((b * kWarps + w) * NT + nt) * 32 + lane];
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
            const int row = rt * 16 + g, tok = nt * 8 + 2 * t;
            put(J, tok, row, v.x);
            put(J, tok + 1, row, v.y);
            put(J, tok, row + 8, v.z);
            put(J, tok + 1, row + 8, v.w);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_s + 8 * b);
    };

#pragma unroll 1
    for (int unit = 0; unit < n_units && !failed; unit++) {
        float y[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int r = 0; r < 4; r++) y[nt][r] = 0.0f;
        bool ok = true;
#pragma unroll 1
        for (int k = 0; k < nkb; k++) {
            ok &= mbar_wait_fast(bar_s + 8 * slot, phase);
            TF::template tile<NT, F32X>(ring + slot * TB, sct4, xrow, (kb_lo + k) * TE, lane, g, t, K, y);
            consumed++;
            if (++slot == stages) {
                slot = 0;
                phase ^= 1u;
            }
            __syncwarp();  // all lanes have read the slot and the scale scratch
            issue();
        }
        if (!ok) {
            failed = true;
            break;
        }
        const int b = unit & 1;
        if (unit >= 2 && !mbar_wait_fast(empty_s + 8 * b, ((unit >> 1) - 1) & 1u)) {
            failed = true;
            break;
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
            part4[((b * kWarps + warp) * NT + nt) * 32 + lane] = make_float4(y[nt][0], y[nt][1], y[nt][2], y[nt][3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(full_s + 8 * b);
        if (unit >= 1 && warp == (unit - 1) % kWarps) finish(unit - 1);
    }
    if (!failed && n_units >= 1 && warp == (n_units - 1) % kWarps) finish(n_units - 1);
    if (failed) {
        if (lane == 0) atomicExch(P.status, 1);
        for (unsigned n = consumed; n < issued; n++) {
            mbar_wait(bar_s + 8 * slot, phase);
            if (++slot == stages) {
                slot = 0;
                phase ^= 1u;
            }
        }
    }
}

// ---------------------------------------------------------------------------------
// Grouped token-column kernel: the expert products of a mixture-of-experts block
// ---------------------------------------------------------------------------------
//
// One launch covers every local expert. The routed rows arrive sorted by expert (offset[e] ..
// offset[e+1], computed on the device by the grouping kernels); a unit is (expert, group of up
// to 8 routed rows, row tile of the expert's weight), units are numbered expert-major, then
// row group, then row tile, and CTA c handles units c, c + grid, ... The eight MMA columns are
// the rows of the group; their activations are read through the row -> token table (first
// product) or directly (second product). Everything else is the token-column kernel: per-warp
// rings of bulk-copied tiles, K split over the 8 warps, partial tiles met in shared memory.

struct GroupedParams {
    const uint8_t *tiled;     // expert e at tiled + e * expert_stride
    size_t expert_stride;
    const float *bias;        // [E][n] or NULL
    const void *x;            // activations, row stride = kblocks * tile elements
    const int *rowtok;        // routed row -> flat assignment index (token = index / top_k), or NULL: row itself
    const int *offset;        // [E + 1] first routed row of each expert
    float *out;               // [rows][n]
    int experts, top_k, n, row_tiles, kblocks, stages;
    int *status;
};

template <int FMT, int SB, int NT, bool F32X>
__global__ void __launch_bounds__(kWarps * 32, 2)
skinny_grouped_kernel(const __grid_constant__ GroupedParams P) {
    using TF = TileFmt<FMT, SB>;
    constexpr int TB = TF::kBytes;
    constexpr int TE = TF::kElems;
    constexpr int kGroupRows = 8 * NT;   // routed rows per unit
    extern __shared__ __align__(128) uint8_t smem[];
    const MnPlan L = mn_plan(TB, P.stages, NT);
    __shared__ int goff[kMoeMaxExperts + 1];   // first row group of each expert
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
    const int g = lane >> 2, t = lane & 3;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int stages = P.stages;
    uint8_t *ring = smem + warp * stages * TB;
    float4 *sct4 = reinterpret_cast<float4 *>(smem + L.sct_off + warp * 1024);
    float4 *part4 = reinterpret_cast<float4 *>(smem + L.part_off);
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t bars_s = smem_u32(smem + L.bar_off);
    const uint32_t bar_s = bars_s + warp * kMaxStages * 8;
    const uint32_t full_s = bars_s + kWarps * kMaxStages * 8;
    const uint32_t empty_s = full_s + 16;

    if (tid == 0) {
        mbar_init(full_s, kWarps);
        mbar_init(full_s + 8, kWarps);
        mbar_init(empty_s, 1);
        mbar_init(empty_s + 8, 1);
    }
    if (lane == 0) {
        for (int d = 0; d < stages; d++) mbar_init(bar_s + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the routing tables come from the kernels before this one
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) {
        int acc = 0;
        for (int e = 0; e < P.experts; e++) {
            goff[e] = acc;
            acc += (P.offset[e + 1] - P.offset[e] + kGroupRows - 1) / kGroupRows;
        }
        goff[P.experts] = acc;
    }
    __syncthreads();
    const int total_units = goff[P.experts] * P.row_tiles;

    const int kb_lo = (warp * P.kblocks) / kWarps, kb_hi = ((warp + 1) * P.kblocks) / kWarps;
    const int nkb = kb_hi - kb_lo;
    const int n_units = cta < total_units ? (total_units - cta + grid - 1) / grid : 0;
    // expert, first routed row, rows in the group and row tile of a unit. A CTA's units come in
    // increasing order, so the expert is found by advancing a cursor (one for the copy stream, which
    // runs ahead, one for the arithmetic).
    auto locate = [&](int unit, int &ecur, int &r0, int &cnt, int &rt) {
        const int u = cta + unit * grid;
        const int q = u / P.row_tiles;
        rt = u - q * P.row_tiles;
        while (ecur + 1 < P.experts && q >= goff[ecur + 1]) ecur++;
        r0 = P.offset[ecur] + (q - goff[ecur]) * kGroupRows;
        cnt = min(kGroupRows, P.offset[ecur + 1] - r0);
    };
    int e_pf = 0, e_main = 0;

    int pf_unit = -1, pf_k = 0, pf_slot = 0;
    unsigned issued = 0;
    const uint8_t *pf_src = nullptr;
    bool pf_done = nkb == 0 || n_units == 0;
    auto pf_advance_unit = [&]() {
        if (++pf_unit >= n_units) {
            pf_done = true;
            return;
        }
        int r0, cnt, rt;
        locate(pf_unit, e_pf, r0, cnt, rt);
        pf_src = P.tiled + (size_t)e_pf * P.expert_stride + ((size_t)rt * P.kblocks + kb_lo) * TB;
        pf_k = 0;
    };
    if (!pf_done) pf_advance_unit();
    const int is_lane0 = lane == 0;
    auto issue = [&]() {
        if (!pf_done) {
            issue_tile_n<TB>(ring_s + pf_slot * TB, pf_src, bar_s + 8 * pf_slot, is_lane0);
            issued++;
            pf_slot = pf_slot + 1 == stages ? 0 : pf_slot + 1;
            pf_src += TB;
            if (++pf_k == nkb) pf_advance_unit();
        }
    };
    for (int d = 0; d < stages; d++) issue();

    MnConsts K;
    K.init();
    unsigned consumed = 0;
    int slot = 0;
    uint32_t phase = 0;
    bool failed = false;
    const size_t xstride = (size_t)P.kblocks * TE * (F32X ? 4 : 2);

    auto finish = [&](int unit, int e, int r0, int cnt, int rt) {
        const int b = unit & 1;
        if (!mbar_wait_fast(full_s + 8 * b, (unit >> 1) & 1u)) {
            failed = true;
            return;
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int w = 0; w < kWarps; w++) {
                const float4 a = part4[((b * kWarps + w) * NT + nt) * 32 + lane];
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
            const int row = rt * 16 + g, tok = nt * 8 + 2 * t;
            const float vals[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int tk = tok + (i & 1), rw = row + (i >> 1) * 8;
                if (tk < cnt && rw < P.n) {
                    float o = vals[i];
                    if (P.bias) o += __ldg(P.bias + (size_t)e * P.n + rw);
                    P.out[(size_t)(r0 + tk) * P.n + rw] = o;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_s + 8 * b);
    };

#pragma unroll 1
    int pe = 0, pr0 = 0, pcnt = 0, prt = 0;   // the previous unit, for its deferred write-out
    for (int unit = 0; unit < n_units && !failed; unit++) {
        int r0, cnt, rt;
        locate(unit, e_main, r0, cnt, rt);
        // this lane's column(s): routed row r0 + g (+ 8); a column beyond the group reads row r0 and is never stored
        const uint8_t *xrow[NT];
        float y[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int col = nt * 8 + g;
            const int r = r0 + (col < cnt ? col : 0);
            const int src = P.rowtok ? __ldg(P.rowtok + r) / P.top_k : r;
            xrow[nt] = reinterpret_cast<const uint8_t *>(P.x) + (size_t)src * xstride;
#pragma unroll
            for (int i = 0; i < 4; i++) y[nt][i] = 0.0f;
        }
        bool ok = true;
#pragma unroll 1
        for (int k = 0; k < nkb; k++) {
            ok &= mbar_wait_fast(bar_s + 8 * slot, phase);
            TF::template tile<NT, F32X>(ring + slot * TB, sct4, xrow, (kb_lo + k) * TE, lane, g, t, K, y);
            consumed++;
            if (++slot == stages) {
                slot = 0;
                phase ^= 1u;
            }
            __syncwarp();
            issue();
        }
        if (!ok) {
            failed = true;
            break;
        }
        const int b = unit & 1;
        if (unit >= 2 && !mbar_wait_fast(empty_s + 8 * b, ((unit >> 1) - 1) & 1u)) {
            failed = true;
            break;
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
            part4[((b * kWarps + warp) * NT + nt) * 32 + lane] = make_float4(y[nt][0], y[nt][1], y[nt][2], y[nt][3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(full_s + 8 * b);
        if (unit >= 1 && warp == (unit - 1) % kWarps) finish(unit - 1, pe, pr0, pcnt, prt);
        pe = e_main; pr0 = r0; pcnt = cnt; prt = rt;
    }
    if (!failed && n_units >= 1 && warp == (n_units - 1) % kWarps) finish(n_units - 1, pe, pr0, pcnt, prt);
    if (failed) {
        if (lane == 0) atomicExch(P.status, 1);
        for (unsigned n = consumed; n < issued; n++) {
            mbar_wait(bar_s + 8 * slot, phase);
            if (++slot == stages) {
                slot = 0;
                phase ^= 1u;
            }
        }
    }
}

// ---------------------------------------------------------------------------------
// repack of Q8_0 and Q6_K raw blocks into their tiled layouts
// ---------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t t16_word(const uint32_t *e) {   // eight four-bit fields
    return (e[0] | (e[2] << 4)) | ((e[4] | (e[6] << 4)) << 8) | ((e[1] | (e[3] << 4)) << 16) | ((e[5] | (e[7] << 4)) << 24);
}

// one thread per (row, super-block of 256, sub-block of 32)
__global__ void repack_q8_0_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ tiled, int n, int kblocks) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)n * kblocks * 8) return;
    const int sb = (int)(idx & 7);
    const int64_t blk = idx >> 3;
    const int kb = (int)(blk % kblocks), row = (int)(blk / kblocks);
    const uint8_t *b = raw + (((int64_t)row * kblocks + kb) * 8 + sb) * 34;
    uint8_t *tile = tiled + ((int64_t)(row >> 4) * kblocks + kb) * 4352;
    const int r16 = row & 15, g = row & 7, upper = (row >> 3) & 1;
    *reinterpret_cast<uint16_t *>(tile + r16 * 16 + sb * 2) = (uint16_t)(b[0] | (b[1] << 8));
#pragma unroll
    for (int t = 0; t < 4; t++) {
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t u = (uint32_t)b[2 + 8 * t + i] ^ 0x80u;   // q + 128
            lo[i] = u & 15u;
            hi[i] = u >> 4;
        }
        uint32_t *dst = reinterpret_cast<uint32_t *>(tile + 256 + 512 * sb + 16 * (4 * g + t) + 8 * upper);
        dst[0] = t16_word(lo);
        dst[1] = t16_word(hi);
    }
}

__global__ void repack_q6_k_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ tiled, int n, int kblocks) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)n * kblocks * 8) return;
    const int sb = (int)(idx & 7);
    const int64_t blk = idx >> 3;
    const int kb = (int)(blk % kblocks), row = (int)(blk / kblocks);
    const uint8_t *b = raw + blk * 210;
    uint8_t *tile = tiled + ((int64_t)(row >> 4) * kblocks + kb) * 3360;
    const int r16 = row & 15, g = row & 7, upper = (row >> 3) & 1;
    tile[r16 * 16 + 2 * sb] = b[192 + 2 * sb];
    tile[r16 * 16 + 2 * sb + 1] = b[192 + 2 * sb + 1];
    if (sb == 0) *reinterpret_cast<uint16_t *>(tile + 256 + 2 * r16) = (uint16_t)(b[208] | (b[209] << 8));
    // six-bit codes of the sub-block: flat element i -> low nibble i & 1 of ql[i / 2], field i & 3 of qh[i / 4]
    auto code = [&](int i) -> uint32_t {
        const int e = sb * 32 + i;
        const uint32_t ql = (b[e >> 1] >> (4 * (e & 1))) & 15u;
        const uint32_t qh = (b[128 + (e >> 2)] >> (2 * (e & 3))) & 3u;
        return ql | (qh << 4);
    };
    uint8_t *cw = tile + 288 + 384 * sb;
#pragma unroll
    for (int t = 0; t < 4; t++) {
        uint32_t lo[8], h2 = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t c = code(i < 4 ? 4 * t + i : 16 + 4 * t + (i - 4));
            lo[i] = c & 15u;
            // pair i / 2: even element in the low half, odd element in the high half
            h2 |= (c >> 4) << ((i & 1) * 16 + (i >> 1) * 2);
        }
        const int lane = 4 * g + t;
        reinterpret_cast<uint32_t *>(cw + 128 * upper)[lane] = t16_word(lo);
        // both rows of a lane share the two-bit word: byte-wise stores keep the other row's bits
        uint8_t *hb = cw + 256 + 4 * lane;
        hb[upper] = (uint8_t)(h2 & 0xFFu);
        hb[2 + upper] = (uint8_t)((h2 >> 16) & 0xFFu);
    }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------

nnq_status skinny_init(nnq_ctx *) { return NNQ_OK; }

// Q4_0 (18-byte blocks: d, 16 code bytes) / Q4_1 (20-byte blocks: d, m, 16 code bytes); element 2j is
// the low nibble of byte j, element 2j + 1 the high nibble (the reference's order). One thread per
// (row, block of 32).
template <bool MIN>
__global__ void repack_q4x_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ tiled, int n, int ktiles) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)n * ktiles * 8) return;
    constexpr int BS = MIN ? 20 : 18, TB = (MIN ? 512 : 256) + 2048;
    const int row = (int)(idx / (ktiles * 8)), blk = (int)(idx % (ktiles * 8));
    const int kb = blk >> 3, sb = blk & 7;
    const uint8_t *b = raw + idx * BS;
    uint8_t *tile = tiled + ((int64_t)(row >> 4) * ktiles + kb) * TB;
    const int r16 = row & 15, g = row & 7, upper = (row >> 3) & 1;
    *reinterpret_cast<uint16_t *>(tile + r16 * 16 + sb * 2) = (uint16_t)(b[0] | (b[1] << 8));
    if (MIN) *reinterpret_cast<uint16_t *>(tile + 256 + r16 * 16 + sb * 2) = (uint16_t)(b[2] | (b[3] << 8));
    const uint8_t *qs = b + (MIN ? 4 : 2);
#pragma unroll
    for (int t = 0; t < 4; t++) {
        uint32_t e[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int el = 8 * t + i;
            e[i] = (el & 1) ? (uint32_t)(qs[el >> 1] >> 4) : (uint32_t)(qs[el >> 1] & 15u);
        }
        reinterpret_cast<uint32_t *>(tile + (MIN ? 512 : 256) + 256 * sb + 8 * (4 * g + t))[upper] = t16_word(e);
    }
}

// MXFP4 -> tiles. CORE: 17-byte blocks (scale, 16 code bytes); SPLIT: codes [N, K/2] and scales
// [N, K/32] apart. Low nibble = even element in both. One thread per (row, block of 32).
template <int SB>
__global__ void repack_mxfp4_kernel(const uint8_t *__restrict__ raw, const uint8_t *__restrict__ scales,
                                    uint8_t *__restrict__ tiled, int n, int ktiles, int split) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t bpr = (int64_t)ktiles * SB;   // blocks per row
    if (idx >= (int64_t)n * bpr) return;
    const int row = (int)(idx / bpr), blk = (int)(idx % bpr);
    const int kb = blk / SB, sb = blk % SB;
    const uint8_t *codes = split ? raw + idx * 16 : raw + idx * 17 + 1;
    const uint8_t e8 = split ? scales[idx] : raw[idx * 17];
    uint8_t *tile = tiled + ((int64_t)(row >> 4) * ktiles + kb) * (128 + 256 * SB);
    const int r16 = row & 15, g = row & 7, upper = (row >> 3) & 1;
    tile[r16 * 8 + sb] = e8;
    if (SB < 8 && sb == 0)
        for (int z = SB; z < 8; z++) tile[r16 * 8 + z] = 0;
#pragma unroll
    for (int t = 0; t < 4; t++) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t byte = codes[4 * t + (i >> 1)];
            const uint32_t c = (i & 1) ? byte >> 4 : byte & 15u;
            word |= (c & 7u) << (4 * i);                                    // magnitude, nibble order
            word |= (c >> 3) << (4 * (i >> 1) + 3 + 16 * (i & 1));          // sign of pair i / 2
        }
        reinterpret_cast<uint32_t *>(tile + 128 + 256 * sb + 8 * (4 * g + t))[upper] = word;
    }
}

// nn-gptoss expert tensor [K, N] (codes [K, N/2], high nibble = even column; scales [K, N/32]) ->
// tiles of the transposed product (rows = n). One thread per (n, block of 32 k).
template <int SB>
__global__ void repack_mxfp4_kn_kernel(const uint8_t *__restrict__ codes, const uint8_t *__restrict__ scales,
                                       uint8_t *__restrict__ tiled, int n, int k, int ktiles) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int kblocks = k / 32;
    if (idx >= (int64_t)n * kblocks) return;
    const int row = (int)(idx / kblocks), blk = (int)(idx % kblocks);
    const int kt = blk / SB, sb = blk % SB;
    constexpr int TB = 32 * SB + 256 * SB;
    uint8_t *tile = tiled + ((int64_t)(row >> 4) * ktiles + kt) * TB;
    const int r16 = row & 15, g = row & 7, upper = (row >> 3) & 1;
    const int k0 = blk * 32;
    if (r16 == 0)
        for (int i = 0; i < 32; i++) tile[sb * 32 + i] = scales[(int64_t)(k0 + i) * (n / 32) + row / 32];
#pragma unroll
    for (int t = 0; t < 4; t++) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t byte = codes[(int64_t)(k0 + 8 * t + i) * (n / 2) + row / 2];
            const uint32_t c = (row & 1) ? byte & 15u : byte >> 4;
            word |= (c & 7u) << (4 * i);
            word |= (c >> 3) << (4 * (i >> 1) + 3 + 16 * (i & 1));
        }
        reinterpret_cast<uint32_t *>(tile + 32 * SB + 256 * sb + 8 * (4 * g + t))[upper] = word;
    }
}

size_t tiled_bytes_kn(int64_t n, int64_t k, int *sb_out) {
    const int sb = k % 256 == 0 ? 8 : (k % 192 == 0 ? 6 : 0);
    if (sb_out) *sb_out = sb;
    if (sb == 0 || n <= 0 || n % 32 != 0 || n > (1 << 24) || k > (1 << 24)) return 0;
    return (size_t)(n / 16) * (size_t)(k / (32 * sb)) * (size_t)(288 * sb);
}

nnq_status repack_kn_into(nnq_ctx *ctx, const uint8_t *d_codes, const uint8_t *d_scales, int64_t n, int64_t k, uint8_t *dst) {
    int sb = 0;
    if (tiled_bytes_kn(n, k, &sb) == 0) return fail(ctx, NNQ_ERR_UNSUPPORTED, "no tiled layout for a [K, N] expert tensor with K = %lld, N = %lld", (long long)k, (long long)n);
    const int64_t total = n * (k / 32);
    const int grid = (int)((total + 255) / 256);
    const int ktiles = (int)(k / (32 * sb));
    if (sb == 8) repack_mxfp4_kn_kernel<8><<<grid, 256>>>(d_codes, d_scales, dst, (int)n, (int)k, ktiles);
    else repack_mxfp4_kn_kernel<6><<<grid, 256>>>(d_codes, d_scales, dst, (int)n, (int)k, ktiles);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "repack launch");
}

static int tile_bytes_of(int fmt, int sb) {
    switch (fmt) {
        case NNQ_Q4_K: case NNQ_Q4_K_GGML: return TileFmt<NNQ_Q4_K>::kBytes;
        case NNQ_Q8_0: return TileFmt<NNQ_Q8_0>::kBytes;
        case NNQ_Q6_K: return TileFmt<NNQ_Q6_K>::kBytes;
        case NNQ_Q4_0: return TileFmt<NNQ_Q4_0>::kBytes;
        case NNQ_Q4_1: return TileFmt<NNQ_Q4_1>::kBytes;
        case NNQ_MXFP4_CORE: case NNQ_MXFP4_SPLIT: return 128 + 256 * sb;
        default: return 0;
    }
}

// Sub-blocks per tile row for this format and K; 0 = no tiled layout.
static int tile_sb_of(int fmt, int64_t k) {
    switch (fmt) {
        case NNQ_Q4_K: case NNQ_Q4_K_GGML: case NNQ_Q8_0: case NNQ_Q6_K: case NNQ_Q4_0: case NNQ_Q4_1: return k % 256 == 0 ? 8 : 0;
        case NNQ_MXFP4_CORE: case NNQ_MXFP4_SPLIT: return k % 256 == 0 ? 8 : (k % 192 == 0 ? 6 : 0);
        default: return 0;
    }
}

size_t tiled_bytes_for(int fmt, int64_t n, int64_t k, int *sb_out) {
    const int sb = tile_sb_of(fmt, k);
    if (sb_out) *sb_out = sb;
    if (sb == 0 || n <= 0 || k <= 0 || n > (1 << 24) || k > (1 << 24)) return 0;
    return (size_t)((n + 15) / 16) * (size_t)(k / (32 * sb)) * tile_bytes_of(fmt, sb);
}

nnq_status repack_into(nnq_ctx *ctx, int fmt, const uint8_t *d_raw, const uint8_t *d_scales, int64_t n, int64_t k,
                       uint8_t *d) {
    int sb = 0;
    const size_t bytes = tiled_bytes_for(fmt, n, k, &sb);
    if (bytes == 0) return fail(ctx, NNQ_ERR_UNSUPPORTED, "no tiled layout for format %d with K = %lld", fmt, (long long)k);
    const int ktiles = (int)(k / (32 * sb));
    nnq_status s = NNQ_OK;
    if (n % 16) s = check_cuda(ctx, cudaMemset(d, 0, bytes), "cudaMemset tiled weight");
    if (s != NNQ_OK) return s;
    const int64_t total = fmt == NNQ_MXFP4_CORE || fmt == NNQ_MXFP4_SPLIT ? n * (k / 32) : n * ktiles * 8;
    const int grid = (int)((total + 255) / 256);
    const int split = fmt == NNQ_MXFP4_SPLIT;
    switch (fmt) {
        case NNQ_Q4_K: repack_q4k_kernel<false><<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        case NNQ_Q4_K_GGML: repack_q4k_kernel<true><<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        case NNQ_Q8_0: repack_q8_0_kernel<<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        case NNQ_Q6_K: repack_q6_k_kernel<<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        case NNQ_Q4_0: repack_q4x_kernel<false><<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        case NNQ_Q4_1: repack_q4x_kernel<true><<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        default:
            if (sb == 8) repack_mxfp4_kernel<8><<<grid, 256>>>(d_raw, d_scales, d, (int)n, ktiles, split);
            else repack_mxfp4_kernel<6><<<grid, 256>>>(d_raw, d_scales, d, (int)n, ktiles, split);
            break;
    }
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "repack launch");
}

nnq_status build_tiled_buffer(nnq_ctx *ctx, int fmt, const uint8_t *d_raw, const uint8_t *d_scales, int64_t n,
                              int64_t k, uint8_t **out, size_t *out_bytes, int *out_sb) {
    *out = nullptr;
    *out_bytes = 0;
    *out_sb = 0;
    int sb = 0;
    const size_t bytes = tiled_bytes_for(fmt, n, k, &sb);
    if (bytes == 0) return NNQ_OK;
    uint8_t *d = nullptr;
    nnq_status s = check_cuda(ctx, cudaMalloc(&d, bytes), "cudaMalloc tiled weight");
    if (s != NNQ_OK) return s;
    s = repack_into(ctx, fmt, d_raw, d_scales, n, k, d);
    if (s == NNQ_OK) s = check_cuda(ctx, cudaDeviceSynchronize(), "repack");
    if (s != NNQ_OK) {
        cudaFree(d);
        return s;
    }
    *out = d;
    *out_bytes = bytes;
    *out_sb = sb;
    return NNQ_OK;
}

static int layout_of(int fmt) {
    switch (fmt) {
        case NNQ_Q4_K: case NNQ_Q4_K_GGML: return kTiledQ4K;
        case NNQ_Q8_0: return kTiledQ8_0;
        case NNQ_Q6_K: return kTiledQ6K;
        case NNQ_MXFP4_CORE: case NNQ_MXFP4_SPLIT: return kTiledMxfp4;
        case NNQ_Q4_0: return kTiledQ4_0;
        case NNQ_Q4_1: return kTiledQ4_1;
        default: return kTiledNone;
    }
}

nnq_status build_tiled(nnq_ctx *ctx, nnq_weight *w) {
    nnq_status s = build_tiled_buffer(ctx, w->fmt, w->d_raw, w->d_scales, w->n, w->k, &w->d_tiled, &w->tiled_bytes, &w->tile_sb);
    if (s != NNQ_OK) return s;
    w->tiled_layout = w->d_tiled ? layout_of(w->fmt) : kTiledNone;
    return NNQ_OK;
}

// Ring depth and CTAs per SM that fit shared memory for this K. More resident warps beat a
// deeper ring (the kernel is bound by instruction latency, not by bytes in flight), so: three
// CTAs per SM with a 2-deep ring when that fits, else two with up to 4 stages, else one;
// stages = 0 when K is too large altogether.
static void pick_stages(int kblocks, bool f32x, int *stages, int *ctas_per_sm) {
    static const char *env_st = getenv("NNQ_SKINNY_STAGES");  // tuning aid
    const int forced = env_st ? atoi(env_st) : 0;
    static const char *env_ctas = getenv("NNQ_SKINNY_CTAS");  // tuning aid
    int max_ctas = f32x ? 2 : 3;   // register budget of the two instantiations
    if (env_ctas && atoi(env_ctas) > 0 && atoi(env_ctas) < max_ctas) max_ctas = atoi(env_ctas);
    for (int ctas = max_ctas; ctas >= 1; ctas--) {
        const int budget = kSmemMax / ctas - 1024;
        const int hi = forced > 0 ? forced : (ctas == 3 ? 2 : kMaxStages);
        const int lo = forced > 0 ? forced : 2;
        for (int st = hi; st >= lo; st--)
            if (smem_plan(kblocks, st, f32x).total <= budget) {
                *stages = st;
                *ctas_per_sm = ctas;
                return;
            }
    }
    *stages = 0;
    *ctas_per_sm = 0;
}

bool skinny_supported(const nnq_weight *w, int64_t m, int x_dt) {
    if (!w || w->tiled_layout == kTiledNone || m < 1 || m > kSkinnyMaxM) return false;
    // token-column kernel: f32 activations (two MMAs per product) up to 8 tokens only
    if (m > 1 || w->tiled_layout != kTiledQ4K) return x_dt == NNQ_BF16 || m <= 8;
    int st, cps;
    pick_stages((int)(w->k / 256), x_dt == NNQ_F32, &st, &cps);
    return st > 0;
}

template <bool F32X, int KS, bool FUSED = false>
static cudaError_t launch_kernel(const SkinnyParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(skinny_q4k_m1_kernel<F32X, KS, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax - 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    // programmatic dependent launch: the kernel prefetches weights while its predecessor in
    // the stream drains, and waits (griddepcontrol.wait) before reading activations
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const char *env_pdl = getenv("NNQ_SKINNY_PDL");  // tuning aid
    cfg.numAttrs = env_pdl && atoi(env_pdl) == 0 ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, skinny_q4k_m1_kernel<F32X, KS, FUSED>, P);
}

template <bool F32X, bool FUSED>
static cudaError_t launch_ks_f(int ksplit, const SkinnyParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    switch (ksplit) {
        case 1: return launch_kernel<F32X, 1, FUSED>(P, grid, smem_bytes, stream);
        case 2: return launch_kernel<F32X, 2, FUSED>(P, grid, smem_bytes, stream);
        case 4: return launch_kernel<F32X, 4, FUSED>(P, grid, smem_bytes, stream);
        default: return launch_kernel<F32X, 8, FUSED>(P, grid, smem_bytes, stream);
    }
}

template <bool F32X>
static cudaError_t launch_ks(int ksplit, const SkinnyParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    return P.fr.enabled ? launch_ks_f<F32X, true>(ksplit, P, grid, smem_bytes, stream)
                        : launch_ks_f<F32X, false>(ksplit, P, grid, smem_bytes, stream);
}

template <int FMT, int SB, int NT, bool F32X>
static cudaError_t launch_mn(const SkinnyParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(skinny_mn_kernel<FMT, SB, NT, F32X>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, skinny_mn_kernel<FMT, SB, NT, F32X>, P);
}

template <int FMT, int SB = 8>
static cudaError_t launch_mn_fmt(const SkinnyParams &P, int nt, bool f32x, int grid, int smem_bytes, cudaStream_t stream) {
    if (f32x) return launch_mn<FMT, SB, 1, true>(P, grid, smem_bytes, stream);
    return nt == 1 ? launch_mn<FMT, SB, 1, false>(P, grid, smem_bytes, stream) : launch_mn<FMT, SB, 2, false>(P, grid, smem_bytes, stream);
}

// Diagnostic only (NNQ_SKINNY_DIAG=4): read the tiled weights of the jobs with plain coalesced
// 16-byte loads and nothing else -- the read bandwidth a launch of this size can reach.
__global__ void __launch_bounds__(256) stream_read_kernel(const SkinnyParams P, int *sink) {
    uint32_t acc = 0;
    for (int j = 0; j < P.njobs; j++) {
        const uint4 *p = reinterpret_cast<const uint4 *>(P.job[j].tiled);
        size_t n16 = (size_t)P.job[j].row_tiles * P.kblocks * (kTileBytes / 16);
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
            uint4 v = __ldg(p + i);
            acc ^= v.x ^ v.y ^ v.z ^ v.w;
        }
    }
    if (acc == 0x12345678u && sink) *sink = 1;   // keeps the loads alive; sink is NULL
}

// One launch: jobs that share their activations (same x pointer, same K).
static nnq_status launch_group(nnq_ctx *ctx, const SkinnyJob *jobs, int count, int x_dt, int m, int y_dt,
                               cudaStream_t stream, const FusedReduce *fr = nullptr) {
    SkinnyParams P;
    memset(&P, 0, sizeof(P));
    if (fr) P.fr = *fr;
    P.njobs = count;
    P.m = m;
    P.y_dt = y_dt;
    P.x = jobs[0].x;
    const int tile_sb = jobs[0].w->tile_sb;
    P.kblocks = (int)(jobs[0].w->k / (32 * tile_sb));
    P.status = ctx->d_status;
    static const char *env_diag = getenv("NNQ_SKINNY_DIAG");
    P.diag = env_diag ? atoi(env_diag) : 0;
    static const char *env_l2 = getenv("NNQ_SKINNY_L2PF");
    P.l2_prefetch = env_l2 ? atoi(env_l2) : 0;
    const bool f32x = x_dt == NNQ_F32;
    int ctas_per_sm = 0;
    const int layout = jobs[0].w->tiled_layout;
    static const char *env_tc = getenv("NNQ_SKINNY_TOKCOL");  // tuning aid: token-column kernel at M = 1 too
    const bool token_columns = m > 1 || layout != kTiledQ4K || (env_tc && atoi(env_tc) == 1 && !f32x);
    if (!token_columns) pick_stages(P.kblocks, f32x, &P.stages, &ctas_per_sm);
    else P.stages = 2;
    if (fr && ctas_per_sm > 2) ctas_per_sm = 2;   // register budget of the fused variant
    if (P.stages == 0) return fail(ctx, NNQ_ERR_UNSUPPORTED, "K = %lld is too large for the skinny kernel", (long long)jobs[0].w->k);
    int tiles = 0;
    for (int i = 0; i < count; i++) {
        const nnq_weight *w = jobs[i].w;
        SkinnyJobDev &J = P.job[i];
        J.tiled = w->d_tiled;
        J.bias = jobs[i].bias;
        J.y = jobs[i].y;
        J.n = (int)w->n;
        J.row_tiles = (int)((w->n + 15) / 16);
        J.tile_begin = tiles;
        tiles += J.row_tiles;
    }
    P.total_tiles = tiles;
    if (token_columns) {
        // a unit is one row tile, its K split over the 8 warps
        const int nt = m <= 8 ? 1 : 2;
        const int smem_bytes = mn_plan(tile_bytes_of(jobs[0].w->fmt, tile_sb), P.stages, nt).total;
        int per_sm = kSmemMax / (smem_bytes + 1024);
        if (per_sm > 2) per_sm = 2;   // register budget of the kernel
        int grid = tiles < ctx->sm_count * per_sm ? tiles : ctx->sm_count * per_sm;
        cudaError_t e;
        if (layout == kTiledQ4K) e = launch_mn_fmt<NNQ_Q4_K>(P, nt, f32x, grid, smem_bytes, stream);
        else if (layout == kTiledQ8_0) e = launch_mn_fmt<NNQ_Q8_0>(P, nt, f32x, grid, smem_bytes, stream);
        else if (layout == kTiledQ6K) e = launch_mn_fmt<NNQ_Q6_K>(P, nt, f32x, grid, smem_bytes, stream);
        else if (layout == kTiledQ4_0) e = launch_mn_fmt<NNQ_Q4_0>(P, nt, f32x, grid, smem_bytes, stream);
        else if (layout == kTiledQ4_1) e = launch_mn_fmt<NNQ_Q4_1>(P, nt, f32x, grid, smem_bytes, stream);
        else if (tile_sb == 8) e = launch_mn_fmt<NNQ_MXFP4_SPLIT, 8>(P, nt, f32x, grid, smem_bytes, stream);
        else e = launch_mn_fmt<NNQ_MXFP4_SPLIT, 6>(P, nt, f32x, grid, smem_bytes, stream);
        ctx->launches++;
        return check_cuda(ctx, e, "skinny launch");
    }
    if (P.diag == 4) {
        stream_read_kernel<<<ctx->sm_count * 8, 256, 0, stream>>>(P, nullptr);
        ctx->launches++;
        return check_cuda(ctx, cudaGetLastError(), "diag launch");
    }
    // K split over the warps of a CTA: all 8 warps share a row tile when K allows, so that even
    // the smallest projections spread over every SM
    const int slots = ctx->sm_count * ctas_per_sm;
    int ksplit = 1;
    while (ksplit < kWarps && P.kblocks >= 2 * ksplit) ksplit *= 2;
    static const char *env_ks = getenv("NNQ_SKINNY_KS");  // tuning aid
    if (env_ks && atoi(env_ks) > 0) ksplit = atoi(env_ks);
    // persistent grid: every CTA resident
    const int rg = kWarps / ksplit;
    const int units = (tiles + rg - 1) / rg;
    int grid = units < slots ? units : slots;
    static const char *env_grid = getenv("NNQ_SKINNY_GRID");  // tuning aid
    if (env_grid && atoi(env_grid) > 0) grid = atoi(env_grid);
    if (grid > units) grid = units;
    if (grid < 1) grid = 1;
    int smem_bytes = smem_plan(P.kblocks, P.stages, f32x).total;
    cudaError_t e = f32x ? launch_ks<true>(ksplit, P, grid, smem_bytes, stream) : launch_ks<false>(ksplit, P, grid, smem_bytes, stream);
    ctx->launches++;
    return check_cuda(ctx, e, "skinny launch");
}

template <int FMT, int SB, int NT, bool F32X>
static cudaError_t launch_grouped_t(const GroupedParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(skinny_grouped_kernel<FMT, SB, NT, F32X>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemMax - 1024);   // the kernel also has a small static table
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    skinny_grouped_kernel<FMT, SB, NT, F32X><<<grid, kWarps * 32, smem_bytes, stream>>>(P);
    return cudaGetLastError();
}

template <int FMT, int SB>
static cudaError_t launch_grouped_x(const GroupedParams &P, bool f32x, int nt, int grid, int smem_bytes, cudaStream_t stream) {
    if (f32x) return launch_grouped_t<FMT, SB, 1, true>(P, grid, smem_bytes, stream);   // two MMAs per product: 8 rows
    return nt == 2 ? launch_grouped_t<FMT, SB, 2, false>(P, grid, smem_bytes, stream)
                   : launch_grouped_t<FMT, SB, 1, false>(P, grid, smem_bytes, stream);
}

nnq_status launch_grouped(nnq_ctx *ctx, const GroupedArgs &a, cudaStream_t stream) {
    if (a.experts < 1 || a.experts > kMoeMaxExperts) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad expert count %d", a.experts);
    int sb = 0;
    if ((a.kn_gptoss ? tiled_bytes_kn(a.n, a.k, &sb) : tiled_bytes_for(a.fmt, a.n, a.k, &sb)) == 0)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "no tiled layout for the grouped product");
    GroupedParams P;
    memset(&P, 0, sizeof(P));
    P.tiled = a.tiled;
    P.expert_stride = a.expert_stride;
    P.bias = a.bias;
    P.x = a.x;
    P.rowtok = a.rowtok;
    P.offset = a.offset;
    P.out = a.out;
    P.experts = a.experts;
    P.top_k = a.top_k;
    P.n = (int)a.n;
    P.row_tiles = (int)((a.n + 15) / 16);
    P.kblocks = (int)(a.k / (32 * sb));
    P.stages = 2;
    P.status = ctx->d_status;
    const bool f32x = a.x_dt == NNQ_F32;
    // 16-row groups once the experts see 5 or more rows on average (bf16 activations only)
    const int nt = !f32x && a.max_rows >= 5 * (int64_t)a.experts ? 2 : 1;
    const int smem_bytes = mn_plan(a.kn_gptoss ? 288 * sb : tile_bytes_of(a.fmt, sb), P.stages, nt).total;
    // every expert may end with a partly filled row group
    const int64_t max_units = (a.max_rows / (8 * nt) + a.experts) * P.row_tiles;
    int64_t grid = 2 * (int64_t)ctx->sm_count;
    if (grid > max_units) grid = max_units;
    if (grid < 1) grid = 1;
    cudaError_t e;
    if (a.kn_gptoss) {
        e = sb == 8 ? launch_grouped_x<NNQ_MXFP4_GPTOSS, 8>(P, f32x, nt, (int)grid, smem_bytes, stream)
                    : launch_grouped_x<NNQ_MXFP4_GPTOSS, 6>(P, f32x, nt, (int)grid, smem_bytes, stream);
        ctx->launches++;
        return check_cuda(ctx, e, "grouped product launch");
    }
    switch (layout_of(a.fmt)) {
        case kTiledQ4K: e = launch_grouped_x<NNQ_Q4_K, 8>(P, f32x, nt, (int)grid, smem_bytes, stream); break;
        case kTiledQ8_0: e = launch_grouped_x<NNQ_Q8_0, 8>(P, f32x, nt, (int)grid, smem_bytes, stream); break;
        case kTiledQ6K: e = launch_grouped_x<NNQ_Q6_K, 8>(P, f32x, nt, (int)grid, smem_bytes, stream); break;
        case kTiledQ4_0: e = launch_grouped_x<NNQ_Q4_0, 8>(P, f32x, nt, (int)grid, smem_bytes, stream); break;
        case kTiledQ4_1: e = launch_grouped_x<NNQ_Q4_1, 8>(P, f32x, nt, (int)grid, smem_bytes, stream); break;
        default:
            e = sb == 8 ? launch_grouped_x<NNQ_MXFP4_SPLIT, 8>(P, f32x, nt, (int)grid, smem_bytes, stream)
                        : launch_grouped_x<NNQ_MXFP4_SPLIT, 6>(P, f32x, nt, (int)grid, smem_bytes, stream);
            break;
    }
    ctx->launches++;
    return check_cuda(ctx, e, "grouped product launch");
}

bool skinny_fused_supported(const nnq_weight *w, int64_t m, int x_dt) {
    return m == 1 && w && w->tiled_layout == kTiledQ4K && skinny_supported(w, m, x_dt);
}

nnq_status launch_skinny_fused(nnq_ctx *ctx, const SkinnyJob &job, int x_dt, int y_dt, const FusedReduce &fr,
                               cudaStream_t stream) {
    if (!skinny_fused_supported(job.w, 1, x_dt)) return fail(ctx, NNQ_ERR_UNSUPPORTED, "fused product + all-reduce needs the M = 1 Q4_K kernel");
    return launch_group(ctx, &job, 1, x_dt, 1, y_dt, stream, &fr);
}

nnq_status launch_skinny(nnq_ctx *ctx, const SkinnyJob *jobs, int count, int x_dt, int64_t m, int y_dt,
                         cudaStream_t stream) {
    if (count < 1 || count > kSkinnyMaxJobs) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad job count %d", count);
    if (m < 1 || m > kSkinnyMaxM) return fail(ctx, NNQ_ERR_UNSUPPORTED, "skinny kernels cover 1 <= M <= %d", kSkinnyMaxM);
    // consecutive jobs with the same activations and K go out together
    int i = 0;
    while (i < count) {
        int jn = i + 1;
        while (jn < count && jobs[jn].x == jobs[i].x && jobs[jn].w->k == jobs[i].w->k && jobs[jn].w->tiled_layout == jobs[i].w->tiled_layout) jn++;
        nnq_status s = launch_group(ctx, jobs + i, jn - i, x_dt, (int)m, y_dt, stream);
        if (s != NNQ_OK) return s;
        i = jn;
    }
    return NNQ_OK;
}

}  // namespace nnq
