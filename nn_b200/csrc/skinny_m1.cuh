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
#pragma once
#include "skinny_common.cuh"

namespace nnq {

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
#ifdef NNQ_TILE_CHAINS4
    // four accumulator pairs (one per sub-block pair) instead of two chains of eight MMAs
    float ca[4][4], cb[4][4];
#pragma unroll
    for (int p = 0; p < 4; p++)
#pragma unroll
        for (int i = 0; i < 4; i++) ca[p][i] = cb[p][i] = 0.0f;
#define c ca[p]
#define c2 cb[p]
#endif
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
#ifdef NNQ_TILE_CHAINS4
#undef c
#undef c2
#pragma unroll
    for (int i = 0; i < 4; i++) {
        c[i] = (ca[0][i] + ca[1][i]) + (ca[2][i] + ca[3][i]);
        c2[i] = (cb[0][i] + cb[1][i]) + (cb[2][i] + cb[3][i]);
    }
#endif
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

// Stage one super-block of activations (256 values, 8 consecutive ones per lane in xv: one word of
// one sub-block). Every super-block gets its own power-of-two prescale to fp16 (its largest |x|
// lands in [1, 2): exact, and fp16 stays in range whatever the magnitude of x), so that a warp can
// stage its own part of K without waiting for the rest of the CTA. Writes the half-expanded
// operand, the per-sub-block offset sums and 1 / prescale.
template <bool F32X>
__device__ __forceinline__ void stage_x_block(const float (&xv)[8], int kb, uint8_t *xs, uint8_t *xs_lo, float *tab,
                                              float *xinv, int lane) {
    const int sb8 = lane >> 2;
    const bool odd = sb8 & 1;
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

// This lane's 8 activations of super-block kb. FRESH = true reads with loads that bypass L1
// (ld.global.cg): for a kernel that stages activations another CTA of the same launch has just written.
template <bool F32X, bool FRESH>
__device__ __forceinline__ void load_x_block(const void *x, int kb, int lane, float (&xv)[8]) {
    const int i = kb * 256 + lane * 8;
    if (F32X) {
        const float4 *px = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + i);
        float4 a = FRESH ? __ldcg(px) : __ldg(px), b = FRESH ? __ldcg(px + 1) : __ldg(px + 1);
        xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w;
        xv[4] = b.x; xv[5] = b.y; xv[6] = b.z; xv[7] = b.w;
    } else {
        const uint4 *pv = reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(x) + i);
        uint4 v = FRESH ? __ldcg(pv) : __ldg(pv);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            xv[2 * k] = __uint_as_float(u[k] << 16);
            xv[2 * k + 1] = __uint_as_float(u[k] & 0xFFFF0000u);
        }
    }
}

// Stage the activations of super-blocks kb_begin, kb_begin + kb_step, ... < kb_end; one warp per
// super-block.
template <bool F32X, bool FRESH = false>
__device__ __forceinline__ void stage_x_warp(const void *x, int kb_begin, int kb_end, int kb_step, uint8_t *xs,
                                             uint8_t *xs_lo, float *tab, float *xinv, int lane) {
#pragma unroll 2
    for (int kb = kb_begin; kb < kb_end; kb += kb_step) {
        float xv[8];
        load_x_block<F32X, FRESH>(x, kb, lane, xv);
        stage_x_block<F32X>(xv, kb, xs, xs_lo, tab, xinv, lane);
    }
}

// The same with the loads of up to BATCH super-blocks issued before the first is processed: one
// memory round trip instead of one per super-block.
template <bool F32X, bool FRESH, int BATCH>
__device__ __forceinline__ void stage_x_warp_batched(const void *x, int kb_begin, int kb_end, int kb_step, uint8_t *xs,
                                                     uint8_t *xs_lo, float *tab, float *xinv, int lane) {
    for (int kb0 = kb_begin; kb0 < kb_end; kb0 += BATCH * kb_step) {
        float xv[BATCH][8];
#pragma unroll
        for (int r = 0; r < BATCH; r++)
            if (kb0 + r * kb_step < kb_end) load_x_block<F32X, FRESH>(x, kb0 + r * kb_step, lane, xv[r]);
#pragma unroll
        for (int r = 0; r < BATCH; r++)
            if (kb0 + r * kb_step < kb_end) stage_x_block<F32X>(xv[r], kb0 + r * kb_step, xs, xs_lo, tab, xinv, lane);
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
#ifdef NNQ_DIAG
    if (!(P.diag & 2))
#endif
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // fused all-reduce: the exchange this launch takes part in (the epoch word is written by the
    // previous exchange, which the wait above has seen complete)
    unsigned ar_seq = 0, ar_limit = 0;
    if (FUSED) {
        ar_seq = *reinterpret_cast<volatile unsigned *>(P.fr.peers[P.fr.rank]) + 1u;
        ar_limit = comm_spin_limit(P.fr.peers[P.fr.rank]);
    }

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
                    } while (tag != ar_seq && ++spins <= ar_limit);
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
#ifdef NNQ_DIAG
                if (!(P.diag & 1))
#endif
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

}  // namespace nnq
