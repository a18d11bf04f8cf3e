// Token-column kernels on tiled weights: 1..16 tokens of every tiled format, and the grouped
// variant for the expert products of a mixture-of-experts block.
#pragma once
#include "skinny_m1.cuh"

namespace nnq {

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

}  // namespace nnq
