// Q4_K tile arithmetic on FP8 tensor-core instructions (bf16 activations, one token).
//
// A four-bit code q placed in the low nibble of a byte IS the e4m3 number q * 2^-9 (codes 0..7 are
// subnormals m/8 * 2^-6, codes 8..15 are 2^-6 * (1 + m/8)), so one AND turns a word of the tiled
// layout into four exact FP8 operands: half the logic ops per weight of the fp16 path (which
// needs one op per two weights plus a magic exponent), no offset to subtract afterwards, and
// mma.sync.m16n8k32.e4m3 issues at twice the rate of m16n8k16.f16 on this part (measured: 4.3
// against 8 clocks per instruction and SM sub-partition). The logic pipe, which runs at half
// rate, is what bounds the kernel; this path takes 32 ANDs per 2304-byte tile off it and moves the
// nibble shifts to the multiplier (mul.hi by 2^28).
//
// A bf16 activation (8 significant bits) is split into two e4m3 terms (4 + 4 bits): hi = rn(x),
// lo = x - hi. Each super-block of 256 activations is prescaled by its own power of two so that
// its largest magnitude lies in [128, 256); hi + lo is then exact for every activation above
// 2^-9 of the super-block's largest one, and carries an absolute error below 2^-17 of that
// largest one otherwise (e4m3's smallest subnormal is 2^-9). Products of the represented values
// are exact; sums are f32.
//
// MMA shape: k = 32 is one 32-weight sub-block; the eight n-columns are the eight sub-blocks of
// the super-block (the activation operand of sub-block s is zero except in column s), so the
// accumulators end up holding the per-sub-block dot products of 16 rows and the 6-bit scales /
// mins are applied once per super-block. The k slots of an A register follow the nibble order of
// the tiled layout (elements {0,4,1,5} and {2,6,3,7} of each 8-element word); the activation
// image is stored in the same order.
#pragma once
#include <cuda_fp8.h>

#include "skinny_m1.cuh"

namespace nnq {

__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// w >> n on the multiplier instead of the (half-rate) logic pipe
template <int N>
__device__ __forceinline__ uint32_t shr_mul(uint32_t w) {
    uint32_t d;
    asm("mul.hi.u32 %0, %1, %2;" : "=r"(d) : "r"(w), "r"(1u << (32 - N)));
    return d;
}

// Activation image of one super-block for the e4m3 path (same 1024-byte slot per super-block as the
// fp16 image): lane = 4 * sub-block + word holds 32 bytes, {hi k 0..3, hi k 16..19, lo k 0..3,
// lo k 16..19} of its word in the first 16 bytes when the sub-block is even, in the last 16 when
// it is odd, zeros in the other half. tab[kb * 16 + s] = (sum of the represented activations of
// sub-block s) / 512; xinv[kb] = 512 / prescale.
__device__ __forceinline__ void stage_x_block_e4m3(const float (&xv)[8], int kb, uint8_t *xs, float *tab, float *xinv,
                                                   int lane) {
    const int sb8 = lane >> 2;
    const bool odd = sb8 & 1;
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; k++) amax = fmaxf(amax, fabsf(xv[k]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    uint32_t ex = (__float_as_uint(amax) >> 23) & 0xFFu;
    ex = amax > 0.0f && ex < 255u ? min(max(ex, 8u), 252u) : 127u;
    const float scale = __uint_as_float((261u - ex) << 23);   // largest magnitude -> [128, 256)
    float s[8], xr[8];
#pragma unroll
    for (int k = 0; k < 8; k++) s[k] = xv[k] * scale;
    // element order of an operand register: {0, 4, 1, 5} then {2, 6, 3, 7}
    uint32_t bh[2], bl[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int e0 = 2 * r, e1 = 2 * r + 4, e2 = 2 * r + 1, e3 = 2 * r + 5;
        const uint32_t h01 = __nv_cvt_float2_to_fp8x2(make_float2(s[e0], s[e1]), __NV_SATFINITE, __NV_E4M3);
        const uint32_t h23 = __nv_cvt_float2_to_fp8x2(make_float2(s[e2], s[e3]), __NV_SATFINITE, __NV_E4M3);
        const __half2_raw f01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)h01, __NV_E4M3);
        const __half2_raw f23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)h23, __NV_E4M3);
        const float hv[4] = {__half2float(__ushort_as_half(f01.x)), __half2float(__ushort_as_half(f01.y)),
                             __half2float(__ushort_as_half(f23.x)), __half2float(__ushort_as_half(f23.y))};
        const int el[4] = {e0, e1, e2, e3};
        float rem[4];
#pragma unroll
        for (int j = 0; j < 4; j++) rem[j] = s[el[j]] - hv[j];
        const uint32_t l01 = __nv_cvt_float2_to_fp8x2(make_float2(rem[0], rem[1]), __NV_SATFINITE, __NV_E4M3);
        const uint32_t l23 = __nv_cvt_float2_to_fp8x2(make_float2(rem[2], rem[3]), __NV_SATFINITE, __NV_E4M3);
        const __half2_raw g01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)l01, __NV_E4M3);
        const __half2_raw g23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)l23, __NV_E4M3);
        const float lv[4] = {__half2float(__ushort_as_half(g01.x)), __half2float(__ushort_as_half(g01.y)),
                             __half2float(__ushort_as_half(g23.x)), __half2float(__ushort_as_half(g23.y))};
#pragma unroll
        for (int j = 0; j < 4; j++) xr[el[j]] = hv[j] + lv[j];
        bh[r] = h01 | (h23 << 16);
        bl[r] = l01 | (l23 << 16);
    }
    uint4 *dst = reinterpret_cast<uint4 *>(xs + kb * 1024 + lane * 32);
    const uint4 val = make_uint4(bh[0], bh[1], bl[0], bl[1]), zero = make_uint4(0, 0, 0, 0);
    dst[0] = odd ? zero : val;
    dst[1] = odd ? val : zero;
    float sx = ((xr[0] + xr[1]) + (xr[2] + xr[3])) + ((xr[4] + xr[5]) + (xr[6] + xr[7]));
    sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 1);
    sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 2);
    if ((lane & 3) == 0) tab[kb * 16 + sb8] = sx * (1.0f / 512.0f);
    if (lane == 0) xinv[kb] = __uint_as_float((ex + 2u) << 23);   // 512 / prescale = 2^(ex - 125)
}

template <bool FRESH, int BATCH>
__device__ __forceinline__ void stage_x_warp_e4m3(const void *x, int kb_begin, int kb_end, int kb_step, uint8_t *xs,
                                                  float *tab, float *xinv, int lane) {
    for (int kb0 = kb_begin; kb0 < kb_end; kb0 += BATCH * kb_step) {
        float xv[BATCH][8];
#pragma unroll
        for (int r = 0; r < BATCH; r++)
            if (kb0 + r * kb_step < kb_end) load_x_block<false, FRESH>(x, kb0 + r * kb_step, lane, xv[r]);
#pragma unroll
        for (int r = 0; r < BATCH; r++)
            if (kb0 + r * kb_step < kb_end) stage_x_block_e4m3(xv[r], kb0 + r * kb_step, xs, tab, xinv, lane);
    }
}

// One 2304-byte tile (16 rows x one super-block) against the staged activations: adds the 16 row
// sums' shares of this lane to yg (row g) and yg8 (row g + 8); the four lanes of a row group hold
// two sub-blocks each.
__device__ __forceinline__ void tile_mac_e4m3(const uint8_t *stage, uint32_t xs_s, const float *tab, float inv, int lane,
                                              int g, int t, BRegs &B, float &yg, float &yg8) {
    const uint4 *st = reinterpret_cast<const uint4 *>(stage);
    // activation operand: only the lanes whose column g is a sub-block of pair p load data for p;
    // every other register of B stays zero for the whole kernel
#pragma unroll
    for (int p = 0; p < 4; p++) lds256_if(B.v[p][0], B.v[p][1], xs_s, (g >> 1) == p);
    float c[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) c[i][j] = 0.0f;
    constexpr uint32_t kLow = 0x0F0F0F0Fu;
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const uint4 q = st[16 + 32 * p + lane];   // {(row g, sb 2p), (row g+8, sb 2p), (row g, sb 2p+1), (row g+8, sb 2p+1)}
        {
            const uint32_t a0 = q.x & kLow, a1 = q.y & kLow, a2 = shr_mul<4>(q.x) & kLow, a3 = shr_mul<4>(q.y) & kLow;
            mma_e4m3(c[0], a0, a1, a2, a3, B.v[p][0].x, B.v[p][0].y);
            mma_e4m3(c[1], a0, a1, a2, a3, B.v[p][0].z, B.v[p][0].w);
        }
        {
            const uint32_t a0 = q.z & kLow, a1 = q.w & kLow, a2 = shr_mul<4>(q.z) & kLow, a3 = shr_mul<4>(q.w) & kLow;
            mma_e4m3(c[2], a0, a1, a2, a3, B.v[p][1].x, B.v[p][1].y);
            mma_e4m3(c[3], a0, a1, a2, a3, B.v[p][1].z, B.v[p][1].w);
        }
    }
    float C[4];
#pragma unroll
    for (int i = 0; i < 4; i++) C[i] = (c[0][i] + c[1][i]) + (c[2][i] + c[3][i]);
    // C[0], C[1]: row g, sub-blocks 2t, 2t+1; C[2], C[3]: row g+8
    const float2 tb = *reinterpret_cast<const float2 *>(tab + 2 * t);
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint4 hd = st[8 * h + g];
        const uint32_t p01 = __byte_perm(hd.x, hd.y, 0x0073);
        const uint32_t p23 = __byte_perm(hd.z, hd.w, 0x0073);
        uint32_t dd = __byte_perm(p01, p23, 0x5410);
        const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&dd));
        const uint32_t o = reinterpret_cast<const uint32_t *>(stage)[(8 * h + g) * 4 + t];
        const float sc0 = (float)(o & 63u), sc1 = (float)(shr_mul<6>(o) & 63u);
        const float mn0 = (float)(shr_mul<12>(o) & 63u), mn1 = (float)(shr_mul<18>(o) & 63u);
        const float dot = sc0 * C[2 * h] + sc1 * C[2 * h + 1];
        const float mins = mn0 * tb.x + mn1 * tb.y;
        const float v = dm.x * dot - dm.y * mins;
        if (h) yg8 = fmaf(v, inv, yg8); else yg = fmaf(v, inv, yg);
    }
}

}  // namespace nnq
