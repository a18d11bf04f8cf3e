// Device-side block decoders on the RAW reference layouts. Every function decodes 32
// consecutive weights (one "chunk": flat elements [32c, 32c+32)) to f32, bit-identically
// to the reference's CPU decoders. Multiplications and subtractions use the explicit
// round-to-nearest intrinsics so that the compiler can never fuse them.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "nnq_internal.h"

namespace nnq {

__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
    return __half2float(__ushort_as_half(h));  // exact IEEE widening
}

__device__ __forceinline__ uint16_t ld_u16(const uint8_t *p) {
    return (uint16_t)(__ldg(p) | ((uint16_t)__ldg(p + 1) << 8));
}

// E2M1 magnitude for code&7 as f32 bits: 0, .5, 1, 1.5, 2, 3, 4, 6
__device__ __forceinline__ float e2m1_value(uint32_t code, float scale) {
    // magnitude m = code&7: m==0 -> 0; m==1 -> 0.5; else (1 + (m&1)/2) * 2^((m>>1)-1)
    uint32_t m = code & 7u;
    uint32_t bits = m == 0 ? 0u : (m == 1 ? 0x3F000000u : (((m >> 1) + 126u) << 23) | ((m & 1u) << 22));
    float v = __fmul_rn(__uint_as_float(bits), scale);
    return __uint_as_float(__float_as_uint(v) ^ ((code & 8u) << 28));
}

// nn-core / GPU-contract scale: 2^(e-127), e = 0 -> the f32 subnormal 2^-127, e = 255 -> +inf
__device__ __forceinline__ float mx_scale_core(uint32_t e) {
    return __uint_as_float(e ? (e << 23) : 0x00400000u);
}
// nn-gptoss scale: e = 0 -> 2^-126
__device__ __forceinline__ float mx_scale_gptoss(uint32_t e) {
    return __uint_as_float(e ? (e << 23) : 0x00800000u);
}

// Small integers as f32 without the conversion unit (a quarter-rate pipe, which the decoders fused
// into tensor-core products would otherwise saturate): the integer is placed in the mantissa of 2^23
// and 2^23 (+ bias) is subtracted, both exact. v < 2^23; returns (float)v - bias.
__device__ __forceinline__ float u2f(uint32_t v) { return __fsub_rn(__uint_as_float(v | 0x4B000000u), 8388608.0f); }
__device__ __forceinline__ float u2f_biased(uint32_t v, float bias) {
    return __fsub_rn(__uint_as_float(v | 0x4B000000u), 8388608.0f + bias);
}
// a byte holding an int8 as f32
__device__ __forceinline__ float s8_to_f(uint32_t byte) { return u2f_biased(byte ^ 0x80u, 128.0f); }

template <int FMT>
struct Decode;

template <>
struct Decode<NNQ_Q4_0> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + c * 18;
        float d = f16_bits_to_f32(ld_u16(b));
#pragma unroll
        for (int j = 0; j < 16; j++) {
            uint32_t q = __ldg(b + 2 + j);
            o[2 * j] = __fmul_rn(d, u2f_biased(q & 15u, 8.0f));
            o[2 * j + 1] = __fmul_rn(d, u2f_biased(q >> 4, 8.0f));
        }
    }
};

template <>
struct Decode<NNQ_Q4_1> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + c * 20;
        float d = f16_bits_to_f32(ld_u16(b));
        float m = f16_bits_to_f32(ld_u16(b + 2));
#pragma unroll
        for (int j = 0; j < 16; j++) {
            uint32_t q = __ldg(b + 4 + j);
            o[2 * j] = __fadd_rn(__fmul_rn(d, u2f(q & 15u)), m);
            o[2 * j + 1] = __fadd_rn(__fmul_rn(d, u2f(q >> 4)), m);
        }
    }
};

template <>
struct Decode<NNQ_Q8_0> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + c * 34;
        float d = f16_bits_to_f32(ld_u16(b));
#pragma unroll
        for (int j = 0; j < 32; j++) o[j] = __fmul_rn(d, s8_to_f(__ldg(b + 2 + j)));
    }
    // one block as 17 halfwords in shared memory (blocks are only 2-byte aligned); two weights per step
    // on the packed f32 pipe: byte 0 becomes 2^23 + (q + 128), byte 1 2^23 + 256 (q + 128), d / 256 is exact
    static __device__ __forceinline__ void chunk_halfwords(const uint16_t *p, float *o) {
        const float d = f16_bits_to_f32(p[0]);
        const float2 unbias = make_float2(-(8388608.0f + 128.0f), -(8388608.0f + 32768.0f));
        const float2 d2 = make_float2(d, __fmul_rn(d, 0.00390625f));
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const uint32_t t = p[1 + i];
            float2 c = make_float2(__uint_as_float((t & 0x00FFu) ^ 0x4B000080u), __uint_as_float((t & 0xFF00u) ^ 0x4B008000u));
            c = __fmul2_rn(__fadd2_rn(c, unbias), d2);
            o[2 * i] = c.x;
            o[2 * i + 1] = c.y;
        }
    }
};

template <>
struct Decode<NNQ_Q4_K> {
    // sub-block j of a super-block whose 16-byte header and 16 quant bytes are already in registers
    static __device__ __forceinline__ void chunk_regs(const uint4 &hdr, const uint4 &q, int j, float *o) {
        float d = f16_bits_to_f32((uint16_t)(hdr.x & 0xFFFFu));
        float dmin = f16_bits_to_f32((uint16_t)(hdr.x >> 16));
        // S[0..3] = hdr.y bytes, S[4..7] = hdr.z bytes, S[8..11] = hdr.w bytes
        uint32_t sc = ((hdr.y >> (8 * (j >> 1) + 4 * (j & 1))) & 15u) |
                      (((hdr.w >> (8 * (j >> 2) + 2 * (j & 3))) & 3u) << 4);
        uint32_t mn = ((hdr.z >> (8 * (j >> 1) + 4 * (j & 1))) & 15u) |
                      (((hdr.w >> (16 + 8 * (j >> 2) + 2 * (j & 3))) & 3u) << 4);
        float s = __fmul_rn(d, u2f(sc));
        float m = __fmul_rn(dmin, u2f(mn));
        uint32_t qw[4] = {q.x, q.y, q.z, q.w};
        // Two weights (one byte) per step on the packed f32 pipe, every lane rounded as the scalar
        // operation would be. The high nibble stays where it is: the mantissa then holds 16 q, and
        // s / 16 (exact) takes its place as the factor; x - m is x + (-m).
        const float2 unbias = make_float2(-8388608.0f, -8388608.0f);
        const float2 s2 = make_float2(s, __fmul_rn(s, 0.0625f));
        const float2 nm2 = make_float2(-m, -m);
#pragma unroll
        for (int v = 0; v < 4; v++) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t t = qw[v] >> (8 * i);
                float2 c = make_float2(__uint_as_float((t & 0x0Fu) | 0x4B000000u), __uint_as_float((t & 0xF0u) | 0x4B000000u));
                c = __fadd2_rn(__fmul2_rn(__fadd2_rn(c, unbias), s2), nm2);
                o[8 * v + 2 * i] = c.x;
                o[8 * v + 2 * i + 1] = c.y;
            }
        }
    }
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + (c >> 3) * 144;  // 144-byte blocks are 16-byte aligned
        int j = (int)(c & 7);
        uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(b));
        uint4 q = __ldg(reinterpret_cast<const uint4 *>(b + 16 + 16 * j));
        chunk_regs(hdr, q, j, o);
    }
};

template <>
struct Decode<NNQ_Q4_K_GGML> {
    // sub-block j of a super-block: the 16-byte header and the 32 quant bytes of the pair of sub-blocks
    // j / 2 are already in registers (low nibbles when j is even)
    static __device__ __forceinline__ void chunk_regs(const uint4 &hdr, const uint4 &q0, const uint4 &q1, int j, float *o) {
        float d = f16_bits_to_f32((uint16_t)(hdr.x & 0xFFFFu));
        float dmin = f16_bits_to_f32((uint16_t)(hdr.x >> 16));
        uint32_t S[3] = {hdr.y, hdr.z, hdr.w};
        auto sbyte = [&](int i) -> uint32_t { return (S[i >> 2] >> (8 * (i & 3))) & 0xFFu; };
        uint32_t sc, mn;
        if (j < 4) {
            sc = sbyte(j) & 63u;
            mn = sbyte(j + 4) & 63u;
        } else {
            sc = (sbyte(j + 4) & 15u) | ((sbyte(j - 4) >> 6) << 4);
            mn = (sbyte(j + 4) >> 4) | ((sbyte(j) >> 6) << 4);
        }
        float s = __fmul_rn(d, u2f(sc));
        float m = __fmul_rn(dmin, u2f(mn));
        // Two weights (two bytes, the same nibble of each) per step on the packed f32 pipe, every lane
        // rounded as the scalar operation would be. The nibbles stay where they are: the mantissa of
        // 2^23 then holds 2^p q, and s / 2^p (exact) takes the place of s; x - m is x + (-m).
        const int sh = 4 * (j & 1);
        const uint32_t mask_lo = 0x0Fu << sh, mask_hi = 0x0F00u << sh;
        const float f_lo = sh ? 0.0625f : 1.0f;
        const float2 unbias = make_float2(-8388608.0f, -8388608.0f);
        const float2 s2 = make_float2(__fmul_rn(s, f_lo), __fmul_rn(s, f_lo * 0.00390625f));
        const float2 nm2 = make_float2(-m, -m);
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int v = 0; v < 8; v++) {
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const uint32_t t = qw[v] >> (16 * i);
                float2 c = make_float2(__uint_as_float((t & mask_lo) | 0x4B000000u), __uint_as_float((t & mask_hi) | 0x4B000000u));
                c = __fadd2_rn(__fmul2_rn(__fadd2_rn(c, unbias), s2), nm2);
                o[4 * v + 2 * i] = c.x;
                o[4 * v + 2 * i + 1] = c.y;
            }
        }
    }
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + (c >> 3) * 144;
        int j = (int)(c & 7);  // sub-block: group g = j/2, low nibbles when j even
        uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(b));
        const uint4 *qp = reinterpret_cast<const uint4 *>(b + 16 + 32 * (j >> 1));
        chunk_regs(hdr, __ldg(qp), __ldg(qp + 1), j, o);
    }
};

template <>
struct Decode<NNQ_Q6_K> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + (c >> 3) * 210;  // only 2-byte aligned: byte loads
        int idx0 = (int)(c & 7) * 32;
        float d = f16_bits_to_f32(ld_u16(b + 208));
        float s0 = __fmul_rn(d, s8_to_f(__ldg(b + 192 + idx0 / 16)));
        float s1 = __fmul_rn(d, s8_to_f(__ldg(b + 192 + idx0 / 16 + 1)));
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint32_t qh = __ldg(b + 128 + idx0 / 4 + i);
            uint32_t ql0 = __ldg(b + idx0 / 2 + 2 * i);
            uint32_t ql1 = __ldg(b + idx0 / 2 + 2 * i + 1);
            float s = i < 4 ? s0 : s1;
            const uint32_t q0 = (ql0 & 15u) | (((qh >> 0) & 3u) << 4);
            const uint32_t q1 = (ql0 >> 4) | (((qh >> 2) & 3u) << 4);
            const uint32_t q2 = (ql1 & 15u) | (((qh >> 4) & 3u) << 4);
            const uint32_t q3 = (ql1 >> 4) | (((qh >> 6) & 3u) << 4);
            o[4 * i + 0] = __fmul_rn(s, u2f_biased(q0, 32.0f));
            o[4 * i + 1] = __fmul_rn(s, u2f_biased(q1, 32.0f));
            o[4 * i + 2] = __fmul_rn(s, u2f_biased(q2, 32.0f));
            o[4 * i + 3] = __fmul_rn(s, u2f_biased(q3, 32.0f));
        }
    }
};

// Q5_0 / Q5_1 (crates/nn-gguf/src/dequant.rs:241-316): element 2j = low nibble of qs[j] with bit 2j
// of the 32-bit qh word as its fifth bit, element 2j+1 = high nibble with bit 2j+1.
template <>
struct Decode<NNQ_Q5_0> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + c * 22;
        float d = f16_bits_to_f32(ld_u16(b));
        uint32_t qh = (uint32_t)ld_u16(b + 2) | ((uint32_t)ld_u16(b + 4) << 16);
#pragma unroll
        for (int j = 0; j < 16; j++) {
            uint32_t q = __ldg(b + 6 + j);
            const uint32_t x0 = (q & 15u) | (((qh >> (2 * j)) & 1u) << 4);
            const uint32_t x1 = (q >> 4) | (((qh >> (2 * j + 1)) & 1u) << 4);
            o[2 * j] = __fmul_rn(d, u2f_biased(x0, 16.0f));
            o[2 * j + 1] = __fmul_rn(d, u2f_biased(x1, 16.0f));
        }
    }
};

template <>
struct Decode<NNQ_Q5_1> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + c * 24;
        float d = f16_bits_to_f32(ld_u16(b));
        float m = f16_bits_to_f32(ld_u16(b + 2));
        uint32_t qh = (uint32_t)ld_u16(b + 4) | ((uint32_t)ld_u16(b + 6) << 16);
#pragma unroll
        for (int j = 0; j < 16; j++) {
            uint32_t q = __ldg(b + 8 + j);
            uint32_t x0 = (q & 15u) | (((qh >> (2 * j)) & 1u) << 4);
            uint32_t x1 = (q >> 4) | (((qh >> (2 * j + 1)) & 1u) << 4);
            o[2 * j] = __fadd_rn(__fmul_rn(d, u2f(x0)), m);
            o[2 * j + 1] = __fadd_rn(__fmul_rn(d, u2f(x1)), m);
        }
    }
};

// Q2_K, nn-gguf variant (dequant.rs:476-512): flat element index; scale byte per 16 weights
// (low nibble scale, high nibble minimum); w = (d*sc)*q2 - dmin*m.
template <>
struct Decode<NNQ_Q2_K> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + (c >> 3) * 84;
        int idx0 = (int)(c & 7) * 32;
        float d = f16_bits_to_f32(ld_u16(b + 80));
        float dmin = f16_bits_to_f32(ld_u16(b + 82));
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t sb = __ldg(b + idx0 / 16 + h);
            float s = __fmul_rn(d, u2f(sb & 15u));
            float m = __fmul_rn(dmin, u2f(sb >> 4));
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t q = __ldg(b + 16 + idx0 / 4 + 4 * h + i);
#pragma unroll
                for (int t = 0; t < 4; t++)
                    o[16 * h + 4 * i + t] = __fsub_rn(__fmul_rn(s, u2f((q >> (2 * t)) & 3u)), m);
            }
        }
    }
};

// Q3_K, nn-gguf variant (dequant.rs:536-600): 16 six-bit scales (stored + 32), q3 = crumb | hmask bit << 2.
template <>
struct Decode<NNQ_Q3_K> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + (c >> 3) * 110;
        int idx0 = (int)(c & 7) * 32;
        float d = f16_bits_to_f32(ld_u16(b + 108));
        int k0 = idx0 / 16;   // even
        uint32_t lo = __ldg(b + 96 + k0 / 2);
        uint32_t hi = __ldg(b + 104 + k0 / 4);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int k = k0 + h;
            const uint32_t sc = ((lo >> (4 * h)) & 15u) | (((hi >> (2 * (k & 3))) & 3u) << 4);
            float s = __fmul_rn(d, u2f_biased(sc, 32.0f));
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t q = __ldg(b + 32 + idx0 / 4 + 4 * h + i);
                uint32_t hm = __ldg(b + idx0 / 8 + 2 * h + i / 2) >> (4 * (i & 1));
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const uint32_t q3 = ((q >> (2 * t)) & 3u) | (((hm >> t) & 1u) << 2);
                    o[16 * h + 4 * i + t] = __fmul_rn(s, u2f_biased(q3, 4.0f));
                }
            }
        }
    }
};

// Q5_K, nn-gguf variant (dequant.rs:614-684): scales packed as in the nn-gguf Q4_K, flat element
// index; q5 = nibble(qs[idx/2]) | bit(qh[idx/8], idx%8) << 4; w = (d*sc)*q5 - dmin*m.
template <>
struct Decode<NNQ_Q5_K> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + (c >> 3) * 176;   // 16-byte aligned blocks
        int j = (int)(c & 7);
        float d = f16_bits_to_f32(ld_u16(b));
        float dmin = f16_bits_to_f32(ld_u16(b + 2));
        const uint8_t *S = b + 4;
        uint32_t sc = ((__ldg(S + j / 2) >> (4 * (j & 1))) & 15u) | (((__ldg(S + 8 + j / 4) >> (2 * (j & 3))) & 3u) << 4);
        uint32_t mn = ((__ldg(S + 4 + j / 2) >> (4 * (j & 1))) & 15u) | (((__ldg(S + 10 + j / 4) >> (2 * (j & 3))) & 3u) << 4);
        float s = __fmul_rn(d, u2f(sc)), m = __fmul_rn(dmin, u2f(mn));
        uint32_t qh = __ldg(reinterpret_cast<const uint32_t *>(b + 16 + 4 * j));
        uint4 qs = __ldg(reinterpret_cast<const uint4 *>(b + 48 + 16 * j));
        uint32_t qw[4] = {qs.x, qs.y, qs.z, qs.w};
#pragma unroll
        for (int i = 0; i < 32; i++) {
            uint32_t q5 = ((qw[i / 8] >> (4 * (i & 7))) & 15u) | (((qh >> i) & 1u) << 4);
            o[i] = __fsub_rn(__fmul_rn(s, u2f(q5)), m);
        }
    }
};

template <>
struct Decode<NNQ_MXFP4_CORE> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint8_t *b = w + c * 17;
        float scale = mx_scale_core(__ldg(b));
#pragma unroll
        for (int j = 0; j < 16; j++) {
            uint32_t q = __ldg(b + 1 + j);
            o[2 * j] = e2m1_value(q & 15u, scale);
            o[2 * j + 1] = e2m1_value(q >> 4, scale);
        }
    }
};

template <>
struct Decode<NNQ_MXFP4_SPLIT> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *sc, int64_t c, float *o) {
        float scale = mx_scale_core(__ldg(sc + c));
        uint4 q = __ldg(reinterpret_cast<const uint4 *>(w + c * 16));
        uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int v = 0; v < 4; v++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t byte = (qw[v] >> (8 * i)) & 0xFFu;
                o[8 * v + 2 * i] = e2m1_value(byte & 15u, scale);
                o[8 * v + 2 * i + 1] = e2m1_value(byte >> 4, scale);
            }
    }
};

template <>
struct Decode<NNQ_MXFP4_GPTOSS> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *sc, int64_t c, float *o) {
        float scale = mx_scale_gptoss(__ldg(sc + c));
        uint4 q = __ldg(reinterpret_cast<const uint4 *>(w + c * 16));
        uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int v = 0; v < 4; v++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t byte = (qw[v] >> (8 * i)) & 0xFFu;
                o[8 * v + 2 * i] = e2m1_value(byte >> 4, scale);      // high nibble = even element
                o[8 * v + 2 * i + 1] = e2m1_value(byte & 15u, scale);
            }
    }
};

// unquantized weights: a "chunk" is 32 consecutive values
template <>
struct Decode<NNQ_F32_DENSE> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const float4 *p = reinterpret_cast<const float4 *>(w) + c * 8;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float4 v = __ldg(p + j);
            o[4 * j] = v.x; o[4 * j + 1] = v.y; o[4 * j + 2] = v.z; o[4 * j + 3] = v.w;
        }
    }
};

template <>
struct Decode<NNQ_BF16_DENSE> {
    static __device__ __forceinline__ void chunk(const uint8_t *w, const uint8_t *, int64_t c, float *o) {
        const uint4 *p = reinterpret_cast<const uint4 *>(w) + c * 4;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint4 v = __ldg(p + j);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                o[8 * j + 2 * i] = __uint_as_float(u[i] << 16);
                o[8 * j + 2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
            }
        }
    }
};

}  // namespace nnq
