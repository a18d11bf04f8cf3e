/*
 * CPU oracle for the block-quantized weight matmul path of alabsystems/nn.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It restates, on the CPU and in plain C, the
 * arithmetic of the reference's own CPU implementation so that the CUDA library
 * can be checked against it. It is never linked into, loaded by, or called from
 * the product library; only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg use it.
 *
 * Parity status: PINNED. The reference is a Rust workspace and cannot be built in
 * this environment (no cargo/rustc), so the oracle is pinned against every
 * known-answer test the reference carries for this path (replayed by
 * tests/test_oracle_golden.py, each citing the reference test it replays).
 *
 * Each function cites the reference file:line it follows (paths relative to the
 * reference repository root). All arithmetic is IEEE f32, compiled with
 * -ffp-contract=off so that "a*b - c" is two roundings exactly as the Rust
 * source evaluates it. f16 -> f32 is the exact IEEE widening that
 * half::f16::to_f32 performs.
 *
 * Build: see oracle/Makefile  (gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* scalar helpers                                                            */
/* ------------------------------------------------------------------------- */

/* Exact binary16 -> binary32 widening (subnormals, inf and NaN included);
 * the same mapping as half::f16::to_f32 used at
 * crates/nn-gguf/src/dequant.rs:187,345-346,428. */
static float f16_bits_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            /* subnormal: normalise */
            int shift = 0;
            while ((man & 0x400u) == 0) {
                man <<= 1;
                shift++;
            }
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + (127 - 15)) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static float f16_at(const uint8_t *p) {
    return f16_bits_to_f32((uint16_t)(p[0] | ((uint16_t)p[1] << 8)));
}

ORC_API float orc_f16_to_f32(uint16_t h) { return f16_bits_to_f32(h); }

/* Number of complete blocks to decode: the element count fixes it unless the
 * byte buffer is short, in which case it is clamped to the whole blocks present.
 * crates/nn-gguf/src/dequant.rs:123-139 (validate_dequant_input). */
static size_t usable_blocks(size_t nbytes, size_t num_elements, size_t block_elems,
                            size_t block_bytes) {
    size_t nb = num_elements / block_elems;
    size_t need = nb * block_bytes;
    if (nb != 0 && need / nb != block_bytes) need = SIZE_MAX; /* saturating_mul */
    return nbytes < need ? nbytes / block_bytes : nb;
}

/* ------------------------------------------------------------------------- */
/* block dequantizers, nn-gguf layouts                                       */
/* ------------------------------------------------------------------------- */

/* Q4_0: 18 B / 32 weights, w = d * (nibble - 8); low nibble = even element.
 * crates/nn-gguf/src/dequant.rs:148-169 (same arithmetic duplicated at
 * crates/nn-core/src/dyn_tensor/quantized.rs:184-203). */
ORC_API size_t orc_dequant_q4_0(const uint8_t *data, size_t nbytes, size_t num_elements,
                                float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 32, 18);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 18;
        float d = f16_at(blk);
        for (int j = 0; j < 16; j++) {
            int lo = (int)(blk[2 + j] & 0x0F) - 8;
            int hi = (int)(blk[2 + j] >> 4) - 8;
            out[b * 32 + 2 * j] = d * (float)lo;
            out[b * 32 + 2 * j + 1] = d * (float)hi;
        }
    }
    return nb * 32;
}

/* Q4_1: 20 B / 32 weights, w = d * nibble + m.
 * crates/nn-core/src/dyn_tensor/quantized.rs:210-230. */
ORC_API size_t orc_dequant_q4_1(const uint8_t *data, size_t nbytes, size_t num_elements,
                                float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 32, 20);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 20;
        float d = f16_at(blk);
        float m = f16_at(blk + 2);
        for (int j = 0; j < 16; j++) {
            float lo = (float)(blk[4 + j] & 0x0F);
            float hi = (float)(blk[4 + j] >> 4);
            out[b * 32 + 2 * j] = d * lo + m;
            out[b * 32 + 2 * j + 1] = d * hi + m;
        }
    }
    return nb * 32;
}

/* Q8_0: 34 B / 32 weights, w = d * (int8)q.
 * crates/nn-gguf/src/dequant.rs:178-196. */
ORC_API size_t orc_dequant_q8_0(const uint8_t *data, size_t nbytes, size_t num_elements,
                                float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 32, 34);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 34;
        float d = f16_at(blk);
        for (int j = 0; j < 32; j++) out[b * 32 + j] = d * (float)(int8_t)blk[2 + j];
    }
    return nb * 32;
}

/* Q4_K, nn-gguf variant: 144 B / 256 weights.
 *   [0,2) d  [2,4) dmin  [4,16) S[12]  [16,144) qs[128]
 *   sc_j = lo4(S[j/2], j%2) | crumb(S[8 + j/4], j%4) << 4
 *   m_j  = lo4(S[4 + j/2], j%2) | crumb(S[10 + j/4], j%4) << 4
 *   element 32j+2i   = low  nibble of qs[16j+i]
 *   element 32j+2i+1 = high nibble of qs[16j+i]
 *   w = (d*sc_j)*q - (dmin*m_j)
 * crates/nn-gguf/src/dequant.rs:335-398. */
static void q4k_gguf_scales(const uint8_t *S, uint8_t sc[8], uint8_t mn[8]) {
    for (int j = 0; j < 8; j++) {
        sc[j] = (uint8_t)((S[j / 2] >> (4 * (j % 2))) & 0x0F);
        mn[j] = (uint8_t)((S[4 + j / 2] >> (4 * (j % 2))) & 0x0F);
    }
    for (int j = 0; j < 4; j++) {
        sc[j] |= (uint8_t)(((S[8] >> (2 * j)) & 3) << 4);
        sc[4 + j] |= (uint8_t)(((S[9] >> (2 * j)) & 3) << 4);
        mn[j] |= (uint8_t)(((S[10] >> (2 * j)) & 3) << 4);
        mn[4 + j] |= (uint8_t)(((S[11] >> (2 * j)) & 3) << 4);
    }
}

ORC_API size_t orc_dequant_q4_k(const uint8_t *data, size_t nbytes, size_t num_elements,
                                float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 256, 144);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 144;
        float d = f16_at(blk);
        float dmin = f16_at(blk + 2);
        uint8_t sc[8], mn[8];
        q4k_gguf_scales(blk + 4, sc, mn);
        const uint8_t *qs = blk + 16;
        float *o = out + b * 256;
        for (int j = 0; j < 8; j++) {
            float s = d * (float)sc[j];
            float m = dmin * (float)mn[j];
            for (int i = 0; i < 16; i++) {
                uint8_t byte = qs[j * 16 + i];
                o[32 * j + 2 * i] = s * (float)(byte & 0x0F) - m;
                o[32 * j + 2 * i + 1] = s * (float)(byte >> 4) - m;
            }
        }
    }
    return nb * 256;
}

/* Q4_K, nn-core BlockQ4K variant over the same 144-byte block: GGML's scale
 * packing (j<4: S[j]&63 / S[j+4]&63; j>=4: split nibbles + top crumbs) and
 * 64-wide groups whose first 32 elements are the low nibbles and next 32 the
 * high nibbles of qs[32g .. 32g+32).
 * crates/nn-core/src/layers/quantized/linear.rs:63-92 (dequantize),
 * :166-176 (get_scale_min_k4). */
static void q4k_ggml_scale_min(int j, const uint8_t *S, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = S[j] & 63;
        *mn = S[j + 4] & 63;
    } else {
        *sc = (uint8_t)((S[j + 4] & 0x0F) | ((S[j - 4] >> 6) << 4));
        *mn = (uint8_t)((S[j + 4] >> 4) | ((S[j] >> 6) << 4));
    }
}

ORC_API size_t orc_dequant_q4_k_ggml(const uint8_t *data, size_t nbytes, size_t num_elements,
                                     float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 256, 144);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 144;
        float d = f16_at(blk);
        float dmin = f16_at(blk + 2);
        const uint8_t *S = blk + 4;
        const uint8_t *qs = blk + 16;
        float *o = out + b * 256;
        for (int g = 0; g < 4; g++) {
            uint8_t sc1, m1, sc2, m2;
            q4k_ggml_scale_min(2 * g, S, &sc1, &m1);
            q4k_ggml_scale_min(2 * g + 1, S, &sc2, &m2);
            float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
            float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
            for (int i = 0; i < 32; i++) o[64 * g + i] = d1 * (float)(qs[32 * g + i] & 0x0F) - mm1;
            for (int i = 0; i < 32; i++) o[64 * g + 32 + i] = d2 * (float)(qs[32 * g + i] >> 4) - mm2;
        }
    }
    return nb * 256;
}

/* Q6_K, nn-gguf variant: 210 B / 256 weights, flat element index.
 *   [0,128) ql  [128,192) qh  [192,208) sc[16] (int8)  [208,210) d
 *   q6 = nibble(ql[idx/2], idx%2) | crumb(qh[idx/4], idx%4) << 4
 *   w = (d * sc[idx/16]) * (q6 - 32)
 * crates/nn-gguf/src/dequant.rs:415-459. */
ORC_API size_t orc_dequant_q6_k(const uint8_t *data, size_t nbytes, size_t num_elements,
                                float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 256, 210);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 210;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *sc = (const int8_t *)(blk + 192);
        float d = f16_at(blk + 208);
        for (int idx = 0; idx < 256; idx++) {
            uint8_t lo4 = (uint8_t)((ql[idx / 2] >> (4 * (idx % 2))) & 0x0F);
            uint8_t hi2 = (uint8_t)((qh[idx / 4] >> (2 * (idx % 4))) & 0x03);
            int q6 = (int)(lo4 | (hi2 << 4));
            out[b * 256 + idx] = d * (float)sc[idx / 16] * (float)(q6 - 32);
        }
    }
    return nb * 256;
}

/* Q5_0: 22 B / 32 weights. [0,2) d  [2,6) qh (u32 LE)  [6,22) qs
 *   element 2j = low nibble of qs[j] | bit 2j of qh << 4; element 2j+1 = high nibble | bit 2j+1 << 4
 *   w = d * (q5 - 16)
 * crates/nn-gguf/src/dequant.rs:241-271. */
ORC_API size_t orc_dequant_q5_0(const uint8_t *data, size_t nbytes, size_t num_elements,
                                float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 32, 22);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 22;
        float d = f16_at(blk);
        uint32_t qh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24);
        for (int j = 0; j < 16; j++) {
            int x0 = (int)((blk[6 + j] & 0x0F) | (((qh >> (2 * j)) & 1u) << 4)) - 16;
            int x1 = (int)((blk[6 + j] >> 4) | (((qh >> (2 * j + 1)) & 1u) << 4)) - 16;
            out[b * 32 + 2 * j] = d * (float)x0;
            out[b * 32 + 2 * j + 1] = d * (float)x1;
        }
    }
    return nb * 32;
}

/* Q5_1: 24 B / 32 weights. [0,2) d  [2,4) m  [4,8) qh  [8,24) qs; w = d * q5 + m.
 * crates/nn-gguf/src/dequant.rs:285-316. */
ORC_API size_t orc_dequant_q5_1(const uint8_t *data, size_t nbytes, size_t num_elements,
                                float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 32, 24);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 24;
        float d = f16_at(blk), m = f16_at(blk + 2);
        uint32_t qh = (uint32_t)blk[4] | ((uint32_t)blk[5] << 8) | ((uint32_t)blk[6] << 16) | ((uint32_t)blk[7] << 24);
        for (int j = 0; j < 16; j++) {
            uint32_t x0 = (uint32_t)(blk[8 + j] & 0x0F) | (((qh >> (2 * j)) & 1u) << 4);
            uint32_t x1 = (uint32_t)(blk[8 + j] >> 4) | (((qh >> (2 * j + 1)) & 1u) << 4);
            out[b * 32 + 2 * j] = d * (float)x0 + m;
            out[b * 32 + 2 * j + 1] = d * (float)x1 + m;
        }
    }
    return nb * 32;
}

/* Q2_K, nn-gguf variant: 84 B / 256 weights, flat element index.
 *   [0,16) scales (low nibble = scale, high nibble = min, per 16 weights)  [16,80) qs  [80,82) d  [82,84) dmin
 *   q2 = crumb(qs[idx/4], idx%4);  w = (d * sc) * q2 - dmin * m
 * crates/nn-gguf/src/dequant.rs:476-512. */
ORC_API size_t orc_dequant_q2_k(const uint8_t *data, size_t nbytes, size_t num_elements,
                                float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 256, 84);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 84;
        const uint8_t *qs = blk + 16;
        float d = f16_at(blk + 80), dmin = f16_at(blk + 82);
        for (int idx = 0; idx < 256; idx++) {
            float sc = (float)(blk[idx / 16] & 0x0F);
            float m = (float)(blk[idx / 16] >> 4);
            float q2 = (float)((qs[idx / 4] >> ((idx % 4) * 2)) & 0x03);
            out[b * 256 + idx] = d * sc * q2 - dmin * m;
        }
    }
    return nb * 256;
}

/* Q3_K, nn-gguf variant: 110 B / 256 weights, flat element index.
 *   [0,32) hmask  [32,96) qs  [96,108) S[12]  [108,110) d
 *   scale_k = (lo4(S[k/2], k%2) | crumb(S[8 + k/4], k%4) << 4) - 32   (16 scales, one per 16 weights)
 *   q3 = crumb(qs[idx/4], idx%4) | bit(hmask[idx/8], idx%8) << 2;  w = (d * scale) * (q3 - 4)
 * crates/nn-gguf/src/dequant.rs:536-600. */
ORC_API size_t orc_dequant_q3_k(const uint8_t *data, size_t nbytes, size_t num_elements,
                                float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 256, 110);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 110;
        const uint8_t *hmask = blk, *qs = blk + 32, *S = blk + 96;
        float d = f16_at(blk + 108);
        for (int k = 0; k < 16; k++) {
            int lo4 = (S[k / 2] >> (4 * (k % 2))) & 0x0F;
            int hi2 = (S[8 + k / 4] >> (2 * (k % 4))) & 0x03;
            float sc = d * (float)((lo4 | (hi2 << 4)) - 32);
            for (int i = 0; i < 16; i++) {
                int idx = 16 * k + i;
                int q3 = ((qs[idx / 4] >> ((idx % 4) * 2)) & 0x03) | (((hmask[idx / 8] >> (idx % 8)) & 1) << 2);
                out[b * 256 + idx] = sc * (float)(q3 - 4);
            }
        }
    }
    return nb * 256;
}

/* Q5_K, nn-gguf variant: 176 B / 256 weights, flat element index.
 *   [0,2) d  [2,4) dmin  [4,16) S[12] (packed as in the nn-gguf Q4_K)  [16,48) qh  [48,176) qs
 *   q5 = nibble(qs[idx/2], idx%2) | bit(qh[idx/8], idx%8) << 4;  w = (d*sc_j)*q5 - dmin*m_j, j = idx/32
 * crates/nn-gguf/src/dequant.rs:614-684. */
ORC_API size_t orc_dequant_q5_k(const uint8_t *data, size_t nbytes, size_t num_elements,
                                float *out) {
    size_t nb = usable_blocks(nbytes, num_elements, 256, 176);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 176;
        const uint8_t *qh = blk + 16, *qs = blk + 48;
        float d = f16_at(blk), dmin = f16_at(blk + 2);
        uint8_t sc[8], mn[8];
        q4k_gguf_scales(blk + 4, sc, mn);
        for (int j = 0; j < 8; j++) {
            float s = d * (float)sc[j], m = dmin * (float)mn[j];
            for (int i = 0; i < 32; i++) {
                int idx = 32 * j + i;
                int q5 = ((qs[idx / 2] >> (4 * (idx % 2))) & 0x0F) | (((qh[idx / 8] >> (idx % 8)) & 1) << 4);
                out[b * 256 + idx] = s * (float)q5 - m;
            }
        }
    }
    return nb * 256;
}

/* ------------------------------------------------------------------------- */
/* MXFP4 decoders                                                            */
/* ------------------------------------------------------------------------- */

/* E2M1 magnitudes for code & 7; bit 3 is the sign (code 8 is -0.0).
 * crates/nn-core/src/layers/quantized/mxfp4.rs:60,
 * crates/nn-gptoss/src/quantize.rs:28-45. */
static const float E2M1_MAG[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* nn-core Mxfp4Block: 17 B = [shared_exp][16 packed]; low nibble = even element;
 * scale = (f32)(2.0f64 ^ (e - 127)), so e = 0 gives the f32 subnormal 2^-127;
 * value = magnitude * scale, negated when the sign bit is set.
 * crates/nn-core/src/layers/quantized/mxfp4.rs:124-134 (decode_e1m2),
 * :177-182 (block_scale_from_exp), :226-242 (dequantize_block). */
ORC_API float orc_mxfp4_core_scale(uint8_t e) { return (float)ldexp(1.0, (int)e - 127); }

ORC_API void orc_dequant_mxfp4_core(const uint8_t *blocks, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 17;
        float scale = orc_mxfp4_core_scale(blk[0]);
        for (int i = 0; i < 32; i++) {
            uint8_t code = (i % 2 == 0) ? (blk[1 + i / 2] & 0x0F) : (blk[1 + i / 2] >> 4);
            float v = E2M1_MAG[code & 7] * scale;
            out[b * 32 + i] = (code & 8) ? -v : v;
        }
    }
}

/* nn-gptoss Mxfp4Tensor: data[n/2] + scales[n/32]; HIGH nibble = even element;
 * scale = f32::from_bits(e << 23), except e = 0 -> 2^-126; value = LUT[code]*scale
 * with a signed 16-entry table (so code 8 yields -0.0 * scale).
 * crates/nn-gptoss/src/quantize.rs:84-90 (decode_e8m0_scale), :167-188. */
ORC_API float orc_mxfp4_gptoss_scale(uint8_t e) {
    uint32_t bits = e == 0 ? 0x00800000u : ((uint32_t)e << 23);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

ORC_API void orc_dequant_mxfp4_gptoss(const uint8_t *data, const uint8_t *scales, size_t nblocks,
                                      float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        float scale = orc_mxfp4_gptoss_scale(scales[b]);
        for (int p = 0; p < 16; p++) {
            uint8_t byte = data[b * 16 + p];
            uint8_t hi = byte >> 4, lo = byte & 0x0F;
            float vh = (hi & 8) ? -E2M1_MAG[hi & 7] : E2M1_MAG[hi & 7];
            float vl = (lo & 8) ? -E2M1_MAG[lo & 7] : E2M1_MAG[lo & 7];
            out[b * 32 + 2 * p] = vh * scale;
            out[b * 32 + 2 * p + 1] = vl * scale;
        }
    }
}

/* Split K-blocked layout of the reference's GPU kernel contract:
 * packed_w[N][K/2] (low nibble = even k), shared_exp[N][K/32],
 * scale = exp2(float(e - 127)).
 * crates/nn-metal/src/mxfp4_gemm_msl.rs:47-61 (buffers), :124-145 (decode). */
ORC_API void orc_dequant_mxfp4_split(const uint8_t *packed, const uint8_t *exps, size_t n_rows,
                                     size_t k, float *out) {
    size_t bpr = k / 32;
    for (size_t r = 0; r < n_rows; r++) {
        for (size_t b = 0; b < bpr; b++) {
            float scale = exp2f((float)((int)exps[r * bpr + b] - 127));
            for (int j = 0; j < 16; j++) {
                uint8_t byte = packed[r * (k / 2) + b * 16 + j];
                uint8_t lo = byte & 0x0F, hi = byte >> 4;
                float vl = (lo & 8) ? -E2M1_MAG[lo & 7] : E2M1_MAG[lo & 7];
                float vh = (hi & 8) ? -E2M1_MAG[hi & 7] : E2M1_MAG[hi & 7];
                out[r * k + b * 32 + 2 * j] = vl * scale;
                out[r * k + b * 32 + 2 * j + 1] = vh * scale;
            }
        }
    }
}

/* The reference GPU kernel's own product: one output per (row, col), sequential
 * f32 accumulation in k order, "acc += w * a" with w = lut * scale, bias last.
 * crates/nn-metal/src/mxfp4_gemm_msl.rs:94-149. */
ORC_API void orc_mxfp4_split_linear(const float *a, const uint8_t *packed, const uint8_t *exps,
                                    const float *bias, float *c, size_t m, size_t k, size_t n) {
    size_t bpr = k / 32;
#pragma omp parallel for schedule(static)
    for (long long col = 0; col < (long long)n; col++) {
        for (size_t row = 0; row < m; row++) {
            float acc = 0.0f;
            for (size_t blk = 0; blk < bpr; blk++) {
                float scale = exp2f((float)((int)exps[col * bpr + blk] - 127));
                for (int j = 0; j < 16; j++) {
                    uint8_t byte = packed[col * (k / 2) + blk * 16 + j];
                    uint8_t lo = byte & 0x0F, hi = byte >> 4;
                    float wl = ((lo & 8) ? -E2M1_MAG[lo & 7] : E2M1_MAG[lo & 7]) * scale;
                    float wh = ((hi & 8) ? -E2M1_MAG[hi & 7] : E2M1_MAG[hi & 7]) * scale;
                    acc += wl * a[row * k + blk * 32 + 2 * j];
                    acc += wh * a[row * k + blk * 32 + 2 * j + 1];
                }
            }
            if (bias) acc += bias[col];
            c[row * n + col] = acc;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* fused quantized matmul of nn-core (Q4_0 / Q8_0)                           */
/* ------------------------------------------------------------------------- */

/* One 32-element block: acc starts at 0, acc += x[j] * (d * q_j) in j order.
 * crates/nn-core/src/dyn_tensor/quantized_matmul.rs:152-187. */
static float dot_block_q8_0(const uint8_t *blk, const float *x) {
    float d = f16_at(blk);
    float acc = 0.0f;
    for (int j = 0; j < 32; j++) acc += x[j] * (d * (float)(int8_t)blk[2 + j]);
    return acc;
}

static float dot_block_q4_0(const uint8_t *blk, const float *x) {
    float d = f16_at(blk);
    float acc = 0.0f;
    for (int j = 0; j < 16; j++) {
        int lo = (int)(blk[2 + j] & 0x0F) - 8;
        int hi = (int)(blk[2 + j] >> 4) - 8;
        acc += x[2 * j] * (d * (float)lo);
        acc += x[2 * j + 1] * (d * (float)hi);
    }
    return acc;
}

/* y[r, n] = sum over blocks of the block dot (row accumulator += block
 * accumulator), rows of x taken in order, then the optional bias broadcast add.
 * fmt: 0 = Q4_0, 2 = Q8_0.
 * crates/nn-core/src/dyn_tensor/quantized_matmul.rs:191-272 (core loops),
 * :367-405 (quantized_linear bias add). */
ORC_API int orc_quantized_linear(int fmt, const float *x, const uint8_t *w, const float *bias,
                                 float *y, size_t rows, size_t n, size_t k) {
    size_t bb = fmt == 0 ? 18 : 34;
    if (fmt != 0 && fmt != 2) return -1;
    size_t bpr = k / 32;
#pragma omp parallel for schedule(static)
    for (long long oc = 0; oc < (long long)n; oc++) {
        for (size_t r = 0; r < rows; r++) {
            const float *xr = x + r * k;
            float acc = 0.0f;
            for (size_t b = 0; b < bpr; b++) {
                const uint8_t *blk = w + ((size_t)oc * bpr + b) * bb;
                acc += fmt == 0 ? dot_block_q4_0(blk, xr + b * 32) : dot_block_q8_0(blk, xr + b * 32);
            }
            if (bias) acc = acc + bias[oc];
            y[r * n + oc] = acc;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* dense f32 product on dequantized weights                                  */
/* ------------------------------------------------------------------------- */

/* Sequential-K f32 product y = x * W^T (+ bias): the tolerance-pinned stand-in
 * for the third-party sgemm behind DynTensor::matmul
 * (crates/nn-core/src/dyn_tensor/ops/matmul.rs:42-52), with Linear's bias
 * broadcast add (crates/nn-core/src/layers/core_layers.rs:131-141). */
ORC_API void orc_linear_f32(const float *x, const float *w, const float *bias, float *y,
                            size_t m, size_t n, size_t k) {
#pragma omp parallel for schedule(static)
    for (long long o = 0; o < (long long)n; o++) {
        for (size_t r = 0; r < m; r++) {
            float acc = 0.0f;
            for (size_t i = 0; i < k; i++) acc += x[r * k + i] * w[(size_t)o * k + i];
            if (bias) acc = acc + bias[o];
            y[r * n + o] = acc;
        }
    }
}

/* Same product accumulated in f64: used only to bound the f32 oracle's own
 * rounding error when a test sets its tolerance. */
ORC_API void orc_linear_f64(const float *x, const float *w, const float *bias, double *y,
                            size_t m, size_t n, size_t k) {
#pragma omp parallel for schedule(static)
    for (long long o = 0; o < (long long)n; o++) {
        for (size_t r = 0; r < m; r++) {
            double acc = 0.0;
            for (size_t i = 0; i < k; i++) acc += (double)x[r * k + i] * (double)w[(size_t)o * k + i];
            if (bias) acc += (double)bias[o];
            y[r * n + o] = acc;
        }
    }
}

/* Sum of |x_k * w_k| per output: the natural scale of the forward error of a
 * dot product; tests express their element-wise bound relative to it. */
ORC_API void orc_linear_abs(const float *x, const float *w, double *y, size_t m, size_t n,
                            size_t k) {
#pragma omp parallel for schedule(static)
    for (long long o = 0; o < (long long)n; o++) {
        for (size_t r = 0; r < m; r++) {
            double acc = 0.0;
            for (size_t i = 0; i < k; i++) acc += fabs((double)x[r * k + i] * (double)w[(size_t)o * k + i]);
            y[r * n + o] = acc;
        }
    }
}

/* nn-cpu row dot: 8-wide FMA accumulation, horizontal add (hi+lo 128, movehdup,
 * movehl), scalar tail; scalar loop when AVX2/FMA are absent.
 * crates/nn-cpu/src/simd_gemv.rs:156-205 (AVX2), :31-51 (scalar);
 * crates/nn-cpu/src/simd_linear.rs:190-225 (the same dot used by linear()). */
#if defined(__x86_64__)
__attribute__((target("avx2,fma"))) static float dot_avx2(const float *a, const float *b, size_t k) {
    size_t chunks = k / 8;
    __m256 acc = _mm256_setzero_ps();
    for (size_t c = 0; c < chunks; c++)
        acc = _mm256_fmadd_ps(_mm256_loadu_ps(a + 8 * c), _mm256_loadu_ps(b + 8 * c), acc);
    __m128 hi = _mm256_extractf128_ps(acc, 1);
    __m128 lo = _mm256_castps256_ps128(acc);
    __m128 s4 = _mm_add_ps(lo, hi);
    __m128 sh = _mm_movehdup_ps(s4);
    __m128 s2 = _mm_add_ps(s4, sh);
    __m128 sh2 = _mm_movehl_ps(s2, s2);
    float r = _mm_cvtss_f32(_mm_add_ss(s2, sh2));
    for (size_t i = chunks * 8; i < k; i++) r += a[i] * b[i];
    return r;
}
#endif

static float dot_scalar(const float *a, const float *b, size_t k) {
    float acc = 0.0f;
    for (size_t i = 0; i < k; i++) acc += a[i] * b[i];
    return acc;
}

static int have_avx2(void) {
#if defined(__x86_64__)
    return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
#else
    return 0;
#endif
}

/* y[r, o] = dot(x[r], w[o]) (+ bias[o]) with nn-cpu's dot; rows of W split over
 * OpenMP threads when threads > 1 (the reference itself is single-threaded).
 * crates/nn-cpu/src/simd_linear.rs:254-292. */
ORC_API void orc_nncpu_linear(const float *x, const float *w, const float *bias, float *y,
                              size_t m, size_t n, size_t k, int threads) {
    int avx = have_avx2();
    (void)avx;
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
    for (long long o = 0; o < (long long)n; o++) {
        for (size_t r = 0; r < m; r++) {
            float v;
#if defined(__x86_64__)
            v = avx ? dot_avx2(x + r * k, w + (size_t)o * k, k) : dot_scalar(x + r * k, w + (size_t)o * k, k);
#else
            v = dot_scalar(x + r * k, w + (size_t)o * k, k);
#endif
            if (bias) v = v + bias[o];
            y[r * n + o] = v;
        }
    }
}

ORC_API int orc_have_avx2(void) { return have_avx2(); }

/* ------------------------------------------------------------------------- */
/* f32 -> block encoders                                                     */
/* ------------------------------------------------------------------------- */

/* binary32 -> binary16, round to nearest even, overflow to infinity, NaN kept quiet:
 * half::f16::from_f32 as used at crates/nn-core/src/layers/quantized/linear.rs:137-138. */
static uint16_t f32_to_f16_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t exp = (x >> 23) & 0xFFu, man = x & 0x7FFFFFu;
    if (exp == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? (0x0200u | (man >> 13)) : 0));
    int e = (int)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return sign;                 /* below half of the smallest subnormal */
        man |= 0x800000u;
        int shift = 14 - e;                       /* 14 .. 24 */
        uint32_t h = man >> shift, rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1))) h++;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((uint32_t)e << 10) | (man >> 13), rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h++;   /* a carry into the exponent is correct */
    return (uint16_t)(sign | h);
}

ORC_API uint16_t orc_f32_to_f16(float f) { return f32_to_f16_bits(f); }

/* nearest_int (linear.rs:178-192): round half away from zero; non-finite or outside i32 is an error. */
static int q4k_nearest_int(float v, int *err) {
    if (!isfinite(v)) { *err = 1; return 0; }
    float r = roundf(v);
    if (r < -2147483648.0f || r > 2147483648.0f) { *err = 1; return 0; }
    if (r >= 2147483648.0f) return INT32_MAX;     /* `as i32` saturates */
    return (int)r;
}

/* f32::min / f32::max folds of the reference: NaN operands are ignored, ties keep the accumulator. */
static float fold_min(float acc, float v) { return v < acc ? v : acc; }
static float fold_max(float acc, float v) { return v > acc ? v : acc; }

/* make_qkx1_quants(nmax, ntry, x[32]) (linear.rs:195-254): (scale, min) of one sub-block. */
static void q4k_make_qkx1(int nmax, int ntry, const float *x, float *scale_out, float *min_out, int *err) {
    const int n = 32;
    uint8_t l[32] = {0};
    float mn = INFINITY, mx = -INFINITY;
    for (int i = 0; i < n; i++) { mn = fold_min(mn, x[i]); mx = fold_max(mx, x[i]); }
    if (mx == mn) {
        if (mn >= 0.0f) { *scale_out = nmax > 0 ? mn / (float)nmax : 0.0f; *min_out = 0.0f; }
        else { *scale_out = 0.0f; *min_out = -mn; }
        return;
    }
    float min = fold_min(mn, 0.0f);
    float iscale = (float)nmax / (mx - min);
    float scale = 1.0f / iscale;
    for (int t = 0; t < ntry; t++) {
        float sumlx = 0.0f;
        int suml2 = 0, changed = 0;
        for (int i = 0; i < n; i++) {
            int li = q4k_nearest_int(iscale * (x[i] - min), err);
            if (*err) return;
            li = li < 0 ? 0 : (li > nmax ? nmax : li);
            if ((uint8_t)li != l[i]) { l[i] = (uint8_t)li; changed = 1; }
            sumlx += (x[i] - min) * (float)li;
            suml2 += li * li;
        }
        if (suml2 == 0) { *scale_out = 0.0f; *min_out = 0.0f; return; }
        scale = sumlx / (float)suml2;
        if (scale == 0.0f) { *scale_out = 0.0f; *min_out = -min; return; }
        float sum = 0.0f;
        for (int i = 0; i < n; i++) sum += x[i] - scale * (float)l[i];
        min = fold_min(sum / (float)n, 0.0f);
        iscale = 1.0f / scale;
        if (!changed) break;
    }
    *scale_out = scale;
    *min_out = -min;
}

/* BlockQ4K::quantize (linear.rs:95-162) over a flat f32 buffer padded with zeros to whole
 * 256-weight blocks as QLinear::from_linear does (linear.rs:318-336). Output: 144-byte blocks
 * in nn-core's element order and scale packing (format code 4). Returns the number of blocks
 * written, or -1 when the reference returns ValueOutOfRange. */
ORC_API long long orc_quantize_q4_k_ggml(const float *src, size_t num_elements, uint8_t *out) {
    size_t nb = (num_elements + 255) / 256;
    for (size_t b = 0; b < nb; b++) {
        float v[256];
        for (int i = 0; i < 256; i++) v[i] = b * 256 + i < num_elements ? src[b * 256 + i] : 0.0f;
        uint8_t *blk = out + b * 144, *S = blk + 4, *qs = blk + 16;
        memset(blk, 0, 144);
        float ss[8], sm[8];
        int err = 0;
        for (int j = 0; j < 8; j++) {
            q4k_make_qkx1(15, 5, v + 32 * j, &ss[j], &sm[j], &err);
            if (err) return -1;
        }
        float max_scale = 0.0f, max_min = 0.0f;
        for (int j = 0; j < 8; j++) { max_scale = fold_max(max_scale, ss[j]); max_min = fold_max(max_min, sm[j]); }
        float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
        float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
        uint8_t LS[8], LM[8];
        for (int j = 0; j < 8; j++) {
            int a = q4k_nearest_int(inv_scale * ss[j], &err), c = q4k_nearest_int(inv_min * sm[j], &err);
            if (err) return -1;
            uint8_t ls = (uint8_t)a, lm = (uint8_t)c;     /* `as u8` keeps the low byte */
            ls = ls < 63 ? ls : 63;
            lm = lm < 63 ? lm : 63;
            LS[j] = ls; LM[j] = lm;
            if (j < 4) { S[j] = ls; S[j + 4] = lm; }
            else {
                S[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                S[j - 4] |= (uint8_t)((ls >> 4) << 6);
                S[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        uint16_t dh = f32_to_f16_bits(max_scale / 63.0f), mh = f32_to_f16_bits(max_min / 63.0f);
        blk[0] = (uint8_t)dh; blk[1] = (uint8_t)(dh >> 8); blk[2] = (uint8_t)mh; blk[3] = (uint8_t)(mh >> 8);
        uint8_t l[256] = {0};
        for (int j = 0; j < 8; j++) {
            float bd = f16_bits_to_f32(dh) * (float)LS[j];
            if (bd != 0.0f) {
                float bm = f16_bits_to_f32(mh) * (float)LM[j];
                for (int i = 0; i < 32; i++) {
                    int q = q4k_nearest_int((v[32 * j + i] + bm) / bd, &err);
                    if (err) return -1;
                    l[32 * j + i] = (uint8_t)(q < 0 ? 0 : (q > 15 ? 15 : q));
                }
            }
        }
        for (int j = 0; j < 256; j += 64)
            for (int k = 0; k < 32; k++) qs[j / 2 + k] = (uint8_t)(l[j + k] | (l[j + k + 32] << 4));
    }
    return (long long)nb;
}

/* Nearest E2M1 magnitude by minimum distance, first wins on ties
 * (encode_e1m2, mxfp4.rs:94-117; quantize_to_fp4, crates/nn-gptoss/src/quantize.rs:93-116). */
static uint8_t nearest_e2m1(float abs_scaled) {
    uint8_t best = 0;
    float best_dist = 3.40282347e+38f;
    for (uint8_t i = 0; i < 8; i++) {
        float dist = fabsf(abs_scaled - E2M1_MAG[i]);
        if (dist < best_dist) { best_dist = dist; best = i; }
    }
    return best;
}

/* quantize_tensor / quantize_block (mxfp4.rs:183-207,307-329) into 17-byte blocks (format code 6):
 * shared exponent = clamp(ceil(log2(max|v| / 6)) + 127, 0, 254), 0 for an all-zero block; the tail
 * block is padded with zeros. Returns the number of blocks, or -1 for a non-finite input. */
ORC_API long long orc_quantize_mxfp4_core(const float *src, size_t num_elements, uint8_t *out) {
    size_t nb = (num_elements + 31) / 32;
    for (size_t b = 0; b < nb; b++) {
        float v[32];
        for (int i = 0; i < 32; i++) {
            v[i] = b * 32 + i < num_elements ? src[b * 32 + i] : 0.0f;
            if (!isfinite(v[i])) return -1;
        }
        float max_abs = 0.0f;
        for (int i = 0; i < 32; i++) { float a = fabsf(v[i]); if (a > max_abs) max_abs = a; }
        uint8_t e = 0;
        if (max_abs != 0.0f) {
            int eb = (int)ceilf(log2f(max_abs / 6.0f)) + 127;
            e = (uint8_t)(eb < 0 ? 0 : (eb > 254 ? 254 : eb));
        }
        float scale = orc_mxfp4_core_scale(e);
        uint8_t *blk = out + b * 17;
        memset(blk, 0, 17);
        blk[0] = e;
        for (int i = 0; i < 32; i++) {
            uint8_t code = 0;
            if (!(v[i] == 0.0f || scale == 0.0f))
                code = (uint8_t)((v[i] < 0.0f ? 8 : 0) | nearest_e2m1(fabsf(v[i]) / scale));
            blk[1 + i / 2] |= (uint8_t)(i % 2 == 0 ? code : code << 4);
        }
    }
    return (long long)nb;
}

/* Mxfp4Tensor::quantize (crates/nn-gptoss/src/quantize.rs:64-153) into data[nb*16] + scales[nb]
 * (format code 8): scale byte = biased exponent of max|v| minus 2 (0 for zero / subnormal maxima,
 * at most 254), non-finite values are skipped in the maximum and encode as 0; the even element
 * goes to the HIGH nibble. Returns the number of blocks. */
ORC_API long long orc_quantize_mxfp4_gptoss(const float *src, size_t num_elements, uint8_t *data, uint8_t *scales) {
    size_t nb = (num_elements + 31) / 32;
    for (size_t b = 0; b < nb; b++) {
        float v[32];
        for (int i = 0; i < 32; i++) v[i] = b * 32 + i < num_elements ? src[b * 32 + i] : 0.0f;
        float max_abs = 0.0f;
        for (int i = 0; i < 32; i++) { float a = fabsf(v[i]); if (isfinite(a) && a > max_abs) max_abs = a; }
        uint8_t sb = 0;
        if (isfinite(max_abs) && max_abs > 0.0f) {
            uint32_t bits;
            memcpy(&bits, &max_abs, 4);
            uint32_t be = (bits >> 23) & 0xFFu;
            if (be != 0) { uint32_t se = be >= 2 ? be - 2 : 0; sb = (uint8_t)(se < 254 ? se : 254); }
        }
        scales[b] = sb;
        float scale = orc_mxfp4_gptoss_scale(sb);
        for (int p = 0; p < 16; p++) {
            uint8_t c[2];
            for (int h = 0; h < 2; h++) {
                float x = v[2 * p + h];
                c[h] = 0;
                if (isfinite(x) && scale > 0.0f) c[h] = (uint8_t)(nearest_e2m1(fabsf(x) / scale) | (x < 0.0f ? 8 : 0));
            }
            data[b * 16 + p] = (uint8_t)((c[0] << 4) | c[1]);
        }
    }
    return (long long)nb;
}

/* ------------------------------------------------------------------------- */
/* INT8 per-channel weights (W8A16)                                          */
/* ------------------------------------------------------------------------- */

/* `as i32` of an f32: saturating, NaN -> 0. */
static int32_t f32_as_i32(float v) {
    if (isnan(v)) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}

/* quantize_per_channel (crates/nn-core/src/layers/quantized/int8.rs:82-137) with
 * compute_channel_params (int8.rs:187-221). mode 0 = symmetric (scale = max|w| / 127, zero
 * point 0), 1 = asymmetric (scale = (max - min) / 255, zero point = round(-128 - min / scale)).
 * q = clamp(round(w / scale + zp), -128, 127), 0 where scale == 0. Returns 0, or -1 when a
 * weight is not finite (ValueOutOfRange). */
ORC_API int orc_int8_quantize_per_channel(const float *w, size_t n, size_t k, int mode, uint8_t *q,
                                          float *scale, int32_t *zp) {
    for (size_t i = 0; i < n * k; i++)
        if (!isfinite(w[i])) return -1;
    for (size_t r = 0; r < n; r++) {
        const float *row = w + r * k;
        float sc = 0.0f;
        int32_t z = 0;
        if (k != 0) {
            if (mode == 0) {
                float abs_max = 0.0f;
                for (size_t i = 0; i < k; i++) abs_max = fold_max(abs_max, fabsf(row[i]));
                if (abs_max != 0.0f) sc = abs_max / 127.0f;
            } else {
                float mn = INFINITY, mx = -INFINITY;
                for (size_t i = 0; i < k; i++) { mn = fold_min(mn, row[i]); mx = fold_max(mx, row[i]); }
                float range = mx - mn;
                if (range != 0.0f) {
                    sc = range / 255.0f;
                    z = f32_as_i32(roundf(-128.0f - mn / sc));
                }
            }
        }
        scale[r] = sc;
        zp[r] = z;
        for (size_t i = 0; i < k; i++) {
            int8_t v = 0;
            if (sc != 0.0f) {
                float qf = roundf(row[i] / sc + (float)z);
                qf = qf < -128.0f ? -128.0f : (qf > 127.0f ? 127.0f : qf);
                v = (int8_t)qf;
            }
            q[r * k + i] = (uint8_t)v;
        }
    }
    return 0;
}

/* dequantize_per_channel (int8.rs:146-185): w = (f32(q as i8) - f32(zp)) * scale. */
ORC_API void orc_int8_dequantize_per_channel(const uint8_t *q, const float *scale, const int32_t *zp, size_t n,
                                             size_t k, float *out) {
    for (size_t r = 0; r < n; r++)
        for (size_t i = 0; i < k; i++)
            out[r * k + i] = ((float)(int8_t)q[r * k + i] - (float)zp[r]) * scale[r];
}

/* ------------------------------------------------------------------------- */
/* INT4 / INT8 per-group weights, GPTQ / AWQ packed weights                   */
/* ------------------------------------------------------------------------- */

/* unpack_element (crates/nn-core/src/layers/quantized/weight_quant.rs:415-433): element `index`
 * of the flat packing; int4 codes sit two per byte (even index = low nibble) in two's complement. */
static int8_t group_code_at(const uint8_t *data, size_t index, int bits) {
    if (bits == 8) return (int8_t)data[index];
    uint8_t nib = (index % 2 == 0) ? (uint8_t)(data[index / 2] & 0x0F) : (uint8_t)(data[index / 2] >> 4);
    return (nib & 0x08) ? (int8_t)(nib | 0xF0) : (int8_t)nib;
}

/* quantize_per_group (weight_quant.rs:232-328) with compute_group_params (weight_quant.rs:334-365).
 * Symmetric: scale = max|w| / qmax (7 or 127), zero point 0. Asymmetric: scale = (max - min) /
 * (15 or 255), zero point = round(qmin - min / scale) with qmin = -8 or -128. Codes
 * clamp(round(w / scale + zp), qmin, qmax'), qmax' = 7 or 127, 0 where scale == 0; int8 codes one
 * per byte, int4 codes two per byte over the flat [n * k] index (a last odd element leaves the high
 * nibble 0). q holds n * k bytes (int8) or (n * k + 1) / 2 (int4). Returns 0; -1 for a non-finite
 * weight and -2 for group_size == 0 (both ValueOutOfRange); -3 when group_size does not divide k
 * (ShapeMismatch). */
ORC_API int orc_group_quantize(const float *w, size_t n, size_t k, int bits, size_t group_size, int symmetric,
                               uint8_t *q, float *scale, int32_t *zp) {
    if (group_size == 0) return -2;
    if (k % group_size != 0) return -3;
    for (size_t i = 0; i < n * k; i++)
        if (!isfinite(w[i])) return -1;
    const float sym_max = bits == 4 ? 7.0f : 127.0f, levels = bits == 4 ? 15.0f : 255.0f;
    const float lo = bits == 4 ? -8.0f : -128.0f, hi = bits == 4 ? 7.0f : 127.0f;
    const size_t gpr = k / group_size;
    if (bits == 4) memset(q, 0, (n * k + 1) / 2);
    for (size_t r = 0; r < n; r++)
        for (size_t g = 0; g < gpr; g++) {
            const float *grp = w + r * k + g * group_size;
            float sc = 0.0f;
            int32_t z = 0;
            if (symmetric) {
                float abs_max = 0.0f;
                for (size_t i = 0; i < group_size; i++) abs_max = fold_max(abs_max, fabsf(grp[i]));
                if (abs_max != 0.0f) sc = abs_max / sym_max;
            } else {
                float mn = INFINITY, mx = -INFINITY;
                for (size_t i = 0; i < group_size; i++) { mn = fold_min(mn, grp[i]); mx = fold_max(mx, grp[i]); }
                float range = mx - mn;
                if (range != 0.0f) {
                    sc = range / levels;
                    z = f32_as_i32(roundf(lo - mn / sc));
                }
            }
            scale[r * gpr + g] = sc;
            zp[r * gpr + g] = z;
            for (size_t i = 0; i < group_size; i++) {
                int8_t v = 0;
                if (sc != 0.0f) {
                    float qf = roundf(grp[i] / sc + (float)z);
                    qf = qf < lo ? lo : (qf > hi ? hi : qf);
                    v = (int8_t)qf;
                }
                const size_t idx = r * k + g * group_size + i;
                if (bits == 8) q[idx] = (uint8_t)v;
                else q[idx / 2] |= (uint8_t)((v & 0x0F) << (4 * (idx % 2)));
            }
        }
    return 0;
}

/* dequantize (weight_quant.rs:381-412): w = (f32(code) - f32(zero point)) * scale of the group. */
ORC_API void orc_group_dequantize(const uint8_t *q, const float *scale, const int32_t *zp, size_t n, size_t k,
                                  int bits, size_t group_size, float *out) {
    const size_t gpr = k / group_size;
    for (size_t r = 0; r < n; r++)
        for (size_t g = 0; g < gpr; g++)
            for (size_t e = 0; e < group_size; e++) {
                const size_t idx = r * k + g * group_size + e;
                out[idx] = ((float)group_code_at(q, idx, bits) - (float)zp[r * gpr + g]) * scale[r * gpr + g];
            }
}

/* unpack_gptq_qweight (crates/nn-core/src/layers/quantized/gptq_loader.rs:69-91; AWQ delegates to it,
 * awq_loader.rs:54-56): packed u32 [rows, cols], bits [4i+3 : 4i] of a word are the i-th of 8
 * consecutive values along the row axis; out f32 [8 * rows, cols], values 0..15. */
ORC_API void orc_gptq_unpack_qweight(const uint32_t *packed, size_t rows, size_t cols, float *out) {
    for (size_t r = 0; r < rows; r++)
        for (size_t c = 0; c < cols; c++)
            for (size_t b = 0; b < 8; b++)
                out[(r * 8 + b) * cols + c] = (float)((packed[r * cols + c] >> (4 * b)) & 0xFu);
}

/* unpack_gptq_qzeros (gptq_loader.rs:101-123): packed u32 [groups, cols], eight consecutive output
 * columns per word; out f32 [groups, 8 * cols]. */
ORC_API void orc_gptq_unpack_qzeros(const uint32_t *packed, size_t groups, size_t cols, float *out) {
    for (size_t g = 0; g < groups; g++)
        for (size_t c = 0; c < cols; c++)
            for (size_t b = 0; b < 8; b++)
                out[g * cols * 8 + c * 8 + b] = (float)((packed[g * cols + c] >> (4 * b)) & 0xFu);
}

/* dequantize_gptq (gptq_loader.rs:139-187): q, out f32 [k, n]; scales, zeros f32 [groups, n];
 * out[i][j] = (q[i][j] - zeros[i / group_size][j]) * scales[i / group_size][j]. Returns 0, or -1
 * when groups != ceil(k / group_size) (DataLengthMismatch). */
ORC_API int orc_gptq_dequantize(const float *q, const float *scales, const float *zeros, size_t k, size_t n,
                                size_t groups, size_t group_size, float *out) {
    if (group_size == 0 || groups != (k + group_size - 1) / group_size) return -1;
    for (size_t i = 0; i < k; i++)
        for (size_t j = 0; j < n; j++) {
            const size_t g = i / group_size;
            out[i * n + j] = (q[i * n + j] - zeros[g * n + j]) * scales[g * n + j];
        }
    return 0;
}

/* The weight load_gptq_linear / load_awq_linear build (gptq_loader.rs:329-351, awq_loader.rs:74-96):
 * unpack both packed tensors, dequantize, transpose to f32 [n, k]. qweight u32 [k / 8, n], scales
 * f32 [groups, n], qzeros u32 [groups, n / 8]. */
ORC_API int orc_gptq_load_weight(const uint32_t *qweight, const float *scales, const uint32_t *qzeros, size_t n,
                                 size_t k, size_t groups, size_t group_size, float *out) {
    if (group_size == 0 || groups != (k + group_size - 1) / group_size || k % 8 || n % 8) return -1;
    for (size_t i = 0; i < k; i++)
        for (size_t j = 0; j < n; j++) {
            const size_t g = i / group_size;
            const float qv = (float)((qweight[(i / 8) * n + j] >> (4 * (i % 8))) & 0xFu);
            const float zv = (float)((qzeros[g * (n / 8) + j / 8] >> (4 * (j % 8))) & 0xFu);
            out[j * k + i] = (qv - zv) * scales[g * n + j];
        }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* the reference's CPU forward of one quantized linear, as it is timed        */
/* ------------------------------------------------------------------------- */

/* Dequantize the whole weight, then the nn-cpu product: what one
 * QLinear::forward costs in the reference
 * (crates/nn-core/src/layers/quantized/linear.rs:374 re-dequantizes per call).
 * fmt uses the codes of include/nnq.h. `scratch` holds n*k floats. With
 * threads > 1 both stages are split by weight rows. Returns 0, or -1 for a
 * format this helper does not cover. */
ORC_API int orc_cpu_forward(int fmt, const uint8_t *w, size_t wbytes, const float *x,
                            const float *bias, float *y, float *scratch, size_t m, size_t n,
                            size_t k, int threads) {
    size_t be, bb;
    switch (fmt) {
        case 0: be = 32; bb = 18; break;
        case 1: be = 32; bb = 20; break;
        case 2: be = 32; bb = 34; break;
        case 3: case 4: be = 256; bb = 144; break;
        case 5: be = 256; bb = 210; break;
        case 9: be = 32; bb = 22; break;
        case 10: be = 32; bb = 24; break;
        case 11: be = 256; bb = 84; break;
        case 12: be = 256; bb = 110; break;
        case 13: be = 256; bb = 176; break;
        default: return -1;
    }
    size_t row_bytes = k / be * bb;
    if (wbytes < row_bytes * n) return -1;
    int nt = threads > 0 ? threads : 1;
#pragma omp parallel for schedule(static) num_threads(nt)
    for (long long r = 0; r < (long long)n; r++) {
        const uint8_t *src = w + (size_t)r * row_bytes;
        float *dst = scratch + (size_t)r * k;
        switch (fmt) {
            case 0: orc_dequant_q4_0(src, row_bytes, k, dst); break;
            case 1: orc_dequant_q4_1(src, row_bytes, k, dst); break;
            case 2: orc_dequant_q8_0(src, row_bytes, k, dst); break;
            case 3: orc_dequant_q4_k(src, row_bytes, k, dst); break;
            case 4: orc_dequant_q4_k_ggml(src, row_bytes, k, dst); break;
            case 5: orc_dequant_q6_k(src, row_bytes, k, dst); break;
            case 9: orc_dequant_q5_0(src, row_bytes, k, dst); break;
            case 10: orc_dequant_q5_1(src, row_bytes, k, dst); break;
            case 11: orc_dequant_q2_k(src, row_bytes, k, dst); break;
            case 12: orc_dequant_q3_k(src, row_bytes, k, dst); break;
            default: orc_dequant_q5_k(src, row_bytes, k, dst); break;
        }
    }
    orc_nncpu_linear(x, scratch, bias, y, m, n, k, nt);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* MoE block of the gpt-oss quantized model                                  */
/* ------------------------------------------------------------------------- */

typedef struct {
    float v;
    int i;
} orc_pair;

static int cmp_desc(const void *a, const void *b) {
    float x = ((const orc_pair *)a)->v, y = ((const orc_pair *)b)->v;
    if (x > y) return -1;
    if (x < y) return 1;
    return ((const orc_pair *)a)->i - ((const orc_pair *)b)->i;
}

/* Router for one token: softmax over all experts, the k largest probabilities in
 * descending order, then division by their sum. Inputs must have no ties (the
 * reference's partial sort is unstable on ties).
 * crates/nn-gptoss/src/quantized_model.rs:136-144;
 * crates/nn-core/src/dyn_tensor/ops/topk.rs:108-133;
 * crates/nn-core/src/dyn_tensor/ops/softmax.rs:115-155 (max-subtracted, f32). */
ORC_API void orc_moe_route(const float *logits, int n_experts, int top_k, int *idx_out,
                           float *w_out) {
    orc_pair *p = (orc_pair *)malloc(sizeof(orc_pair) * (size_t)n_experts);
    float mx = logits[0];
    for (int e = 1; e < n_experts; e++) mx = logits[e] > mx ? logits[e] : mx;
    float sum = 0.0f;
    for (int e = 0; e < n_experts; e++) {
        p[e].v = expf(logits[e] - mx);
        p[e].i = e;
        sum += p[e].v;
    }
    for (int e = 0; e < n_experts; e++) p[e].v = p[e].v / sum;
    qsort(p, (size_t)n_experts, sizeof(orc_pair), cmp_desc);
    float ws = 0.0f;
    for (int s = 0; s < top_k; s++) ws += p[s].v;
    for (int s = 0; s < top_k; s++) {
        idx_out[s] = p[s].i;
        w_out[s] = p[s].v / ws;
    }
    free(p);
}

static float silu_f32(float x) { return x / (1.0f + expf(-x)); }

/* Whole MoE block on dequantized expert weights stored [E][K][N] (x * W, W is
 * [K, N] per expert): router linear (+bias), routing as above, then for experts
 * in index order: gate_up = x*W_gu + b_gu; hidden = clamp(silu(gate), +-limit) * up
 * with gate = first half, up = second half; out = hidden*W_d + b_d; the token's
 * output accumulates routing_weight * out.
 * crates/nn-gptoss/src/quantized_model.rs:99-130 (expert_forward), :132-194. */
ORC_API void orc_moe_forward(const float *x, size_t tokens, size_t hidden, size_t inter,
                             int n_experts, int top_k, const float *router_w /*[E,hidden]*/,
                             const float *router_b /*[E]*/, const float *w_gu /*[E,hidden,2*inter]*/,
                             const float *b_gu /*[E,2*inter]*/, const float *w_d /*[E,inter,hidden]*/,
                             const float *b_d /*[E,hidden]*/, float limit, float *y,
                             int *idx_out /*[tokens,top_k] or NULL*/,
                             float *wt_out /*[tokens,top_k] or NULL*/) {
    size_t f = 2 * inter;
    int *idx = (int *)malloc(sizeof(int) * tokens * (size_t)top_k);
    float *wt = (float *)malloc(sizeof(float) * tokens * (size_t)top_k);
#pragma omp parallel for schedule(static)
    for (long long t = 0; t < (long long)tokens; t++) {
        float *logit = (float *)malloc(sizeof(float) * (size_t)n_experts);
        for (int e = 0; e < n_experts; e++) {
            float acc = 0.0f;
            for (size_t i = 0; i < hidden; i++) acc += x[t * hidden + i] * router_w[(size_t)e * hidden + i];
            logit[e] = acc + router_b[e];
        }
        orc_moe_route(logit, n_experts, top_k, idx + t * top_k, wt + t * top_k);
        free(logit);
    }
    memset(y, 0, sizeof(float) * tokens * hidden);
#pragma omp parallel for schedule(dynamic)
    for (long long t = 0; t < (long long)tokens; t++) {
        float *gu = (float *)malloc(sizeof(float) * f);
        float *h = (float *)malloc(sizeof(float) * inter);
        /* experts visited in index order, as the reference's per-expert loop does */
        for (int e = 0; e < n_experts; e++) {
            float rw = 0.0f;
            int hit = 0;
            for (int s = 0; s < top_k; s++)
                if (idx[t * top_k + s] == e) {
                    rw = wt[t * top_k + s];
                    hit = 1;
                }
            if (!hit) continue;
            const float *wg = w_gu + (size_t)e * hidden * f;
            for (size_t j = 0; j < f; j++) gu[j] = 0.0f;
            for (size_t i = 0; i < hidden; i++) {
                float xv = x[t * hidden + i];
                const float *wr = wg + i * f;
                for (size_t j = 0; j < f; j++) gu[j] += xv * wr[j];
            }
            for (size_t j = 0; j < f; j++) gu[j] = gu[j] + b_gu[(size_t)e * f + j];
            for (size_t j = 0; j < inter; j++) {
                float g = silu_f32(gu[j]);
                g = g < -limit ? -limit : (g > limit ? limit : g);
                h[j] = g * gu[inter + j];
            }
            const float *wd = w_d + (size_t)e * inter * hidden;
            float *o = (float *)calloc(hidden, sizeof(float));
            for (size_t i = 0; i < inter; i++) {
                float hv = h[i];
                const float *wr = wd + i * hidden;
                for (size_t j = 0; j < hidden; j++) o[j] += hv * wr[j];
            }
            for (size_t j = 0; j < hidden; j++) {
                float v = o[j] + b_d[(size_t)e * hidden + j];
                y[t * hidden + j] += v * rw;
            }
            free(o);
        }
        free(gu);
        free(h);
    }
    if (idx_out) memcpy(idx_out, idx, sizeof(int) * tokens * (size_t)top_k);
    if (wt_out) memcpy(wt_out, wt, sizeof(float) * tokens * (size_t)top_k);
    free(idx);
    free(wt);
}
