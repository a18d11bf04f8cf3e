// INT4 / INT8 weights with one (scale, zero point) pair per group of weights along K, and the
// GPTQ / AWQ packed form of the same idea.
//
// Reference (crates/nn-core/src/layers/quantized/):
//   weight_quant.rs:232-365  quantize_per_group + compute_group_params
//   weight_quant.rs:381-433  dequantize + unpack_element: w = (f32(code) - f32(zp)) * scale
//   weight_quant.rs:451-473  quantized_matmul: x @ dequantize(W)^T
//   gptq_loader.rs:69-123    unpack_gptq_qweight / unpack_gptq_qzeros (eight 4-bit values per u32)
//   gptq_loader.rs:139-187   dequantize_gptq: (q - zero[group]) * scale[group]
//   gptq_loader.rs:283-351   GptqLinear::forward, load_gptq_linear; awq_loader.rs:54-96 delegates
//
// The reference materialises the f32 weight (at every product for the per-group form, at load for
// GPTQ / AWQ). Here the packed codes stay packed: both forms are brought to one device layout at
// load (codes row-major [N, K], so that a 32-bit word holds 8 (or 4) consecutive weights of one
// output row; scale and zero point as f32 [N, groups]) and the product streams half a byte (or one
// byte) per weight. A warp owns four output rows, lanes take 16-byte chunks, a code becomes a float
// with one shift-and-mask into the mantissa of 2^23 and one subtraction (the zero point rides in
// the subtraction's constant), the group's scale is applied to the partial sum of 8 weights. From
// 17 tokens on the weight is decoded to bf16 once and the tensor-core product follows.
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include "gemm_tc.h"
#include "nnq_internal.h"

struct nnq_gq_weight {
    nnq_ctx *ctx;
    int64_t n, k, groups;   // groups per row: ceil(k / group_size)
    int bits, group_size;
    int is_signed;          // two's complement codes (per-group rows); 0: codes 0..15 (GPTQ / AWQ)
    int fast;               // rows on 16-byte boundaries, groups on 8-weight boundaries, small zero points
    uint8_t *codes;         // flat row-major packing of [n * k] codes
    size_t code_bytes;
    float *scale, *zpf;     // [n, groups]
};

namespace nnq {
namespace {

constexpr int kGqThreads = 256;

__device__ int g_gq_flag;       // raised by the encoder on a non-finite weight
__device__ unsigned g_gq_zpmax; // bits of the largest |zero point| seen at creation

__device__ __forceinline__ float gmin(float a, float b) { return b < a ? b : a; }
__device__ __forceinline__ float gmax(float a, float b) { return b > a ? b : a; }

__device__ __forceinline__ int gq_f32_as_i32(float v) {   // `as i32`: saturating, NaN -> 0
    if (isnan(v)) return 0;
    if (v >= 2147483648.0f) return 2147483647;
    if (v <= -2147483648.0f) return (-2147483647 - 1);
    return (int)v;
}

// element `idx` of the flat packing
__device__ __forceinline__ int gq_code_at(const uint8_t *codes, int64_t idx, int bits, int is_signed) {
    if (bits == 8) return (int)(int8_t)__ldg(codes + idx);
    const int nib = (__ldg(codes + (idx >> 1)) >> (4 * (int)(idx & 1))) & 0xF;
    return is_signed ? ((nib ^ 8) - 8) : nib;
}

// One warp per group: the group's scale and zero point.
__global__ void __launch_bounds__(kGqThreads)
gq_params_kernel(const float *__restrict__ w, int64_t total_groups, int64_t gpr, int64_t k, int g, int bits, int symmetric,
                 float *__restrict__ scale, int *__restrict__ zp) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (kGqThreads / 32);
    const float sym_max = bits == 4 ? 7.0f : 127.0f, levels = bits == 4 ? 15.0f : 255.0f, lo = bits == 4 ? -8.0f : -128.0f;
    for (int64_t gi = (int64_t)blockIdx.x * (kGqThreads / 32) + (threadIdx.x >> 5); gi < total_groups; gi += warps) {
        const float *grp = w + (gi / gpr) * k + (gi % gpr) * g;
        float mn = INFINITY, mx = -INFINITY;
        bool bad = false;
        for (int i = lane; i < g; i += 32) {
            const float v = __ldg(grp + i);
            bad |= !isfinite(v);
            mn = gmin(mn, v);
            mx = gmax(mx, v);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            mn = gmin(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = gmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if (bad) atomicExch(&g_gq_flag, 1);
        if (lane == 0) {
            float sc = 0.0f;
            int z = 0;
            if (symmetric) {
                const float abs_max = gmax(gmax(0.0f, fabsf(mn)), fabsf(mx));
                if (abs_max != 0.0f) sc = __fdiv_rn(abs_max, sym_max);
            } else {
                const float range = __fsub_rn(mx, mn);
                if (range != 0.0f) {
                    sc = __fdiv_rn(range, levels);
                    z = gq_f32_as_i32(roundf(__fsub_rn(lo, __fdiv_rn(mn, sc))));
                }
            }
            scale[gi] = sc;
            zp[gi] = z;
        }
    }
}

__device__ __forceinline__ int gq_encode_one(const float *w, int64_t idx, int64_t k, int64_t gpr, int g, float lo, float hi,
                                             const float *scale, const int *zp) {
    const int64_t row = idx / k, col = idx - row * k;
    const int64_t gi = row * gpr + col / g;
    const float sc = __ldg(scale + gi);
    if (sc == 0.0f) return 0;
    float qf = roundf(__fadd_rn(__fdiv_rn(__ldg(w + idx), sc), (float)__ldg(zp + gi)));
    qf = qf < lo ? lo : (qf > hi ? hi : qf);
    return isnan(qf) ? 0 : (int)qf;
}

// One thread per output byte: one int8 code, or two int4 codes (even index in the low nibble).
__global__ void __launch_bounds__(kGqThreads)
gq_encode_kernel(const float *__restrict__ w, int64_t total, int64_t k, int64_t gpr, int g, int bits,
                 const float *__restrict__ scale, const int *__restrict__ zp, uint8_t *__restrict__ q) {
    const float lo = bits == 4 ? -8.0f : -128.0f, hi = bits == 4 ? 7.0f : 127.0f;
    const int64_t nbytes = bits == 8 ? total : (total + 1) / 2;
    for (int64_t b = (int64_t)blockIdx.x * kGqThreads + threadIdx.x; b < nbytes; b += (int64_t)gridDim.x * kGqThreads) {
        if (bits == 8) {
            q[b] = (uint8_t)(int8_t)gq_encode_one(w, b, k, gpr, g, lo, hi, scale, zp);
        } else {
            const int c0 = gq_encode_one(w, 2 * b, k, gpr, g, lo, hi, scale, zp);
            const int c1 = 2 * b + 1 < total ? gq_encode_one(w, 2 * b + 1, k, gpr, g, lo, hi, scale, zp) : 0;
            q[b] = (uint8_t)((c0 & 0xF) | ((c1 & 0xF) << 4));
        }
    }
}

__device__ __forceinline__ void gq_put8(float *out, int64_t idx, const float *v) {
    reinterpret_cast<float4 *>(out + idx)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4 *>(out + idx)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void gq_put8(__nv_bfloat16 *out, int64_t idx, const float *v) {
    uint32_t p[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        p[i] = *reinterpret_cast<uint32_t *>(&h);
    }
    *reinterpret_cast<uint4 *>(out + idx) = make_uint4(p[0], p[1], p[2], p[3]);
}
__device__ __forceinline__ void gq_put1(float *out, int64_t idx, float v) { out[idx] = v; }
__device__ __forceinline__ void gq_put1(__nv_bfloat16 *out, int64_t idx, float v) { out[idx] = __float2bfloat16_rn(v); }

// Decode to f32 (bit-exact with the reference's dequantize) or to bf16 (operand of the tensor-core
// product). VEC: k and the group size are multiples of 8, one thread decodes 8 weights of one group.
template <typename OUT, typename ZT, bool VEC>
__global__ void __launch_bounds__(kGqThreads)
gq_decode_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ scale, const ZT *__restrict__ zp, int64_t total,
                 int64_t k, int64_t groups, int g, int bits, int is_signed, OUT *__restrict__ out) {
    const int64_t stride = (int64_t)gridDim.x * kGqThreads;
    if (VEC) {
        for (int64_t e = (int64_t)blockIdx.x * kGqThreads + threadIdx.x; e < total / 8; e += stride) {
            const int64_t idx = e * 8, row = idx / k, col = idx - row * k;
            const int64_t gi = row * groups + col / g;
            const float sc = __ldg(scale + gi), zf = (float)__ldg(zp + gi);
            float v[8];
            if (bits == 4) {
                const uint32_t word = __ldg(reinterpret_cast<const uint32_t *>(codes + idx / 2));
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int nib = (word >> (4 * i)) & 0xF;
                    v[i] = __fmul_rn(__fsub_rn((float)(is_signed ? ((nib ^ 8) - 8) : nib), zf), sc);
                }
            } else {
                const uint2 two = __ldg(reinterpret_cast<const uint2 *>(codes + idx));
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint32_t word = i < 4 ? two.x : two.y;
                    v[i] = __fmul_rn(__fsub_rn((float)(int8_t)((word >> (8 * (i & 3))) & 0xFF), zf), sc);
                }
            }
            gq_put8(out, idx, v);
        }
    } else {
        for (int64_t idx = (int64_t)blockIdx.x * kGqThreads + threadIdx.x; idx < total; idx += stride) {
            const int64_t row = idx / k, col = idx - row * k;
            const int64_t gi = row * groups + col / g;
            gq_put1(out, idx, __fmul_rn(__fsub_rn((float)gq_code_at(codes, idx, bits, is_signed), (float)__ldg(zp + gi)), __ldg(scale + gi)));
        }
    }
}

template <typename XT>
__device__ __forceinline__ void gq_load_x8(const XT *p, float *o);
template <>
__device__ __forceinline__ void gq_load_x8<float>(const float *p, float *o) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <>
__device__ __forceinline__ void gq_load_x8<__nv_bfloat16>(const __nv_bfloat16 *p, float *o) {
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        o[2 * j] = __uint_as_float(w[j] << 16);
        o[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
}
__device__ __forceinline__ float gq_x_at(const float *p, int64_t i) { return __ldg(p + i); }
__device__ __forceinline__ float gq_x_at(const __nv_bfloat16 *p, int64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void gq_store_y(void *y, int y_dt, int64_t i, float v) {
    if (y_dt == NNQ_F32) reinterpret_cast<float *>(y)[i] = v;
    else reinterpret_cast<__nv_bfloat16 *>(y)[i] = __float2bfloat16_rn(v);
}

constexpr int kGqLinThreads = 128;
constexpr int kGqRows = 4;   // output rows per warp: one load of the activations serves four rows

// y[t][r] = sum over groups of scale[r][g] * sum_{k in g} (code[r][k] - zp[r][g]) * x[t][k] (+ bias[r])
// for tokens [t0, t0 + MT). Needs k % 32 == 0, group_size % 8 == 0, 16-byte aligned x, |zp| < 4e6.
// GC: a 16-byte chunk never straddles a group (group_size a multiple of 32 / 16 weights), so scale and
// zero point are fetched once per chunk and row.
template <int BITS, typename XT, int MT, bool GC>
__global__ void __launch_bounds__(kGqLinThreads)
gq_linear_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ scale, const float *__restrict__ zpf,
                 int64_t groups, int g, int gshift, int is_signed, const XT *__restrict__ x, const float *__restrict__ bias,
                 void *__restrict__ y, int y_dt, int64_t m, int64_t n, int64_t k, int64_t t0) {
    constexpr int R = kGqRows;
    constexpr int WPC = BITS == 4 ? 32 : 16;   // weights per 16-byte chunk
    constexpr int SUBS = WPC / 8;
    const int lane = threadIdx.x & 31;
    const int64_t units = (n + R - 1) / R;
    const int64_t warps = (int64_t)gridDim.x * (kGqLinThreads / 32);
    const int64_t row_bytes = k * BITS / 8;
    // float(code + bias) sits in the mantissa of 2^23; subtracting 2^23 + bias + zp leaves code - zp exactly
    const float off = 8388608.0f + (BITS == 8 ? 128.0f : (is_signed ? 8.0f : 0.0f));
    const uint32_t flip = BITS == 8 ? 0x80808080u : (is_signed ? 0x88888888u : 0u);
    for (int64_t u = (int64_t)blockIdx.x * (kGqLinThreads / 32) + (threadIdx.x >> 5); u < units; u += warps) {
        const uint8_t *row[R];
        const float *sc[R], *zp[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int64_t rr = u * R + r < n ? u * R + r : n - 1;   // rows past the end repeat the last one; not stored
            row[r] = codes + rr * row_bytes;
            sc[r] = scale + rr * groups;
            zp[r] = zpf + rr * groups;
        }
        float acc[R][MT];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int t = 0; t < MT; t++) acc[r][t] = 0.0f;
#pragma unroll 2
        for (int64_t k0 = (int64_t)lane * WPC; k0 < k; k0 += 32 * WPC) {
            uint32_t raw[R][4];
#pragma unroll
            for (int r = 0; r < R; r++) {
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(row[r] + k0 * BITS / 8));
                raw[r][0] = v.x ^ flip; raw[r][1] = v.y ^ flip; raw[r][2] = v.z ^ flip; raw[r][3] = v.w ^ flip;
            }
            float cc[R], gsc[R];
            if (GC) {
                const int64_t gi = gshift >= 0 ? (k0 >> gshift) : k0 / g;
#pragma unroll
                for (int r = 0; r < R; r++) {
                    cc[r] = __fadd_rn(off, __ldg(zp[r] + gi));
                    gsc[r] = __ldg(sc[r] + gi);
                }
            }
#pragma unroll
            for (int s = 0; s < SUBS; s++) {
                const int64_t kk = k0 + 8 * s;
                const int64_t gi = GC ? 0 : (gshift >= 0 ? (kk >> gshift) : kk / g);
                float xv[MT][8];
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    const int64_t tt = t0 + t < m ? t0 + t : m - 1;
                    gq_load_x8<XT>(x + tt * k + kk, xv[t]);
                }
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const float c = GC ? cc[r] : __fadd_rn(off, __ldg(zp[r] + gi));
                    const float gs = GC ? gsc[r] : __ldg(sc[r] + gi);
                    float wv[8];
                    if (BITS == 4) {
                        const uint32_t word = raw[r][s];
#pragma unroll
                        for (int i = 0; i < 8; i++) wv[i] = __fsub_rn(__uint_as_float(((word >> (4 * i)) & 0xFu) | 0x4B000000u), c);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; i++)
                            wv[i] = __fsub_rn(__uint_as_float(__byte_perm(raw[r][2 * s + (i >> 2)], 0x4B000000u, 0x7540u + (i & 3))), c);
                    }
#pragma unroll
                    for (int t = 0; t < MT; t++) {
                        float part = 0.0f;
#pragma unroll
                        for (int i = 0; i < 8; i++) part = fmaf(wv[i], xv[t][i], part);
                        acc[r][t] = fmaf(gs, part, acc[r][t]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int64_t rr = u * R + r;
#pragma unroll
            for (int t = 0; t < MT; t++) {
                float v = acc[r][t];
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && rr < n && t0 + t < m) gq_store_y(y, y_dt, (t0 + t) * n + rr, v + (bias ? __ldg(bias + rr) : 0.0f));
            }
        }
    }
}

// Any k, group size and packing: a warp per (token, output row), element by element, each weight
// formed exactly as the reference's dequantize forms it.
template <typename XT>
__global__ void __launch_bounds__(kGqLinThreads)
gq_linear_generic_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ scale, const float *__restrict__ zpf,
                         int64_t groups, int g, int bits, int is_signed, const XT *__restrict__ x,
                         const float *__restrict__ bias, void *__restrict__ y, int y_dt, int64_t m, int64_t n, int64_t k) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (kGqLinThreads / 32);
    for (int64_t p = (int64_t)blockIdx.x * (kGqLinThreads / 32) + (threadIdx.x >> 5); p < m * n; p += warps) {
        const int64_t t = p / n, r = p - t * n;
        float acc = 0.0f;
        for (int64_t col = lane; col < k; col += 32) {
            const int64_t gi = r * groups + col / g;
            const float wv = __fmul_rn(__fsub_rn((float)gq_code_at(codes, r * k + col, bits, is_signed), __ldg(zpf + gi)), __ldg(scale + gi));
            acc = fmaf(wv, gq_x_at(x, t * k + col), acc);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) gq_store_y(y, y_dt, p, acc + (bias ? __ldg(bias + r) : 0.0f));
    }
}

// u32 [rows, cols] -> [cols, rows] through a padded shared-memory tile
__global__ void __launch_bounds__(256)
gq_transpose_u32_kernel(const uint32_t *__restrict__ in, int64_t rows, int64_t cols, uint32_t *__restrict__ out) {
    __shared__ uint32_t tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t r0 = (int64_t)blockIdx.y * 32, c0 = (int64_t)blockIdx.x * 32;
#pragma unroll
    for (int j = ty; j < 32; j += 8)
        if (r0 + j < rows && c0 + tx < cols) tile[j][tx] = __ldg(in + (r0 + j) * cols + c0 + tx);
    __syncthreads();
#pragma unroll
    for (int j = ty; j < 32; j += 8)
        if (c0 + j < cols && r0 + tx < rows) out[(c0 + j) * rows + r0 + tx] = tile[tx][j];
}

// GPTQ scales f32 [groups, n] and packed zero points u32 [groups, n / 8] -> f32 [n, groups] each
__global__ void __launch_bounds__(kGqThreads)
gq_gptq_params_kernel(const float *__restrict__ scales, const uint32_t *__restrict__ qzeros, int64_t n, int64_t groups,
                      float *__restrict__ scale_out, float *__restrict__ zpf_out) {
    for (int64_t i = (int64_t)blockIdx.x * kGqThreads + threadIdx.x; i < n * groups; i += (int64_t)gridDim.x * kGqThreads) {
        const int64_t gi = i / n, j = i - gi * n;   // consecutive threads read consecutive columns
        scale_out[j * groups + gi] = __ldg(scales + i);
        zpf_out[j * groups + gi] = (float)((__ldg(qzeros + gi * (n / 8) + j / 8) >> (4 * (int)(j & 7))) & 0xFu);
    }
}

__global__ void __launch_bounds__(kGqThreads)
gq_zp_to_f32_kernel(const int32_t *__restrict__ zp, int64_t count, float *__restrict__ zpf) {
    float big = 0.0f;
    for (int64_t i = (int64_t)blockIdx.x * kGqThreads + threadIdx.x; i < count; i += (int64_t)gridDim.x * kGqThreads) {
        const float f = (float)__ldg(zp + i);
        zpf[i] = f;
        big = gmax(big, fabsf(f));
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) big = gmax(big, __shfl_xor_sync(0xffffffffu, big, o));
    if ((threadIdx.x & 31) == 0 && big > 0.0f) atomicMax(&g_gq_zpmax, __float_as_uint(big));   // non-negative floats order as their bits
}

// unpack_gptq_qweight: thread per packed word, eight rows of the output
__global__ void __launch_bounds__(kGqThreads)
gq_unpack_rows_kernel(const uint32_t *__restrict__ packed, int64_t rows, int64_t cols, float *__restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * kGqThreads + threadIdx.x; i < rows * cols; i += (int64_t)gridDim.x * kGqThreads) {
        const int64_t r = i / cols, c = i - r * cols;
        const uint32_t word = __ldg(packed + i);
#pragma unroll
        for (int b = 0; b < 8; b++) out[(r * 8 + b) * cols + c] = (float)((word >> (4 * b)) & 0xFu);
    }
}

// unpack_gptq_qzeros: thread per packed word, eight consecutive columns of the output
__global__ void __launch_bounds__(kGqThreads)
gq_unpack_cols_kernel(const uint32_t *__restrict__ packed, int64_t words, float *__restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * kGqThreads + threadIdx.x; i < words; i += (int64_t)gridDim.x * kGqThreads) {
        const uint32_t word = __ldg(packed + i);
        float v[8];
#pragma unroll
        for (int b = 0; b < 8; b++) v[b] = (float)((word >> (4 * b)) & 0xFu);
        gq_put8(out, i * 8, v);
    }
}

// dequantize_gptq over unpacked f32 values [k, n]
__global__ void __launch_bounds__(kGqThreads)
gq_gptq_dequantize_kernel(const float *__restrict__ q, const float *__restrict__ scales, const float *__restrict__ zeros,
                          int64_t k, int64_t n, int64_t g, float *__restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * kGqThreads + threadIdx.x; i < k * n; i += (int64_t)gridDim.x * kGqThreads) {
        const int64_t row = i / n, j = i - row * n, gi = row / g;
        out[i] = __fmul_rn(__fsub_rn(__ldg(q + i), __ldg(zeros + gi * n + j)), __ldg(scales + gi * n + j));
    }
}

int grid_for(const nnq_ctx *ctx, int64_t work, int threads) {
    const int64_t want = (work + threads - 1) / threads, cap = (int64_t)ctx->sm_count * 16;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

template <typename OUT, typename ZT>
cudaError_t launch_decode(nnq_ctx *ctx, const uint8_t *codes, const float *scale, const ZT *zp, int64_t n, int64_t k,
                          int64_t groups, int g, int bits, int is_signed, OUT *out, cudaStream_t st) {
    const int64_t total = n * k;
    const bool vec = k % 8 == 0 && g % 8 == 0 && !((uintptr_t)codes & 7u) && !((uintptr_t)out & 15u);
    if (vec) gq_decode_kernel<OUT, ZT, true><<<grid_for(ctx, total / 8, kGqThreads), kGqThreads, 0, st>>>(codes, scale, zp, total, k, groups, g, bits, is_signed, out);
    else gq_decode_kernel<OUT, ZT, false><<<grid_for(ctx, total, kGqThreads), kGqThreads, 0, st>>>(codes, scale, zp, total, k, groups, g, bits, is_signed, out);
    ctx->launches++;
    return cudaGetLastError();
}

template <int BITS, typename XT>
void launch_fast(nnq_gq_weight *w, const void *x, const float *bias, void *y, int y_dt, int64_t m, cudaStream_t st) {
    nnq_ctx *ctx = w->ctx;
    const int64_t units = (w->n + kGqRows - 1) / kGqRows, per_cta = kGqLinThreads / 32;
    const int64_t want = (units + per_cta - 1) / per_cta, cap = (int64_t)ctx->sm_count * 16;
    const int grid = (int)(want < cap ? want : cap);
    const bool gc = w->group_size % (BITS == 4 ? 32 : 16) == 0;
    int gshift = -1;
    if ((w->group_size & (w->group_size - 1)) == 0)
        for (gshift = 0; (1 << gshift) < w->group_size; gshift++) {}
    for (int64_t t0 = 0; t0 < m; t0 += 4) {   // four tokens share a pass over the weights
        const int64_t left = m - t0;
#define NNQ_GQ(MT, GC) gq_linear_kernel<BITS, XT, MT, GC><<<grid, kGqLinThreads, 0, st>>>(w->codes, w->scale, w->zpf, w->groups, w->group_size, \
                           gshift, w->is_signed, (const XT *)x, bias, y, y_dt, m, w->n, w->k, t0)
        if (gc) {
            if (left == 1) NNQ_GQ(1, true);
            else if (left == 2) NNQ_GQ(2, true);
            else NNQ_GQ(4, true);
        } else {
            if (left == 1) NNQ_GQ(1, false);
            else if (left == 2) NNQ_GQ(2, false);
            else NNQ_GQ(4, false);
        }
#undef NNQ_GQ
        ctx->launches++;
    }
}

nnq_status gq_alloc(nnq_ctx *ctx, int64_t n, int64_t k, int bits, int group_size, int64_t groups, int is_signed, nnq_gq_weight **out) {
    nnq_gq_weight *w = new (std::nothrow) nnq_gq_weight();
    if (!w) return fail(ctx, NNQ_ERR_OUT_OF_MEMORY, "host allocation failed");
    w->ctx = ctx;
    w->n = n; w->k = k; w->groups = groups;
    w->bits = bits; w->group_size = group_size; w->is_signed = is_signed;
    w->code_bytes = bits == 8 ? (size_t)(n * k) : (size_t)((n * k + 1) / 2);
    const size_t pbytes = (size_t)(n * groups) * 4;
    nnq_status s = check_cuda(ctx, cudaMalloc(&w->codes, w->code_bytes ? w->code_bytes : 16), "cudaMalloc codes");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMalloc(&w->scale, pbytes ? pbytes : 16), "cudaMalloc group scales");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMalloc(&w->zpf, pbytes ? pbytes : 16), "cudaMalloc group zero points");
    if (s == NNQ_OK) s = dense_scratch_reserve(ctx, n, k);
    if (s != NNQ_OK) {
        cudaFree(w->codes); cudaFree(w->scale); cudaFree(w->zpf);
        delete w;
        return s;
    }
    *out = w;
    return NNQ_OK;
}

void gq_set_fast(nnq_gq_weight *w, float zp_abs_max) {
    w->fast = w->k >= 32 && w->k % 32 == 0 && w->group_size % 8 == 0 && zp_abs_max < 4.0e6f;
}

}  // namespace
}  // namespace nnq

using namespace nnq;

extern "C" {

nnq_status nnq_group_quantize(nnq_ctx *ctx, const float *w_dev, int64_t n, int64_t k, int bits, int64_t group_size,
                              int symmetric, void *q_dev, float *scale_dev, int32_t *zp_dev, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (n < 0 || k < 0 || (bits != 4 && bits != 8)) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad per-group quantize arguments");
    if (group_size <= 0) return fail(ctx, NNQ_ERR_VALUE_OUT_OF_RANGE, "quantize_per_group: group_size must be > 0");
    if (k % group_size != 0) return fail(ctx, NNQ_ERR_SHAPE_MISMATCH, "quantize_per_group: in_features %lld not divisible by group_size %lld", (long long)k, (long long)group_size);
    if (group_size > 0x7fffffff) return fail(ctx, NNQ_ERR_UNSUPPORTED, "group_size too large");
    if (n == 0 || k == 0) return NNQ_OK;
    if (!w_dev || !q_dev || !scale_dev || !zp_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    cudaStream_t st = (cudaStream_t)stream;
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    int *flag = nullptr;
    s = check_cuda(ctx, cudaGetSymbolAddress((void **)&flag, g_gq_flag), "per-group flag");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemsetAsync(flag, 0, sizeof(int), st), "per-group flag clear");
    if (s != NNQ_OK) return s;
    const int64_t gpr = k / group_size, total_groups = n * gpr;
    gq_params_kernel<<<grid_for(ctx, total_groups, kGqThreads / 32), kGqThreads, 0, st>>>(w_dev, total_groups, gpr, k, (int)group_size, bits, symmetric ? 1 : 0, scale_dev, zp_dev);
    const int64_t nbytes = bits == 8 ? n * k : (n * k + 1) / 2;
    gq_encode_kernel<<<grid_for(ctx, nbytes, kGqThreads), kGqThreads, 0, st>>>(w_dev, n * k, k, gpr, (int)group_size, bits, scale_dev, zp_dev, (uint8_t *)q_dev);
    ctx->launches += 2;
    s = check_cuda(ctx, cudaGetLastError(), "per-group quantize launch");
    if (s != NNQ_OK) return s;
    int raised = 0;
    s = check_cuda(ctx, cudaMemcpyAsync(&raised, flag, sizeof(int), cudaMemcpyDeviceToHost, st), "per-group flag read");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaStreamSynchronize(st), "per-group quantize synchronize");
    if (s != NNQ_OK) return s;
    if (raised) return fail(ctx, NNQ_ERR_VALUE_OUT_OF_RANGE, "quantize_per_group: non-finite weight value");
    return NNQ_OK;
}

nnq_status nnq_group_dequantize(nnq_ctx *ctx, const void *q_dev, const float *scale_dev, const int32_t *zp_dev, int64_t n,
                                int64_t k, int bits, int64_t group_size, float *dst_dev, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (n < 0 || k < 0 || (bits != 4 && bits != 8) || group_size <= 0 || group_size > 0x7fffffff)
        return fail(ctx, NNQ_ERR_INVALID_ARG, "bad per-group dequantize arguments");
    if (k % group_size != 0) return fail(ctx, NNQ_ERR_SHAPE_MISMATCH, "in_features %lld not divisible by group_size %lld", (long long)k, (long long)group_size);
    if (n == 0 || k == 0) return NNQ_OK;
    if (!q_dev || !scale_dev || !zp_dev || !dst_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    return check_cuda(ctx, launch_decode<float, int32_t>(ctx, (const uint8_t *)q_dev, scale_dev, zp_dev, n, k, k / group_size, (int)group_size, bits, 1, dst_dev, (cudaStream_t)stream),
                      "per-group dequantize launch");
}

nnq_status nnq_gq_create_per_group(nnq_ctx *ctx, const void *q_dev, const float *scale_dev, const int32_t *zp_dev, int64_t n,
                                   int64_t k, int bits, int64_t group_size, void *stream, nnq_gq_weight **out) {
    if (!ctx || !out) return NNQ_ERR_INVALID_ARG;
    *out = nullptr;
    if (n < 0 || k < 0 || (bits != 4 && bits != 8) || group_size <= 0 || group_size > 0x7fffffff)
        return fail(ctx, NNQ_ERR_INVALID_ARG, "bad per-group weight arguments");
    if (k % group_size != 0) return fail(ctx, NNQ_ERR_SHAPE_MISMATCH, "in_features %lld not divisible by group_size %lld", (long long)k, (long long)group_size);
    if (n * k > 0 && (!q_dev || !scale_dev || !zp_dev)) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    nnq_gq_weight *w = nullptr;
    const int64_t groups = k / group_size;
    s = gq_alloc(ctx, n, k, bits, (int)group_size, groups, 1, &w);
    if (s != NNQ_OK) return s;
    float big = 0.0f;
    if (n * k > 0) {
        unsigned *zmax = nullptr;
        s = check_cuda(ctx, cudaGetSymbolAddress((void **)&zmax, g_gq_zpmax), "zero point bound");
        if (s == NNQ_OK) s = check_cuda(ctx, cudaMemsetAsync(zmax, 0, sizeof(unsigned), st), "zero point bound clear");
        if (s == NNQ_OK) s = check_cuda(ctx, cudaMemcpyAsync(w->codes, q_dev, w->code_bytes, cudaMemcpyDeviceToDevice, st), "codes copy");
        if (s == NNQ_OK) s = check_cuda(ctx, cudaMemcpyAsync(w->scale, scale_dev, (size_t)(n * groups) * 4, cudaMemcpyDeviceToDevice, st), "scales copy");
        if (s == NNQ_OK) {
            gq_zp_to_f32_kernel<<<grid_for(ctx, n * groups, kGqThreads), kGqThreads, 0, st>>>(zp_dev, n * groups, w->zpf);
            ctx->launches++;
            s = check_cuda(ctx, cudaGetLastError(), "zero point conversion launch");
        }
        unsigned bits_max = 0;
        if (s == NNQ_OK) s = check_cuda(ctx, cudaMemcpyAsync(&bits_max, zmax, sizeof(unsigned), cudaMemcpyDeviceToHost, st), "zero point bound read");
        if (s == NNQ_OK) s = check_cuda(ctx, cudaStreamSynchronize(st), "weight creation synchronize");
        if (s != NNQ_OK) { nnq_gq_destroy(w); return s; }
        memcpy(&big, &bits_max, 4);
    }
    gq_set_fast(w, big);
    *out = w;
    return NNQ_OK;
}

nnq_status nnq_gq_create_gptq(nnq_ctx *ctx, const uint32_t *qweight_dev, const float *scales_dev, const uint32_t *qzeros_dev,
                              int64_t n, int64_t k, int64_t groups, int64_t group_size, void *stream, nnq_gq_weight **out) {
    if (!ctx || !out) return NNQ_ERR_INVALID_ARG;
    *out = nullptr;
    if (n < 0 || k < 0 || groups < 0 || group_size <= 0 || group_size > 0x7fffffff) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad GPTQ weight arguments");
    if (k % 8 != 0 || n % 8 != 0) return fail(ctx, NNQ_ERR_SHAPE_MISMATCH, "GPTQ weight: in_features %lld and out_features %lld must be multiples of 8", (long long)k, (long long)n);
    if (groups != (k + group_size - 1) / group_size)
        return fail(ctx, NNQ_ERR_DATA_LENGTH, "GPTQ weight: %lld groups, expected %lld", (long long)groups, (long long)((k + group_size - 1) / group_size));
    if (n * k > 0 && (!qweight_dev || !scales_dev || !qzeros_dev)) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    nnq_gq_weight *w = nullptr;
    s = gq_alloc(ctx, n, k, 4, (int)group_size, groups, 0, &w);
    if (s != NNQ_OK) return s;
    if (n * k > 0) {
        // [k / 8, n] words -> [n, k / 8] words: a word keeps its 8 consecutive in-features
        dim3 grid((unsigned)((n + 31) / 32), (unsigned)((k / 8 + 31) / 32));
        gq_transpose_u32_kernel<<<grid, 256, 0, st>>>(qweight_dev, k / 8, n, reinterpret_cast<uint32_t *>(w->codes));
        gq_gptq_params_kernel<<<grid_for(ctx, n * groups, kGqThreads), kGqThreads, 0, st>>>(scales_dev, qzeros_dev, n, groups, w->scale, w->zpf);
        ctx->launches += 2;
        s = check_cuda(ctx, cudaGetLastError(), "GPTQ repack launch");
        if (s == NNQ_OK) s = check_cuda(ctx, cudaStreamSynchronize(st), "weight creation synchronize");
        if (s != NNQ_OK) { nnq_gq_destroy(w); return s; }
    }
    gq_set_fast(w, 15.0f);
    *out = w;
    return NNQ_OK;
}

nnq_status nnq_gq_info(const nnq_gq_weight *w, int64_t *n, int64_t *k, int *bits, int64_t *group_size, int64_t *groups, int *streaming) {
    if (!w) return NNQ_ERR_INVALID_ARG;
    if (n) *n = w->n;
    if (k) *k = w->k;
    if (bits) *bits = w->bits;
    if (group_size) *group_size = w->group_size;
    if (groups) *groups = w->groups;
    if (streaming) *streaming = w->fast;
    return NNQ_OK;
}

nnq_status nnq_gq_dequantize(nnq_gq_weight *w, float *dst_dev, void *stream) {
    if (!w) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = w->ctx;
    if (w->n == 0 || w->k == 0) return NNQ_OK;
    if (!dst_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    return check_cuda(ctx, launch_decode<float, float>(ctx, w->codes, w->scale, w->zpf, w->n, w->k, w->groups, w->group_size, w->bits, w->is_signed, dst_dev, (cudaStream_t)stream),
                      "group weight dequantize launch");
}

nnq_status nnq_gq_linear(nnq_gq_weight *w, const void *x_dev, nnq_dtype x_dt, int64_t m, const float *bias_dev, void *y_dev,
                         nnq_dtype y_dt, void *stream) {
    if (!w) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = w->ctx;
    if (m < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative size");
    if ((int)x_dt < 0 || x_dt > NNQ_BF16 || (int)y_dt < 0 || y_dt > NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown dtype");
    if (m == 0 || w->n == 0) return NNQ_OK;
    if (!y_dev || (w->k && !x_dev)) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t n = w->n, k = w->k;
    // from 17 tokens on: one decode to bf16 in the context's scratch, then the tensor-core product
    if (m > 16 && k >= 64 && k % 64 == 0 && ctx->d_dense && (size_t)n * (size_t)k * 2 <= ctx->dense_bytes && ctx->path != NNQ_PATH_GENERIC) {
        s = check_cuda(ctx, launch_decode<__nv_bfloat16, float>(ctx, w->codes, w->scale, w->zpf, n, k, w->groups, w->group_size, w->bits, w->is_signed,
                                                                reinterpret_cast<__nv_bfloat16 *>(ctx->d_dense), st), "bf16 decode launch");
        if (s != NNQ_OK) return s;
        TcArgs a = {reinterpret_cast<const uint8_t *>(ctx->d_dense), nullptr, x_dev, bias_dev, y_dev, m, n, k, NNQ_BF16_DENSE, (int)x_dt, (int)y_dt};
        if (gemm_dense_shape_ok(ctx, m, n, k, x_dt)) return launch_gemm_dense_bf16(ctx, ctx->d_dense, a, st);
        return launch_gemm_tc(ctx, a, st);
    }
    if (w->fast && !((uintptr_t)x_dev & 15u) && ctx->path != NNQ_PATH_GENERIC) {
        if (w->bits == 4) {
            if (x_dt == NNQ_F32) launch_fast<4, float>(w, x_dev, bias_dev, y_dev, y_dt, m, st);
            else launch_fast<4, __nv_bfloat16>(w, x_dev, bias_dev, y_dev, y_dt, m, st);
        } else {
            if (x_dt == NNQ_F32) launch_fast<8, float>(w, x_dev, bias_dev, y_dev, y_dt, m, st);
            else launch_fast<8, __nv_bfloat16>(w, x_dev, bias_dev, y_dev, y_dt, m, st);
        }
        return check_cuda(ctx, cudaGetLastError(), "group weight product launch");
    }
    const int grid = grid_for(ctx, m * n, kGqLinThreads / 32);
    if (x_dt == NNQ_F32)
        gq_linear_generic_kernel<float><<<grid, kGqLinThreads, 0, st>>>(w->codes, w->scale, w->zpf, w->groups, w->group_size, w->bits, w->is_signed,
                                                                        (const float *)x_dev, bias_dev, y_dev, y_dt, m, n, k);
    else
        gq_linear_generic_kernel<__nv_bfloat16><<<grid, kGqLinThreads, 0, st>>>(w->codes, w->scale, w->zpf, w->groups, w->group_size, w->bits, w->is_signed,
                                                                                (const __nv_bfloat16 *)x_dev, bias_dev, y_dev, y_dt, m, n, k);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "group weight product launch");
}

void nnq_gq_destroy(nnq_gq_weight *w) {
    if (!w) return;
    cudaSetDevice(w->ctx->device);
    cudaFree(w->codes);
    cudaFree(w->scale);
    cudaFree(w->zpf);
    delete w;
}

nnq_status nnq_gptq_unpack_qweight(nnq_ctx *ctx, const uint32_t *packed_dev, int64_t rows, int64_t cols, float *dst_dev, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (rows < 0 || cols < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative size");
    if (rows == 0 || cols == 0) return NNQ_OK;
    if (!packed_dev || !dst_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    gq_unpack_rows_kernel<<<grid_for(ctx, rows * cols, kGqThreads), kGqThreads, 0, (cudaStream_t)stream>>>(packed_dev, rows, cols, dst_dev);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "GPTQ unpack launch");
}

nnq_status nnq_gptq_unpack_qzeros(nnq_ctx *ctx, const uint32_t *packed_dev, int64_t groups, int64_t cols, float *dst_dev, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (groups < 0 || cols < 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "negative size");
    if (groups == 0 || cols == 0) return NNQ_OK;
    if (!packed_dev || !dst_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    if ((uintptr_t)dst_dev & 15u) return fail(ctx, NNQ_ERR_INVALID_ARG, "output must be 16-byte aligned");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    gq_unpack_cols_kernel<<<grid_for(ctx, groups * cols, kGqThreads), kGqThreads, 0, (cudaStream_t)stream>>>(packed_dev, groups * cols, dst_dev);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "GPTQ zero point unpack launch");
}

nnq_status nnq_gptq_dequantize(nnq_ctx *ctx, const float *q_dev, const float *scales_dev, const float *zeros_dev, int64_t k,
                               int64_t n, int64_t groups, int64_t group_size, float *dst_dev, void *stream) {
    if (!ctx) return NNQ_ERR_INVALID_ARG;
    if (k < 0 || n < 0 || groups < 0 || group_size <= 0) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad GPTQ dequantize arguments");
    if (groups != (k + group_size - 1) / group_size)
        return fail(ctx, NNQ_ERR_DATA_LENGTH, "dequantize_gptq: %lld groups, expected %lld", (long long)groups, (long long)((k + group_size - 1) / group_size));
    if (k == 0 || n == 0) return NNQ_OK;
    if (!q_dev || !scales_dev || !zeros_dev || !dst_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    gq_gptq_dequantize_kernel<<<grid_for(ctx, k * n, kGqThreads), kGqThreads, 0, (cudaStream_t)stream>>>(q_dev, scales_dev, zeros_dev, k, n, group_size, dst_dev);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "GPTQ dequantize launch");
}

}  // extern "C"
