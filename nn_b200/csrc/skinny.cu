// Skinny (decode, M = 1) streaming kernels for Q4_K weights on the tiled "T16" layout.
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

#include "decode.cuh"
#include "skinny.h"

namespace nnq {

constexpr int kTileBytes = 2304;
constexpr int kWarps = 8;               // warps per CTA = row tiles per CTA
constexpr size_t kPartialFloats = 2u << 20;   // 8 MiB split-K workspace
constexpr size_t kCounters = 1u << 16;

struct SkinnyJobDev {
    const uint8_t *tiled;
    const void *x;
    const float *bias;
    void *y;
    int n;            // real rows
    int row_tiles;    // ceil(n / 16)
    int kblocks;      // K / 256
    int kc;           // super-blocks per k-chunk
    int ksplit;       // ceil(kblocks / kc)
    int cta_begin;    // first CTA of this job
    int group_begin;  // first row-group (arrival counter) of this job
    int partial_begin;  // first float of this job in the split-K workspace
};

struct SkinnyParams {
    SkinnyJobDev job[kSkinnyMaxJobs];
    int njobs;
    int y_dt;
    float *partials;
    unsigned int *counters;
    int *status;
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
template <bool F32X>
struct SmemLayout {
    static constexpr int kMaxKC = F32X ? 4 : 8;
    static constexpr int kImgBytes = kMaxKC * 4096;
    static constexpr int kImgParts = F32X ? 2 : 1;
    static constexpr int kTabOff = kImgBytes * kImgParts;
    static constexpr int kTabBytes = kMaxKC * 4 * 16;
    static constexpr int kRedOff = kTabOff + kTabBytes;  // amax per warp, then the split-K flag
    static constexpr int kTotal = kRedOff + 64;
};

struct TileRegs {
    uint4 q[4];
    uint4 hg, hg8;
};

__device__ __forceinline__ void load_tile(TileRegs &r, const uint4 *tile, int lane, int g) {
#pragma unroll
    for (int p = 0; p < 4; p++) r.q[p] = __ldg(tile + 16 + 32 * p + lane);
    r.hg = __ldg(tile + g);
    r.hg8 = __ldg(tile + 8 + g);
}

template <bool F32X>
__device__ __forceinline__ void tile_mac(const TileRegs &r, const uint8_t *img_hi, const uint8_t *img_lo,
                                         const float *tab, int lane, int t, const Consts &K, float &yg,
                                         float &yg8) {
    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const uint2 *bh = reinterpret_cast<const uint2 *>(img_hi) + lane;
    const uint2 *bl = reinterpret_cast<const uint2 *>(img_lo) + lane;
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const uint32_t w0 = r.q[p].x, w1 = r.q[p].y, w2 = r.q[p].z, w3 = r.q[p].w;
        const uint32_t v0 = w0 >> 8, v1 = w1 >> 8, v2 = w2 >> 8, v3 = w3 >> 8;
        uint32_t a[4][4] = {
            {and_or(w0, K.mlo, K.k1024), and_or(w1, K.mlo, K.k1024), and_or(w2, K.mlo, K.k1024), and_or(w3, K.mlo, K.k1024)},
            {and_or(w0, K.mhi, K.k64), and_or(w1, K.mhi, K.k64), and_or(w2, K.mhi, K.k64), and_or(w3, K.mhi, K.k64)},
            {and_or(v0, K.mlo, K.k1024), and_or(v1, K.mlo, K.k1024), and_or(v2, K.mlo, K.k1024), and_or(v3, K.mlo, K.k1024)},
            {and_or(v0, K.mhi, K.k64), and_or(v1, K.mhi, K.k64), and_or(v2, K.mhi, K.k64), and_or(v3, K.mhi, K.k64)}};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            mma_f16(c, a[e][0], a[e][1], a[e][2], a[e][3], bh[(4 * p + e) * 32]);
            if (F32X) mma_f16(c, a[e][0], a[e][1], a[e][2], a[e][3], bl[(4 * p + e) * 32]);
        }
    }
    // c[0], c[1]: row g, sub-blocks 2t, 2t+1; c[2], c[3]: row g+8
    const float4 tb = *reinterpret_cast<const float4 *>(tab + t * 4);
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint4 &hd = h ? r.hg8 : r.hg;
        uint32_t p01 = __byte_perm(hd.x, hd.y, 0x0073);
        uint32_t p23 = __byte_perm(hd.z, hd.w, 0x0073);
        uint32_t dd = __byte_perm(p01, p23, 0x5410);
        float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&dd));
        uint32_t o = sel4(hd, t);
        float sc0 = (float)(o & 63u), sc1 = (float)((o >> 6) & 63u);
        float mn0 = (float)((o >> 12) & 63u), mn1 = (float)((o >> 18) & 63u);
        float dot = sc0 * (c[2 * h] - tb.x) + sc1 * (c[2 * h + 1] - tb.y);
        float mins = mn0 * tb.z + mn1 * tb.w;
        float v = dm.x * dot - dm.y * mins;
        if (h) yg8 += v; else yg += v;
    }
}

template <bool F32X>
__global__ void __launch_bounds__(kWarps * 32, 2)
skinny_q4k_m1_kernel(const __grid_constant__ SkinnyParams P) {
    using L = SmemLayout<F32X>;
    __shared__ __align__(16) uint8_t smem[L::kTotal];
    uint8_t *img_hi = smem;
    uint8_t *img_lo = smem + L::kImgBytes;
    float *tab = reinterpret_cast<float *>(smem + L::kTabOff);
    float *red = reinterpret_cast<float *>(smem + L::kRedOff);
    int *flag = reinterpret_cast<int *>(smem + L::kRedOff + 32);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // ---- which job / row group / k-chunk ----
    int j = 0;
#pragma unroll
    for (int i = 1; i < kSkinnyMaxJobs; i++)
        if (i < P.njobs && (int)blockIdx.x >= P.job[i].cta_begin) j = i;
    const SkinnyJobDev &J = P.job[j];
    const int local = blockIdx.x - J.cta_begin;
    const int s = local % J.ksplit;
    const int rg = local / J.ksplit;
    const int kb0 = s * J.kc;
    const int nkb = min(J.kc, J.kblocks - kb0);
    const int rt = rg * kWarps + warp;
    const bool live = rt < J.row_tiles;

    // ---- weights first: they do not depend on anything an earlier kernel produced ----
    const uint4 *tile = reinterpret_cast<const uint4 *>(J.tiled + ((size_t)(live ? rt : 0) * J.kblocks + kb0) * kTileBytes);
    TileRegs r0, r1;
    if (live) {
        load_tile(r0, tile, lane, g);
        if (nkb > 1) load_tile(r1, tile + kTileBytes / 16, lane, g);
    }

    // ---- zero pattern of the activation image ----
    {
        uint4 z = make_uint4(0, 0, 0, 0);
        uint4 *zi = reinterpret_cast<uint4 *>(smem);
        const int n16 = nkb * 256 * L::kImgParts;
        if (!F32X) {
            for (int i = tid; i < nkb * 256; i += kWarps * 32) zi[i] = z;
        } else {
            for (int i = tid; i < nkb * 256; i += kWarps * 32) {
                zi[i] = z;
                zi[L::kImgBytes / 16 + i] = z;
            }
        }
        (void)n16;
    }

    // ---- activations: 8 consecutive elements per thread (the k-chunk has at most 2048) ----
    const int i0 = tid * 8;
    const bool has_x = i0 < nkb * 256;
    float xv[8];
#pragma unroll
    for (int k = 0; k < 8; k++) xv[k] = 0.0f;
    if (has_x) {
        const size_t src = (size_t)kb0 * 256 + i0;
        if (F32X) {
            const float4 *xp = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(J.x) + src);
            float4 a = __ldg(xp), b = __ldg(xp + 1);
            xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w; xv[4] = b.x; xv[5] = b.y; xv[6] = b.z; xv[7] = b.w;
        } else {
            uint4 v = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(J.x) + src));
            uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                xv[2 * k] = __uint_as_float(w[k] << 16);
                xv[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
            }
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; k++) amax = fmaxf(amax, fabsf(xv[k]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    if (lane == 0) red[warp] = amax;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < kWarps; w++) amax = fmaxf(amax, red[w]);
    // power-of-two prescale so that the chunk's largest |x| lands in [1, 2): exact, keeps fp16 in range
    uint32_t ex = (__float_as_uint(amax) >> 23) & 0xFFu;
    ex = amax > 0.0f && ex < 255u ? min(max(ex, 1u), 253u) : 127u;
    const float scale = __uint_as_float((254u - ex) << 23);
    const float inv_scale = __uint_as_float(ex << 23);
    {
        uint32_t ph[4], pl[4];
        float xr[8];  // the value the MMAs will see
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
        // this thread holds word tt of sub-block sb8 of super-block kbl
        const int sbk = i0 >> 5, kbl = sbk >> 3, sb8 = sbk & 7, tt = tid & 3;
        if (has_x) {
            uint32_t *dst = reinterpret_cast<uint32_t *>(img_hi + kbl * 4096 + (sb8 >> 1) * 1024) + (4 * sb8 + tt) * 2 + (sb8 & 1);
#pragma unroll
            for (int e = 0; e < 4; e++) dst[e * 64] = ph[e];
            if (F32X) {
                uint32_t *dl = reinterpret_cast<uint32_t *>(img_lo + kbl * 4096 + (sb8 >> 1) * 1024) + (4 * sb8 + tt) * 2 + (sb8 & 1);
#pragma unroll
                for (int e = 0; e < 4; e++) dl[e * 64] = pl[e];
            }
        }
        // elements 0,1,4,5 of each group of 8 carry offset 1024, elements 2,3,6,7 offset 64
        float sa = (xr[0] + xr[1]) + (xr[4] + xr[5]);
        float sb = (xr[2] + xr[3]) + (xr[6] + xr[7]);
        float ox = 1024.0f * sa + 64.0f * sb;
        float sx = sa + sb;
        ox += __shfl_xor_sync(0xFFFFFFFFu, ox, 1);
        sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 1);
        ox += __shfl_xor_sync(0xFFFFFFFFu, ox, 2);
        sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 2);
        if (has_x && tt == 0) {
            float *e = tab + (kbl * 4 + (sb8 >> 1)) * 4 + (sb8 & 1);
            e[0] = ox;
            e[2] = sx;
        }
    }
    __syncthreads();

    // ---- main loop over the super-blocks of this k-chunk, two register sets in turn ----
    float yg = 0.0f, yg8 = 0.0f;
    if (live) {
        Consts K;
        K.init();
        for (int kbl = 0; kbl < nkb; kbl += 2) {
            tile_mac<F32X>(r0, img_hi + kbl * 4096, img_lo + kbl * 4096, tab + kbl * 16, lane, t, K, yg, yg8);
            if (kbl + 2 < nkb) load_tile(r0, tile + (kbl + 2) * (kTileBytes / 16), lane, g);
            if (kbl + 1 < nkb) {
                tile_mac<F32X>(r1, img_hi + (kbl + 1) * 4096, img_lo + (kbl + 1) * 4096, tab + (kbl + 1) * 16, lane, t, K, yg, yg8);
                if (kbl + 3 < nkb) load_tile(r1, tile + (kbl + 3) * (kTileBytes / 16), lane, g);
            }
        }
        yg += __shfl_xor_sync(0xFFFFFFFFu, yg, 1);
        yg8 += __shfl_xor_sync(0xFFFFFFFFu, yg8, 1);
        yg += __shfl_xor_sync(0xFFFFFFFFu, yg, 2);
        yg8 += __shfl_xor_sync(0xFFFFFFFFu, yg8, 2);
        yg *= inv_scale;
        yg8 *= inv_scale;
    }

    // ---- output ----
    const int npad = J.row_tiles * 16;
    auto store = [&](int row, float v) {
        if (row < J.n) {
            if (J.bias) v += __ldg(J.bias + row);
            if (P.y_dt == NNQ_F32) reinterpret_cast<float *>(J.y)[row] = v;
            else reinterpret_cast<__nv_bfloat16 *>(J.y)[row] = __float2bfloat16_rn(v);
        }
    };
    if (J.ksplit == 1) {
        if (live && t == 0) {
            store(rt * 16 + g, yg);
            store(rt * 16 + 8 + g, yg8);
        }
        return;
    }
    // split-K: publish this chunk's partial sums; the last CTA of the row group to arrive adds
    // the chunks in order (deterministic) and writes the output.
    float *part = P.partials + J.partial_begin;
    if (live && t == 0) {
        part[(size_t)s * npad + rt * 16 + g] = yg;
        part[(size_t)s * npad + rt * 16 + 8 + g] = yg8;
    }
    __syncthreads();
    unsigned int *counter = P.counters + J.group_begin + rg;
    if (tid == 0) {
        __threadfence();  // cumulative: orders the CTA's partial sums (seen through the barrier) first
        unsigned int old = atomicAdd(counter, 1u);
        *flag = (old == (unsigned int)J.ksplit - 1u);
        if (*flag) __threadfence();
    }
    __syncthreads();
    if (!*flag) return;
    if (tid < kWarps * 16) {
        int row = rg * kWarps * 16 + tid;
        if (row < npad) {
            float v = 0.0f;
            for (int ss = 0; ss < J.ksplit; ss++) v += __ldcg(part + (size_t)ss * npad + row);
            store(row, v);
        }
    }
    if (tid == 0) *counter = 0u;  // ready for the next launch
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------

nnq_status skinny_init(nnq_ctx *ctx) {
    nnq_status s = check_cuda(ctx, cudaMalloc(&ctx->d_partials, kPartialFloats * sizeof(float)), "cudaMalloc split-K workspace");
    if (s != NNQ_OK) return s;
    ctx->partials_bytes = kPartialFloats * sizeof(float);
    s = check_cuda(ctx, cudaMalloc(&ctx->d_counters, kCounters * sizeof(unsigned int)), "cudaMalloc counters");
    if (s != NNQ_OK) return s;
    ctx->counters_count = kCounters;
    return check_cuda(ctx, cudaMemset(ctx->d_counters, 0, kCounters * sizeof(unsigned int)), "cudaMemset counters");
}

nnq_status build_tiled(nnq_ctx *ctx, nnq_weight *w) {
    if (w->fmt != NNQ_Q4_K && w->fmt != NNQ_Q4_K_GGML) return NNQ_OK;
    if (w->n == 0 || w->k == 0 || w->k % 256 != 0) return NNQ_OK;
    if (w->n > (1 << 24) || w->k > (1 << 24)) return NNQ_OK;
    int kblocks = (int)(w->k / 256);
    int64_t row_tiles = (w->n + 15) / 16;
    size_t bytes = (size_t)row_tiles * kblocks * kTileBytes;
    nnq_status s = check_cuda(ctx, cudaMalloc(&w->d_tiled, bytes), "cudaMalloc tiled weight");
    if (s != NNQ_OK) return s;
    w->tiled_bytes = bytes;
    if (w->n % 16) {
        s = check_cuda(ctx, cudaMemset(w->d_tiled, 0, bytes), "cudaMemset tiled weight");
        if (s != NNQ_OK) return s;
    }
    int64_t total = w->n * kblocks * 8;
    int grid = (int)((total + 255) / 256);
    if (w->fmt == NNQ_Q4_K)
        repack_q4k_kernel<false><<<grid, 256>>>(w->d_raw, w->d_tiled, (int)w->n, kblocks);
    else
        repack_q4k_kernel<true><<<grid, 256>>>(w->d_raw, w->d_tiled, (int)w->n, kblocks);
    ctx->launches++;
    s = check_cuda(ctx, cudaGetLastError(), "repack launch");
    if (s != NNQ_OK) return s;
    s = check_cuda(ctx, cudaDeviceSynchronize(), "repack");
    if (s != NNQ_OK) return s;
    w->tiled_layout = kTiledQ4K;
    return NNQ_OK;
}

bool skinny_supported(const nnq_weight *w, int64_t m) {
    return w && w->tiled_layout == kTiledQ4K && m == 1;
}

nnq_status launch_skinny(nnq_ctx *ctx, const SkinnyJob *jobs, int count, int x_dt, int64_t m, int y_dt,
                         cudaStream_t stream) {
    if (count < 1 || count > kSkinnyMaxJobs) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad job count %d", count);
    if (m != 1) return fail(ctx, NNQ_ERR_UNSUPPORTED, "skinny kernel covers M = 1 only");
    SkinnyParams P;
    memset(&P, 0, sizeof(P));
    P.njobs = count;
    P.y_dt = y_dt;
    P.partials = ctx->d_partials;
    P.counters = ctx->d_counters;
    P.status = ctx->d_status;
    // k-chunk length: enough warps to cover the machine a few times over, at most kMaxKC
    int64_t tiles = 0;
    for (int i = 0; i < count; i++) tiles += ((jobs[i].w->n + 15) / 16) * (jobs[i].w->k / 256);
    int64_t warps_target = (int64_t)ctx->sm_count * 16;
    int kc_want = (int)((tiles + warps_target - 1) / warps_target);
    if (kc_want < 1) kc_want = 1;
    const int kc_max = x_dt == NNQ_F32 ? SmemLayout<true>::kMaxKC : SmemLayout<false>::kMaxKC;
    if (kc_want > kc_max) kc_want = kc_max;
    int cta = 0, group = 0;
    size_t part = 0;
    for (int i = 0; i < count; i++) {
        const nnq_weight *w = jobs[i].w;
        SkinnyJobDev &J = P.job[i];
        J.tiled = w->d_tiled;
        J.x = jobs[i].x;
        J.bias = jobs[i].bias;
        J.y = jobs[i].y;
        J.n = (int)w->n;
        J.row_tiles = (int)((w->n + 15) / 16);
        J.kblocks = (int)(w->k / 256);
        J.kc = kc_want < J.kblocks ? kc_want : J.kblocks;
        J.ksplit = (J.kblocks + J.kc - 1) / J.kc;
        J.kc = (J.kblocks + J.ksplit - 1) / J.ksplit;  // even out the chunks
        J.ksplit = (J.kblocks + J.kc - 1) / J.kc;
        int groups = (J.row_tiles + kWarps - 1) / kWarps;
        J.cta_begin = cta;
        J.group_begin = group;
        J.partial_begin = (int)part;
        cta += groups * J.ksplit;
        group += groups;
        if (J.ksplit > 1) part += (size_t)J.ksplit * J.row_tiles * 16;
    }
    if (part > kPartialFloats || (size_t)group > kCounters)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "split-K workspace too small for this launch");
    if (x_dt == NNQ_F32)
        skinny_q4k_m1_kernel<true><<<cta, kWarps * 32, 0, stream>>>(P);
    else
        skinny_q4k_m1_kernel<false><<<cta, kWarps * 32, 0, stream>>>(P);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "skinny launch");
}

}  // namespace nnq
