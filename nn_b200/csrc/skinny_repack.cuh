// One-time repack of raw blocks into the tiled layouts (Q4_K lives with its kernel in skinny_m1.cuh).
#pragma once
#include "skinny_mn.cuh"

namespace nnq {

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

}  // namespace nnq
