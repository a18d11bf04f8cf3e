// Prefill product (M > 16) on the 5th-generation tensor cores: y[M, N] = x[M, K] * W[N, K]^T (+ bias)
// with block-quantized W of any format.
//
// One CTA computes a (128 * MT) x 128 output tile (MT = 1, 2 or 4 accumulators of 128 x 128 f32
// in tensor memory). Per 64-wide k step
//   * the (128 * MT) x 64 bf16 activation tile arrives by TMA (cp.async.bulk.tensor.2d through a
//     tensor map of x with 128-byte swizzle, issued by one thread, counted on the stage's "full"
//     barrier; rows beyond M are zero-filled); f32 activations are converted by the producers;
//   * 8 producer warps dequantize the 128 x 64 weight tile to bf16 (f32 decode, the bit-exact
//     one, then round-to-nearest-even) into the same K-major 128-byte-swizzled layout; up to
//     three such groups of warps take k steps in turn (with one group an SM held two warps per
//     scheduler and the decode's dependent chains, not its instruction count, set the pace of a
//     k step); Q4_K and Q8_0 blocks reach them through a TMA ring in shared memory (below);
//   * one thread issues 4 * MT tcgen05.mma (M 128, N 128, K 16, bf16 x bf16 -> f32) from shared
//     memory descriptors into the accumulators and commits them onto the stage's "empty" barrier.
// The larger MT, the more activation rows reuse each dequantized weight tile (the dequantization,
// not the MMA, is the expensive part at small M); where that leaves few tiles, K is split over
// gridDim.z CTAs and a second kernel adds the partial sums in slice order. After the last k step
// sixteen warps read the accumulators back with tcgen05.ld, turn them through shared memory, add
// the bias and store coalesced rows of f32 / bf16.
// Weights are rounded to bf16, so results carry the 1e-2 tolerance of the tensor path.
// Every barrier wait is bounded; on a timeout the CTA records it, skips the rest and still frees
// its tensor memory.
#include <cuda.h>
#include <cuda_bf16.h>

#include "decode.cuh"
#include "gemm_tc.h"
#include <stdlib.h>
#include <string.h>

#include "sync.cuh"

namespace nnq {

constexpr int kTcProducerWarps = 8;          // warps that decode one weight tile
constexpr int kTcGroups = 3;                 // producer groups (at most); group g of G fills the k steps g, g + G, ...
constexpr int kTcMmaWarp = kTcProducerWarps * kTcGroups;
constexpr int kTcLoadWarp = kTcMmaWarp + 1;  // streams the raw blocks of formats that take the raw ring
constexpr int kTcThreads = (kTcLoadWarp + 1) * 32;
constexpr int kTcBK = 64;                    // k per stage: one 128-byte swizzle row of bf16
constexpr int kTcTileBytes = 128 * 128;      // 128 rows x 128 bytes
constexpr int kTcEpiWarps = 16;                 // warps that carry the accumulators out (four per TMEM lane quarter)
constexpr int kTcEpiBytes = kTcEpiWarps * 32 * 33 * 4;   // epilogue staging: a 32 x 32 f32 block (+ pad) per warp

// Raw ring (Q4_K in both element orders, Q8_0): the raw blocks of the CTA's 128 weight rows arrive by TMA
// (the raw tensor seen as rows of 32-bit words): per box, of every row, one or two 144-byte Q4_K
// super-blocks or eight 34-byte Q8_0 blocks (256 weights = 4 k steps each), one copy per box and two boxes
// in flight. Per-thread register loads of the 32 bytes a k step needs kept less than a megabyte in flight
// on the whole device, and the memory system's latency, not the decode, set the pace (0.47 TB/s of reads in
// the profile of a 128-row product); a bulk copy per row (128 per box) was bound by the rate at which the
// copy unit takes small copies. Q8_0 rows are whole 32-bit words (and boxes start on 16 bytes) only when
// K is a multiple of 256: other K, and the 512-row tile (no room for the ring), load from global memory.
template <int FMT, int MT>
struct TcRawGeom {
    static constexpr bool kQ8 = FMT == NNQ_Q8_0;
    static constexpr bool kRing = FMT == NNQ_Q4_K || FMT == NNQ_Q4_K_GGML || (kQ8 && MT <= 2);
    static constexpr int kUnitBytes = kQ8 ? 272 : 144;              // bytes of a row per 256 weights
    static constexpr int kSB = (kQ8 || MT == 4) ? 1 : 2;            // units of a row per box
    static constexpr int kKb = 4 * kSB;                             // k steps per box
    static constexpr int kPitch = kUnitBytes * kSB;                 // the box is stored densely
    static constexpr int kBytes = 128 * kPitch;                     // one box (a multiple of 1024)
};
// does a product of this format and K take the ring (given a tile size that has one)?
static inline bool tc_raw_ring(int fmt, int64_t k) {
    return fmt == NNQ_Q4_K || fmt == NNQ_Q4_K_GGML || (fmt == NNQ_Q8_0 && k % 256 == 0);
}
static inline int tc_raw_unit_bytes(int fmt) { return fmt == NNQ_Q8_0 ? 272 : 144; }
template <int FMT, int MT>
__host__ __device__ constexpr int tc_ring_bytes() { return TcRawGeom<FMT, MT>::kRing ? 2 * TcRawGeom<FMT, MT>::kBytes : 0; }
template <int FMT, int MT>
constexpr int tc_max_stages() { return TcRawGeom<FMT, MT>::kRing ? (MT == 4 ? 2 : (MT == 2 ? 3 : 4)) : (MT == 4 ? 2 : (MT == 2 ? 4 : 6)); }
template <int FMT, int MT>
static int tc_smem_bytes(int stages) {
    const int tiles = stages * (MT + 1) * kTcTileBytes;
    return 1024 + tc_ring_bytes<FMT, MT>() + (tiles > kTcEpiBytes ? tiles : kTcEpiBytes);
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint32_t lo = ((addr >> 4) & 0x3FFFu) | (1u << 16);           // start address, leading byte offset (unused) = 1
    uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);          // stride byte offset, descriptor version 1, SWIZZLE_128B
    return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx_only(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// one 64 x 128 box (k0 .. k0+63, rows r0 .. r0+127) of the activation tensor -> swizzled shared tile
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int k0, int r0, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(k0), "r"(r0), "r"(bar) : "memory");
}

// byte offset of 16-byte chunk c (0..7) of row r (0..127) inside a swizzled 128 x 128-byte tile
__device__ __forceinline__ uint32_t swz(int r, int c) {
    return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
}

// Grouped launches (expert products): rows sorted by expert, blockIdx.y numbers the row tiles of
// all experts (expert-major); offsets == NULL means a plain product.
struct TcGroup {
    const int *offsets;
    int experts;
    size_t w_stride, s_stride;
};

template <int FMT, int MT, typename XT, bool TMAX>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const uint8_t *__restrict__ w, const uint8_t *__restrict__ wscales,
               const XT *__restrict__ x, const float *__restrict__ bias, void *__restrict__ y, int64_t M, int64_t N,
               int64_t K, int y_dt, int stages, int use_ring, float *__restrict__ partials, int *status, const TcGroup grp) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment of the tiles (the dynamic window is not guaranteed to start on one)
    uint8_t *smem_al = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    using RG = TcRawGeom<FMT, MT>;
    const bool kRawRing = RG::kRing && use_ring;   // (compile-time false for formats without a ring)
    uint8_t *rawring = smem_al;                                  // two raw chunks (ring formats only)
    uint8_t *smem = smem_al + tc_ring_bytes<FMT, MT>();          // the tile stages; reused by the epilogue
    constexpr int kStageBytes = (MT + 1) * kTcTileBytes;   // MT activation tiles, then the weight tile
    // full[stages], empty[stages], accumulators ready, raw chunk full[2], raw chunk empty[2]
    __shared__ __align__(8) uint64_t bars[2 * 8 + 1 + 4];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t n0 = (int64_t)blockIdx.x * 128;
    int64_t m0 = (int64_t)blockIdx.y * 128 * MT;
    int wrow0 = (int)n0;   // first row of this CTA's weight tile in the raw tensor map (all experts' rows)
    if (grp.offsets) {
        // which expert this row tile belongs to; row tiles beyond the last expert have nothing to do
        __shared__ int gsel[3];
        if (tid == 0) {
            int q = (int)blockIdx.y, e = -1, begin = 0, end = 0;
            for (int i = 0; i < grp.experts; i++) {
                const int lo = grp.offsets[i], hi = grp.offsets[i + 1];
                const int tiles = (hi - lo + 128 * MT - 1) / (128 * MT);
                if (q < tiles) {
                    e = i;
                    begin = lo + q * 128 * MT;
                    end = hi;
                    break;
                }
                q -= tiles;
            }
            gsel[0] = e;
            gsel[1] = begin;
            gsel[2] = end;
        }
        __syncthreads();
        if (gsel[0] < 0) return;
        m0 = gsel[1];
        M = gsel[2];                    // rows of this expert end here: later rows are not stored
        w += (size_t)gsel[0] * grp.w_stride;
        wrow0 += gsel[0] * (int)N;
        if (wscales) wscales += (size_t)gsel[0] * grp.s_stride;
        if (bias) bias += (size_t)gsel[0] * N;
    }
    // this CTA's share of the k steps (gridDim.z slices of K; partial sums go to `partials`)
    const int nkb_all = (int)(K / kTcBK);
    int kb_lo, nkb;
    if (kRawRing) {
        // slices of whole raw chunks (the host asks for no more slices than there are chunks)
        const int nch_all = (nkb_all + RG::kKb - 1) / RG::kKb;
        kb_lo = (int)(((long long)blockIdx.z * nch_all) / gridDim.z) * RG::kKb;
        const int kb_hi = (int)(((long long)(blockIdx.z + 1) * nch_all) / gridDim.z) * RG::kKb;
        nkb = (kb_hi < nkb_all ? kb_hi : nkb_all) - kb_lo;
    } else {
        kb_lo = (int)(((long long)blockIdx.z * nkb_all) / gridDim.z);
        nkb = (int)(((long long)(blockIdx.z + 1) * nkb_all) / gridDim.z) - kb_lo;
    }
    const uint32_t full_s = smem_u32(bars), empty_s = full_s + 8 * 8, acc_s = full_s + 16 * 8;
    const uint32_t rawfull_s = full_s + 17 * 8, rawempty_s = full_s + 19 * 8;
    constexpr uint32_t kTmemCols = 128 * MT;

    if (tid == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(full_s + 8 * s, kTcProducerWarps);
            mbar_init(empty_s + 8 * s, 1);
        }
        mbar_init(acc_s, 1);
        for (int b = 0; b < 2; b++) {
            mbar_init(rawfull_s + 8 * b, 1);
            mbar_init(rawempty_s + 8 * b, kTcProducerWarps * (stages >= kTcGroups ? kTcGroups : 2));
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTcMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    bool ok = true;
    // Producer groups in use: never more than stages. A group waits for "the stage was freed u times" by
    // parity, which is only right while it cannot be two uses ahead of the tensor core; its own previous
    // k step (G steps back) was filled after the step G + stages back had been consumed, so G <= stages
    // keeps it within one use. (The 512-row tile has room for two stages: two groups, eight idle warps.)
    const int ngroups = stages >= kTcGroups ? kTcGroups : 2;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    int raw_issued = 0;   // loader warp: raw chunks whose copies were started

    if (warp < kTcProducerWarps * ngroups) {
        // ---------------- producers ----------------
        const int64_t cpr = K / 32;                 // 32-weight chunks per weight row
        const int pgroup = warp / kTcProducerWarps;             // this warp's producer group
        const int ptid = tid - pgroup * kTcProducerWarps * 32;  // thread within the group
        const int brow = ptid & 127, bhalf = ptid >> 7;   // weight tile: row and which 32 of the 64 k
        // Software pipeline: the tile data of this group's next step is decoded into registers right after
        // the current step has been handed to the tensor core, so that the work runs under the MMAs and
        // under the wait for a free stage. Ring formats decode from the raw chunk in shared memory, the
        // others load their blocks from global memory inside the decode.
        constexpr int kAChunks = (128 * MT * 8) / (kTcProducerWarps * 32);   // 16-byte activation chunks per thread
        uint4 wreg[4];
        const int ac = ptid & 7;
        auto fetch = [&](int kb) {
            float wv[32];
            if (kRawRing) {
                // k step kb of the whole product = step kl of this CTA's slice (slices start on chunk
                // boundaries, so sub-block and super-block positions follow from kl alone)
                const int kl = kb - kb_lo, lc = kl / RG::kKb, inch = kl % RG::kKb;
                if (inch < ngroups) ok = mbar_wait_fast(rawfull_s + 8 * (lc & 1), (uint32_t)(lc >> 1) & 1u);   // this group's first step in the chunk
                const uint8_t *rb = rawring + (lc & 1) * RG::kBytes + brow * RG::kPitch + (inch >> 2) * RG::kUnitBytes;
                const int j = (inch & 3) * 2 + bhalf;
                if (ok && n0 + brow < N) {
                    if (FMT == NNQ_Q4_K) {
                        Decode<NNQ_Q4_K>::chunk_regs(*reinterpret_cast<const uint4 *>(rb), *reinterpret_cast<const uint4 *>(rb + 16 + 16 * j), j, wv);
                    } else if (FMT == NNQ_Q4_K_GGML) {
                        const uint4 *qp = reinterpret_cast<const uint4 *>(rb + 16 + 32 * (j >> 1));
                        Decode<NNQ_Q4_K_GGML>::chunk_regs(*reinterpret_cast<const uint4 *>(rb), qp[0], qp[1], j, wv);
                    } else {
                        Decode<NNQ_Q8_0>::chunk_halfwords(reinterpret_cast<const uint16_t *>(rb + 34 * j), wv);   // block j of the 8
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) wv[i] = 0.0f;
                }
                if (inch + ngroups >= RG::kKb || kl + ngroups >= nkb) {   // this group's last step in the chunk
                    __syncwarp();
                    if (lane == 0) mbar_arrive(rawempty_s + 8 * (lc & 1));
                }
            } else if (n0 + brow < N) {
                Decode<FMT>::chunk(w, wscales, (n0 + brow) * cpr + (int64_t)kb * 2 + bhalf, wv);
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) wv[i] = 0.0f;
            }
#pragma unroll
            for (int c = 0; c < 4; c++)
                wreg[c] = make_uint4(pack_bf16(wv[8 * c], wv[8 * c + 1]), pack_bf16(wv[8 * c + 2], wv[8 * c + 3]),
                                     pack_bf16(wv[8 * c + 4], wv[8 * c + 5]), pack_bf16(wv[8 * c + 6], wv[8 * c + 7]));
        };
        // activation chunk i of this thread for k step kb (the path without TMA: f32 activations, or a
        // row pitch the tensor map cannot express); loaded when the stage is filled, four at a time
        auto load_a = [&](int kb, int i) {
            const int r = (ptid >> 3) + 32 * i;
            uint4 v = make_uint4(0, 0, 0, 0);
            const int64_t row = m0 + r;
            if (row < M) {
                const XT *src = x + row * K + (int64_t)kb * kTcBK + ac * 8;
                if (sizeof(XT) == 2) {
                    v = __ldg(reinterpret_cast<const uint4 *>(src));
                } else {
                    float4 fa = __ldg(reinterpret_cast<const float4 *>(src));
                    float4 fb = __ldg(reinterpret_cast<const float4 *>(src) + 1);
                    v = make_uint4(pack_bf16(fa.x, fa.y), pack_bf16(fa.z, fa.w), pack_bf16(fb.x, fb.y), pack_bf16(fb.z, fb.w));
                }
            }
            return v;
        };
        if (pgroup < nkb) fetch(kb_lo + pgroup);
        for (int kb = pgroup; kb < nkb && ok; kb += ngroups) {
            const int slot = kb % stages;
            const uint32_t phase = (uint32_t)(kb / stages) & 1u;
            if (kb >= stages) ok = mbar_wait_fast(empty_s + 8 * slot, phase ^ 1u);
            if (!ok) break;
            uint8_t *stage = smem + (size_t)slot * kStageBytes;
            uint8_t *bt = stage + MT * kTcTileBytes;
            if (kb == pgroup && (!TMAX || ptid == 0))
                asm volatile("griddepcontrol.wait;" ::: "memory");   // activations come from the kernel before this one
            if (TMAX && ptid == 0) {
                // the stage is free: let the activation tiles of this k step stream in while the
                // weight tile is written
                mbar_expect_tx_only(full_s + 8 * slot, MT * kTcTileBytes);
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
                    tma_load_2d(smem_u32(stage + mt * kTcTileBytes), &xmap, (kb_lo + kb) * kTcBK, (int)m0 + mt * 128, full_s + 8 * slot);
            }
#pragma unroll
            for (int c = 0; c < 4; c++) *reinterpret_cast<uint4 *>(bt + swz(brow, bhalf * 4 + c)) = wreg[c];
#pragma unroll
            for (int i0 = 0; i0 < (TMAX ? 0 : kAChunks); i0 += 4) {
                uint4 av[4];
#pragma unroll
                for (int j = 0; j < 4; j++) av[j] = load_a(kb_lo + kb, i0 + j);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int r = (ptid >> 3) + 32 * (i0 + j);
                    *reinterpret_cast<uint4 *>(stage + (r >> 7) * kTcTileBytes + swz(r & 127, ac)) = av[j];
                }
            }
            fence_async_smem();      // generic-proxy writes -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(full_s + 8 * slot);
            if (kb + ngroups < nkb) fetch(kb_lo + kb + ngroups);
        }
        // ---------------- epilogue ----------------
        if (ok) ok = mbar_wait_fast(acc_s, 0);
        asm volatile("griddepcontrol.wait;" ::: "memory");   // (returns at once: the activations were waited for) before any store
        if (ok && warp < kTcEpiWarps) {
            tc_fence_after();
            constexpr int kColsPerWarp = 128 / (kTcEpiWarps / 4);
            const int q = warp & 3, cpart = warp >> 2;   // TMEM lane quarter, column part
            // A lane reads one accumulator row; the block is turned through shared memory (the tile stages
            // are free by now) so that a warp stores 32 consecutive columns of one row per instruction.
            float *stg = reinterpret_cast<float *>(smem) + warp * (32 * 33);
#pragma unroll 1
            for (int mt = 0; mt < MT; mt++) {
#pragma unroll 1
                for (int cc = 0; cc < kColsPerWarp / 32; cc++) {
                    const int col0 = cpart * kColsPerWarp + cc * 32;
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * 128 + col0), v);
#pragma unroll
                    for (int i = 0; i < 32; i++) stg[lane * 33 + i] = __uint_as_float(v[i]);
                    __syncwarp();
                    const int64_t col = n0 + col0 + lane;
                    const float bv = (bias && !partials && col < N) ? __ldg(bias + col) : 0.0f;
#pragma unroll 4
                    for (int rr = 0; rr < 32; rr++) {
                        const int64_t row = m0 + mt * 128 + q * 32 + rr;
                        if (row < M && col < N) {
                            const float f = stg[rr * 33 + lane];
                            if (partials) partials[((size_t)blockIdx.z * M + row) * N + col] = f;   // bias and conversion happen in the reduction
                            else if (y_dt == NNQ_F32) reinterpret_cast<float *>(y)[row * N + col] = f + bv;
                            else reinterpret_cast<__nv_bfloat16 *>(y)[row * N + col] = __float2bfloat16_rn(f + bv);
                        }
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
        }
    } else if (warp == kTcMmaWarp && lane == 0) {
        // ---------------- MMA issuer ----------------
        // instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, N = 128, M = 128
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
        int slot = 0;
        uint32_t phase = 0;
        for (int kb = 0; kb < nkb && ok; kb++) {
            ok = mbar_wait_fast(full_s + 8 * slot, phase);
            if (!ok) break;
            tc_fence_after();
            const uint32_t stage_s = smem_u32(smem + (size_t)slot * kStageBytes);
            const uint64_t db = smem_desc(stage_s + MT * kTcTileBytes);
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const uint64_t da = smem_desc(stage_s + mt * kTcTileBytes);
#pragma unroll
                for (int k = 0; k < 4; k++)   // 16 bf16 = 32 bytes = 2 descriptor units per k step
                    umma_bf16(tmem_base + mt * 128, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
            }
            umma_commit(empty_s + 8 * slot);   // frees the stage when these MMAs have read it
            if (++slot == stages) {
                slot = 0;
                phase ^= 1u;
            }
        }
        if (ok) umma_commit(acc_s);            // accumulators complete
    } else if (RG::kRing && kRawRing && warp == kTcLoadWarp) {
        // ---------------- raw block loader ----------------
        const int nch = (nkb + RG::kKb - 1) / RG::kKb;
        const uint32_t ring_s = smem_u32(rawring);
        for (int lc = 0; lc < nch && ok; lc++) {
            const int buf = lc & 1;
            if (lc >= 2) ok = mbar_wait_fast(rawempty_s + 8 * buf, ((uint32_t)(lc >> 1) & 1u) ^ 1u);
            if (!ok) break;
            // a box of 128 rows x kSB units of 256 weights; what lies beyond the row's end or the
            // tensor's last row arrives as zeros and counts like the rest
            if (lane == 0) {
                mbar_expect_tx(rawfull_s + 8 * buf, RG::kBytes);
                tma_load_2d(ring_s + buf * RG::kBytes, &wmap, (kb_lo / 4 + lc * RG::kSB) * (RG::kUnitBytes / 4), wrow0, rawfull_s + 8 * buf);
            }
            raw_issued = lc + 1;
        }
    }
    if (!ok) {
        abort_s = 1;
        if (lane == 0) atomicExch(status, 1);
    }
    __syncthreads();
    if (RG::kRing && kRawRing && warp == kTcLoadWarp && abort_s) {
        // an aborted CTA may leave before its raw chunks were consumed: wait (bounded) for the copies
        for (int lc = raw_issued > 2 ? raw_issued - 2 : 0; lc < raw_issued; lc++) mbar_wait(rawfull_s + 8 * (lc & 1), (uint32_t)(lc >> 1) & 1u);
    }
    if (warp == kTcMmaWarp) {
        // with an aborted CTA, MMAs may still be in flight: give them a bounded chance to finish
        if (abort_s) mbar_wait(acc_s, 0);
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// y = sum over the K slices (in order) + bias
__global__ void __launch_bounds__(256)
gemm_tc_reduce_kernel(const float *__restrict__ partials, int slices, const float *__restrict__ bias, void *__restrict__ y,
                      int64_t M, int64_t N, int y_dt) {
    const int64_t total = M * N;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the partial sums of the product before this kernel
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float f = 0.0f;
        for (int z = 0; z < slices; z++) f += partials[(size_t)z * total + i];
        if (bias) f += __ldg(bias + i % N);
        if (y_dt == NNQ_F32) reinterpret_cast<float *>(y)[i] = f;
        else reinterpret_cast<__nv_bfloat16 *>(y)[i] = __float2bfloat16_rn(f);
    }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------

bool gemm_tc_supported(const nnq_weight *w, int64_t m) {
    // (the raw ring's bulk copies read 16-byte aligned super-blocks)
    return w && w->d_raw && m >= 1 && w->k >= kTcBK && w->k % kTcBK == 0 && w->n >= 1 &&
           !(tc_raw_ring(w->fmt, w->k) && ((uintptr_t)w->d_raw & 15u));
}

// Tensor map of the bf16 activations [M, K]: boxes of 64 x 128 elements, 128-byte swizzle, zero fill
// beyond M. Returns false when the driver entry point is not available (the producers then stage
// the activations themselves).
typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                             const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(p);
        cudaGetLastError();
    }
    return fn;
}
static bool make_x_map(const TcArgs &a, CUtensorMap *map) {
    EncodeFn fn = encode_fn();
    if (!fn || ((uintptr_t)a.x & 15u) || (a.k * 2) % 16) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
    const cuuint64_t strides[1] = {(cuuint64_t)a.k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTcBK, 128u};
    const cuuint32_t estr[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(a.x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor map of raw blocks as 32-bit words: [rows, K / 256 * unit_bytes / 4], boxes of 128 rows x sb units.
static bool make_w_map(const void *w, int64_t rows, int64_t k, int unit_bytes, int sb, CUtensorMap *map) {
    EncodeFn fn = encode_fn();
    const cuuint64_t row_bytes = (cuuint64_t)(k / 256) * (cuuint64_t)unit_bytes;
    if (!fn || ((uintptr_t)w & 15u) || rows < 1 || rows >= (1ll << 31)) return false;
    const cuuint64_t dims[2] = {row_bytes / 4, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(unit_bytes / 4 * sb), 128u};
    const cuuint32_t estr[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int FMT, int MT, typename XT, bool TMAX>
static cudaError_t launch_cfg(const TcArgs &a, const CUtensorMap &map, const CUtensorMap &wmap, bool ring, int *status, int ksplit, float *partials, int stages,
                              int smem_bytes, cudaStream_t stream, const TcGroup &grp = TcGroup{nullptr, 0, 0, 0}, int grid_y = 0) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<FMT, MT, XT, TMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    dim3 grid((unsigned)((a.n + 127) / 128), (unsigned)(grid_y ? grid_y : (a.m + 128 * MT - 1) / (128 * MT)), (unsigned)ksplit);
    // Plain products are launched with programmatic stream serialization: the kernel may become resident
    // while its predecessor drains, streams and decodes its first weight tiles (which depend on nothing),
    // and waits for the predecessor before it reads activations or writes anything. Grouped launches read
    // the expert offsets right away and keep the ordinary stream order.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = grp.offsets ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<FMT, MT, XT, TMAX>, map, wmap, a.w, a.scales, reinterpret_cast<const XT *>(a.x),
                              a.bias, a.y, a.m, a.n, a.k, a.y_dt, stages, ring ? 1 : 0, ksplit > 1 ? partials : (float *)nullptr, status, grp);
}

template <int FMT, int MT, typename XT>
static cudaError_t launch_one(const TcArgs &a, int *status, int ksplit, float *partials, cudaStream_t stream) {
    // one CTA per SM: as many stages as fit beside the raw ring
    int stages = tc_max_stages<FMT, MT>();
    const int nkb = (int)(a.k / kTcBK);
    if (stages > nkb / ksplit) stages = nkb / ksplit > 0 ? nkb / ksplit : 1;
    const int smem_bytes = tc_smem_bytes<FMT, MT>(stages);
    CUtensorMap map, wmap;
    memset(&map, 0, sizeof(map));
    memset(&wmap, 0, sizeof(wmap));
    using RG = TcRawGeom<FMT, MT>;
    const bool ring = RG::kRing && tc_raw_ring(FMT, a.k);
    if (ring && !make_w_map(a.w, a.n, a.k, RG::kUnitBytes, RG::kSB, &wmap)) return cudaErrorNotSupported;
    cudaError_t e;
    if (sizeof(XT) == 2 && make_x_map(a, &map))
        e = launch_cfg<FMT, MT, XT, sizeof(XT) == 2>(a, map, wmap, ring, status, ksplit, partials, stages, smem_bytes, stream);
    else
        e = launch_cfg<FMT, MT, XT, false>(a, map, wmap, ring, status, ksplit, partials, stages, smem_bytes, stream);
    if (e != cudaSuccess || ksplit == 1) return e;
    const int64_t total = a.m * a.n;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_tc_reduce_kernel, (const float *)partials, ksplit, a.bias, a.y, a.m, a.n, a.y_dt);
}

template <int FMT>
static cudaError_t launch_fmt(const TcArgs &a, int *status, int mt, int ksplit, float *partials, cudaStream_t stream) {
    const bool f32 = a.x_dt == NNQ_F32;
    if (mt == 1) return f32 ? launch_one<FMT, 1, float>(a, status, ksplit, partials, stream) : launch_one<FMT, 1, __nv_bfloat16>(a, status, ksplit, partials, stream);
    if (mt == 2) return f32 ? launch_one<FMT, 2, float>(a, status, ksplit, partials, stream) : launch_one<FMT, 2, __nv_bfloat16>(a, status, ksplit, partials, stream);
    return f32 ? launch_one<FMT, 4, float>(a, status, ksplit, partials, stream) : launch_one<FMT, 4, __nv_bfloat16>(a, status, ksplit, partials, stream);
}

template <int FMT, int MT>
static cudaError_t launch_grouped_mt(const TcGroupArgs &g, int *status, cudaStream_t stream) {
    TcArgs a = {g.w, g.scales, g.x_bf16, g.bias, g.y, g.rows_upper, g.n, g.k, g.fmt, NNQ_BF16, NNQ_F32};
    CUtensorMap map, wmap;
    memset(&map, 0, sizeof(map));
    memset(&wmap, 0, sizeof(wmap));
    if (!make_x_map(a, &map)) return cudaErrorNotSupported;
    // the experts' raw tensors are one contiguous [experts, N, K] tensor (checked by the caller)
    using RG = TcRawGeom<FMT, MT>;
    const bool ring = RG::kRing && tc_raw_ring(FMT, g.k);
    if (ring && !make_w_map(g.w, (int64_t)g.experts * g.n, g.k, RG::kUnitBytes, RG::kSB, &wmap)) return cudaErrorNotSupported;
    int stages = tc_max_stages<FMT, MT>();
    const int nkb = (int)(g.k / kTcBK);
    if (stages > nkb) stages = nkb;
    const TcGroup grp = {g.offsets, g.experts, g.w_stride, g.s_stride};
    // every expert may end with a partly filled row tile
    const int grid_y = (int)(g.rows_upper / (128 * MT)) + g.experts;
    return launch_cfg<FMT, MT, __nv_bfloat16, true>(a, map, wmap, ring, status, 1, nullptr, stages, tc_smem_bytes<FMT, MT>(stages), stream, grp, grid_y);
}

template <int FMT>
static cudaError_t launch_grouped_fmt(const TcGroupArgs &g, int *status, cudaStream_t stream) {
    const int64_t avg = g.rows_upper / (g.experts > 0 ? g.experts : 1);
    if (avg >= 384) return launch_grouped_mt<FMT, 4>(g, status, stream);
    if (avg >= 160) return launch_grouped_mt<FMT, 2>(g, status, stream);
    return launch_grouped_mt<FMT, 1>(g, status, stream);
}

nnq_status launch_gemm_tc_grouped(nnq_ctx *ctx, const TcGroupArgs &g, cudaStream_t stream) {
    if (g.k < kTcBK || g.k % kTcBK || g.experts < 1 || g.rows_upper < 1 || (tc_raw_ring(g.fmt, g.k) && (((uintptr_t)g.w & 15u) || g.w_stride != (size_t)g.n * (size_t)(g.k / 256) * (size_t)tc_raw_unit_bytes(g.fmt))))
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "grouped tensor product: unsupported shape");
    cudaError_t e;
    switch (g.fmt) {
        case NNQ_Q4_0: e = launch_grouped_fmt<NNQ_Q4_0>(g, ctx->d_status, stream); break;
        case NNQ_Q4_1: e = launch_grouped_fmt<NNQ_Q4_1>(g, ctx->d_status, stream); break;
        case NNQ_Q8_0: e = launch_grouped_fmt<NNQ_Q8_0>(g, ctx->d_status, stream); break;
        case NNQ_Q4_K: e = launch_grouped_fmt<NNQ_Q4_K>(g, ctx->d_status, stream); break;
        case NNQ_Q4_K_GGML: e = launch_grouped_fmt<NNQ_Q4_K_GGML>(g, ctx->d_status, stream); break;
        case NNQ_Q6_K: e = launch_grouped_fmt<NNQ_Q6_K>(g, ctx->d_status, stream); break;
        case NNQ_MXFP4_CORE: e = launch_grouped_fmt<NNQ_MXFP4_CORE>(g, ctx->d_status, stream); break;
        case NNQ_MXFP4_SPLIT: e = launch_grouped_fmt<NNQ_MXFP4_SPLIT>(g, ctx->d_status, stream); break;
        case NNQ_MXFP4_GPTOSS: e = launch_grouped_fmt<NNQ_MXFP4_GPTOSS>(g, ctx->d_status, stream); break;
        case NNQ_F32_DENSE: e = launch_grouped_fmt<NNQ_F32_DENSE>(g, ctx->d_status, stream); break;
        case NNQ_BF16_DENSE: e = launch_grouped_fmt<NNQ_BF16_DENSE>(g, ctx->d_status, stream); break;
        default: return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", g.fmt);
    }
    ctx->launches++;
    return check_cuda(ctx, e, "grouped tensor-core GEMM launch");
}

nnq_status launch_gemm_tc(nnq_ctx *ctx, const TcArgs &a, cudaStream_t stream) {
    cudaError_t e;
    // Rows per CTA: as many 128-row accumulators (1, 2 or 4) as the activation rows fill, because every
    // CTA decodes its weight tile for itself and the decode, not the MMA, is the expensive part. Where that
    // leaves fewer tiles than half the SMs, K is split over CTAs instead of shrinking the tile (a smaller
    // tile decodes every weight tile several times); the f32 partial sums go through a scratch buffer owned
    // by the context and are added in slice order by a second kernel.
    const int64_t ntiles = (a.n + 127) / 128;
    int mt = a.m > 256 ? 4 : (a.m > 128 ? 2 : 1);
    if (mt == 4 && a.fmt == NNQ_Q8_0 && tc_raw_ring(a.fmt, a.k)) mt = 2;   // the 512-row tile leaves no room for the Q8_0 ring
    static const char *env_mt = diag_env("NNQ_TC_MT");   // tuning aid
    if (env_mt && (atoi(env_mt) == 1 || atoi(env_mt) == 2 || atoi(env_mt) == 4)) mt = atoi(env_mt);
    int ksplit = 1;
    {
        const int64_t ctas = ntiles * ((a.m + 128 * mt - 1) / (128 * mt));
        const int64_t nkb = a.k / kTcBK;
        const int64_t target = ctx->sm_count;   // one CTA per SM
        if (ctas * 2 <= target) {
            ksplit = (int)(target / ctas);
            if (ksplit > 8) ksplit = 8;
            if (ksplit > nkb / 4) ksplit = (int)(nkb / 4);
            // formats on the raw ring slice K in whole boxes
            const int64_t box_kb = (a.fmt == NNQ_Q8_0 || mt == 4) ? 4 : 8;
            if (tc_raw_ring(a.fmt, a.k) && ksplit > (nkb + box_kb - 1) / box_kb) ksplit = (int)((nkb + box_kb - 1) / box_kb);
            if (ksplit < 1) ksplit = 1;
        }
        // the scratch is sized once, at context creation, for the largest split this rule can ask
        // for (ksplit * ctas <= SMs tiles of 512 x 128 f32): nothing is allocated here
        while (ksplit > 1 && (size_t)ksplit * a.m * a.n * sizeof(float) > ctx->partials_bytes) ksplit--;
    }
    switch (a.fmt) {
        case NNQ_Q4_0: e = launch_fmt<NNQ_Q4_0>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q4_1: e = launch_fmt<NNQ_Q4_1>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q8_0: e = launch_fmt<NNQ_Q8_0>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q4_K: e = launch_fmt<NNQ_Q4_K>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q4_K_GGML: e = launch_fmt<NNQ_Q4_K_GGML>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q6_K: e = launch_fmt<NNQ_Q6_K>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_MXFP4_CORE: e = launch_fmt<NNQ_MXFP4_CORE>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_MXFP4_SPLIT: e = launch_fmt<NNQ_MXFP4_SPLIT>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_MXFP4_GPTOSS: e = launch_fmt<NNQ_MXFP4_GPTOSS>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q5_0: e = launch_fmt<NNQ_Q5_0>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q5_1: e = launch_fmt<NNQ_Q5_1>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q2_K: e = launch_fmt<NNQ_Q2_K>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q3_K: e = launch_fmt<NNQ_Q3_K>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q5_K: e = launch_fmt<NNQ_Q5_K>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_F32_DENSE: e = launch_fmt<NNQ_F32_DENSE>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        case NNQ_BF16_DENSE: e = launch_fmt<NNQ_BF16_DENSE>(a, ctx->d_status, mt, ksplit, ctx->d_partials, stream); break;
        default: return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", a.fmt);
    }
    ctx->launches += ksplit > 1 ? 2 : 1;
    return check_cuda(ctx, e, "tensor-core GEMM launch");
}

}  // namespace nnq
