// Prefill product (M > 16) on the 5th-generation tensor cores: y[M, N] = x[M, K] * W[N, K]^T (+ bias)
// with block-quantized W of any format.
//
// One CTA computes a (128 * MT) x 128 output tile (MT = 1, 2 or 4 accumulators of 128 x 128 f32
// in tensor memory). Per 64-wide k step
//   * the (128 * MT) x 64 bf16 activation tile arrives by TMA (cp.async.bulk.tensor.2d through a
//     tensor map of x with 128-byte swizzle, issued by one thread, counted on the stage's "full"
//     barrier; rows beyond M are zero-filled); f32 activations are converted by the producers;
//   * 8 producer warps dequantize the 128 x 64 weight tile to bf16 (f32 decode, the bit-exact
//     one, then round-to-nearest-even) into the same K-major 128-byte-swizzled layout;
//   * one thread issues 4 * MT tcgen05.mma (M 128, N 128, K 16, bf16 x bf16 -> f32) from shared
//     memory descriptors into the accumulators and commits them onto the stage's "empty" barrier.
// The larger MT, the more activation rows reuse each dequantized weight tile (the dequantization,
// not the MMA, is the expensive part at small M). After the last k step the producer warps read
// the accumulators back with tcgen05.ld, add the bias and store f32 / bf16.
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

constexpr int kTcProducerWarps = 8;
constexpr int kTcThreads = (kTcProducerWarps + 1) * 32;
constexpr int kTcBK = 64;                    // k per stage: one 128-byte swizzle row of bf16
constexpr int kTcTileBytes = 128 * 128;      // 128 rows x 128 bytes

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
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const uint8_t *__restrict__ w, const uint8_t *__restrict__ wscales,
               const XT *__restrict__ x, const float *__restrict__ bias, void *__restrict__ y, int64_t M, int64_t N,
               int64_t K, int y_dt, int stages, float *__restrict__ partials, int *status, const TcGroup grp) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment of the tiles (the dynamic window is not guaranteed to start on one)
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int kStageBytes = (MT + 1) * kTcTileBytes;   // MT activation tiles, then the weight tile
    __shared__ __align__(8) uint64_t bars[2 * 8 + 1];      // full[stages], empty[stages], accumulators ready
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t n0 = (int64_t)blockIdx.x * 128;
    int64_t m0 = (int64_t)blockIdx.y * 128 * MT;
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
        if (wscales) wscales += (size_t)gsel[0] * grp.s_stride;
        if (bias) bias += (size_t)gsel[0] * N;
    }
    // this CTA's share of the k steps (gridDim.z slices of K; partial sums go to `partials`)
    const int nkb_all = (int)(K / kTcBK);
    const int kb_lo = (int)(((long long)blockIdx.z * nkb_all) / gridDim.z);
    const int nkb = (int)(((long long)(blockIdx.z + 1) * nkb_all) / gridDim.z) - kb_lo;
    const uint32_t full_s = smem_u32(bars), empty_s = full_s + 8 * 8, acc_s = full_s + 16 * 8;
    constexpr uint32_t kTmemCols = 128 * MT;

    if (tid == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(full_s + 8 * s, kTcProducerWarps);
            mbar_init(empty_s + 8 * s, 1);
        }
        mbar_init(acc_s, 1);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTcProducerWarps) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    bool ok = true;

    if (warp < kTcProducerWarps) {
        // ---------------- producers ----------------
        const int64_t cpr = K / 32;                 // 32-weight chunks per weight row
        const int brow = tid & 127, bhalf = tid >> 7;   // weight tile: row and which 32 of the 64 k
        int slot = 0;
        uint32_t phase = 0;
        // Software pipeline: the tile data of step kb + 1 is decoded into registers right after step kb
        // has been handed to the tensor core, so that the work runs under the MMAs and under the wait
        // for a free stage. For Q4_K the raw bytes are loaded one step earlier still (two steps
        // ahead of their use), so that the decode never waits for global memory.
        constexpr int kAChunks = (128 * MT * 8) / (kTcProducerWarps * 32);   // 16-byte activation chunks per thread
        uint4 wreg[4];
        uint4 areg[kAChunks];
        const int ac = tid & 7;
        constexpr bool kSplitLoad = FMT == NNQ_Q4_K;
        uint4 raw_h = make_uint4(0, 0, 0, 0), raw_q = make_uint4(0, 0, 0, 0);
        auto load_raw = [&](int kb) {
            if (kSplitLoad && n0 + brow < N) {
                const int64_t c = (n0 + brow) * cpr + (int64_t)kb * 2 + bhalf;
                const uint8_t *b = w + (c >> 3) * 144;
                raw_h = __ldg(reinterpret_cast<const uint4 *>(b));
                raw_q = __ldg(reinterpret_cast<const uint4 *>(b + 16 + 16 * (int)(c & 7)));
            }
        };
        auto fetch = [&](int kb) {
            float wv[32];
            if (n0 + brow < N) {
                if (kSplitLoad) Decode<NNQ_Q4_K>::chunk_regs(raw_h, raw_q, (kb * 2 + bhalf) & 7, wv);
                else Decode<FMT>::chunk(w, wscales, (n0 + brow) * cpr + (int64_t)kb * 2 + bhalf, wv);
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) wv[i] = 0.0f;
            }
#pragma unroll
            for (int c = 0; c < 4; c++)
                wreg[c] = make_uint4(pack_bf16(wv[8 * c], wv[8 * c + 1]), pack_bf16(wv[8 * c + 2], wv[8 * c + 3]),
                                     pack_bf16(wv[8 * c + 4], wv[8 * c + 5]), pack_bf16(wv[8 * c + 6], wv[8 * c + 7]));
#pragma unroll
            for (int i = 0; i < (TMAX ? 0 : kAChunks); i++) {
                const int r = (tid >> 3) + 32 * i;
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
                areg[i] = v;
            }
        };
        load_raw(kb_lo);
        fetch(kb_lo);
        if (nkb > 1) load_raw(kb_lo + 1);
        for (int kb = 0; kb < nkb && ok; kb++) {
            if (kb >= stages) ok = mbar_wait_fast(empty_s + 8 * slot, phase ^ 1u);
            if (!ok) break;
            uint8_t *stage = smem + (size_t)slot * kStageBytes;
            uint8_t *bt = stage + MT * kTcTileBytes;
            if (TMAX && tid == 0) {
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
            for (int i = 0; i < (TMAX ? 0 : kAChunks); i++) {
                const int r = (tid >> 3) + 32 * i;
                *reinterpret_cast<uint4 *>(stage + (r >> 7) * kTcTileBytes + swz(r & 127, ac)) = areg[i];
            }
            fence_async_smem();      // generic-proxy writes -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(full_s + 8 * slot);
            if (++slot == stages) {
                slot = 0;
                phase ^= 1u;
            }
            if (kb + 1 < nkb) {
                fetch(kb_lo + kb + 1);
                if (kb + 2 < nkb) load_raw(kb_lo + kb + 2);
            }
        }
        // ---------------- epilogue ----------------
        if (ok) ok = mbar_wait_fast(acc_s, 0);
        if (ok) {
            tc_fence_after();
            const int q = warp & 3, chalf = warp >> 2;   // TMEM lane quarter, column half
#pragma unroll 1
            for (int mt = 0; mt < MT; mt++) {
                const int64_t row = m0 + mt * 128 + q * 32 + lane;
#pragma unroll 1
                for (int cc = 0; cc < 2; cc++) {
                    const int col0 = chalf * 64 + cc * 32;
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * 128 + col0), v);
                    if (row < M) {
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            const int64_t col = n0 + col0 + i;
                            if (col < N) {
                                float f = __uint_as_float(v[i]);
                                if (partials) {   // K is split over CTAs: bias and conversion happen in the reduction
                                    partials[((size_t)blockIdx.z * M + row) * N + col] = f;
                                    continue;
                                }
                                if (bias) f += __ldg(bias + col);
                                if (y_dt == NNQ_F32) reinterpret_cast<float *>(y)[row * N + col] = f;
                                else reinterpret_cast<__nv_bfloat16 *>(y)[row * N + col] = __float2bfloat16_rn(f);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
        }
    } else if (lane == 0) {
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
    }
    if (!ok) {
        abort_s = 1;
        if (lane == 0) atomicExch(status, 1);
    }
    __syncthreads();
    if (warp == kTcProducerWarps) {
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
    return w && w->d_raw && m >= 1 && w->k >= kTcBK && w->k % kTcBK == 0 && w->n >= 1;
}

// Tensor map of the bf16 activations [M, K]: boxes of 64 x 128 elements, 128-byte swizzle, zero fill
// beyond M. Returns false when the driver entry point is not available (the producers then stage
// the activations themselves).
static bool make_x_map(const TcArgs &a, CUtensorMap *map) {
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
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
    if (!fn || ((uintptr_t)a.x & 15u) || (a.k * 2) % 16) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
    const cuuint64_t strides[1] = {(cuuint64_t)a.k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTcBK, 128u};
    const cuuint32_t estr[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(a.x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int FMT, int MT, typename XT, bool TMAX>
static cudaError_t launch_cfg(const TcArgs &a, const CUtensorMap &map, int *status, int ksplit, float *partials, int stages,
                              int smem_bytes, cudaStream_t stream, const TcGroup &grp = TcGroup{nullptr, 0, 0, 0}, int grid_y = 0) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<FMT, MT, XT, TMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    dim3 grid((unsigned)((a.n + 127) / 128), (unsigned)(grid_y ? grid_y : (a.m + 128 * MT - 1) / (128 * MT)), (unsigned)ksplit);
    gemm_tc_kernel<FMT, MT, XT, TMAX><<<grid, kTcThreads, smem_bytes, stream>>>(
        map, a.w, a.scales, reinterpret_cast<const XT *>(a.x), a.bias, a.y, a.m, a.n, a.k, a.y_dt, stages,
        ksplit > 1 ? partials : nullptr, status, grp);
    return cudaGetLastError();
}

template <int FMT, int MT, typename XT>
static cudaError_t launch_one(const TcArgs &a, int *status, int ksplit, float *partials, cudaStream_t stream) {
    const int stage_bytes = (MT + 1) * kTcTileBytes;
    // MT = 1, 2: 96 KB of stages, so that two CTAs (2 x 128 * MT tensor-memory columns) share an SM and
    // one CTA's decode overlaps the other's MMAs; MT = 4 fills the SM alone
    int stages = MT == 4 ? 2 : (MT == 2 ? 2 : 3);
    const int nkb = (int)(a.k / kTcBK);
    if (stages > nkb / ksplit) stages = nkb / ksplit > 0 ? nkb / ksplit : 1;
    const int smem_bytes = stages * stage_bytes + 1024;
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    cudaError_t e;
    if (sizeof(XT) == 2 && make_x_map(a, &map))
        e = launch_cfg<FMT, MT, XT, sizeof(XT) == 2>(a, map, status, ksplit, partials, stages, smem_bytes, stream);
    else
        e = launch_cfg<FMT, MT, XT, false>(a, map, status, ksplit, partials, stages, smem_bytes, stream);
    if (e != cudaSuccess || ksplit == 1) return e;
    const int64_t total = a.m * a.n;
    gemm_tc_reduce_kernel<<<(int)((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048), 256, 0, stream>>>(
        partials, ksplit, a.bias, a.y, a.m, a.n, a.y_dt);
    return cudaGetLastError();
}

template <int FMT>
static cudaError_t launch_fmt(const TcArgs &a, int *status, int sm_count, int ksplit, float *partials, cudaStream_t stream) {
    const bool f32 = a.x_dt == NNQ_F32;
    // Rows per CTA: the more rows share a decoded weight tile the less decode work, but the grid
    // must still cover the machine. Take the largest tile that leaves at least one CTA per two SMs.
    // (Decoding the whole weight to bf16 first and multiplying afterwards was measured slower than
    // decoding per tile even at M = 4096: the tile pipeline, not the decode, is the limit.)
    const int64_t ntiles = (a.n + 127) / 128;
    auto ctas = [&](int mt) { return ntiles * ((a.m + 128 * mt - 1) / (128 * mt)); };
    int mt = 1;
    // (measured with the activation tiles arriving by TMA: half a wave of the largest tile still beats
    // a full wave of smaller ones, because every CTA decodes its weight tile for itself)
    if (a.m > 256 && 2 * ctas(4) >= sm_count) mt = 4;
    else if (a.m > 128 && 2 * ctas(2) >= sm_count) mt = 2;
    static const char *env_mt = diag_env("NNQ_TC_MT");   // tuning aid
    if (env_mt && (atoi(env_mt) == 1 || atoi(env_mt) == 2 || atoi(env_mt) == 4)) mt = atoi(env_mt);
    if (mt != 1) ksplit = 1;
    if (mt == 1) return f32 ? launch_one<FMT, 1, float>(a, status, ksplit, partials, stream) : launch_one<FMT, 1, __nv_bfloat16>(a, status, ksplit, partials, stream);
    if (mt == 2) return f32 ? launch_one<FMT, 2, float>(a, status, 1, nullptr, stream) : launch_one<FMT, 2, __nv_bfloat16>(a, status, 1, nullptr, stream);
    return f32 ? launch_one<FMT, 4, float>(a, status, 1, nullptr, stream) : launch_one<FMT, 4, __nv_bfloat16>(a, status, 1, nullptr, stream);
}

template <int FMT, int MT>
static cudaError_t launch_grouped_mt(const TcGroupArgs &g, int *status, cudaStream_t stream) {
    TcArgs a = {g.w, g.scales, g.x_bf16, g.bias, g.y, g.rows_upper, g.n, g.k, g.fmt, NNQ_BF16, NNQ_F32};
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    if (!make_x_map(a, &map)) return cudaErrorNotSupported;
    const int stage_bytes = (MT + 1) * kTcTileBytes;
    int stages = MT == 4 ? 2 : (MT == 2 ? 2 : 3);
    const int nkb = (int)(g.k / kTcBK);
    if (stages > nkb) stages = nkb;
    const TcGroup grp = {g.offsets, g.experts, g.w_stride, g.s_stride};
    // every expert may end with a partly filled row tile
    const int grid_y = (int)(g.rows_upper / (128 * MT)) + g.experts;
    return launch_cfg<FMT, MT, __nv_bfloat16, true>(a, map, status, 1, nullptr, stages, stages * stage_bytes + 1024, stream, grp, grid_y);
}

template <int FMT>
static cudaError_t launch_grouped_fmt(const TcGroupArgs &g, int *status, cudaStream_t stream) {
    const int64_t avg = g.rows_upper / (g.experts > 0 ? g.experts : 1);
    if (avg >= 384) return launch_grouped_mt<FMT, 4>(g, status, stream);
    if (avg >= 160) return launch_grouped_mt<FMT, 2>(g, status, stream);
    return launch_grouped_mt<FMT, 1>(g, status, stream);
}

nnq_status launch_gemm_tc_grouped(nnq_ctx *ctx, const TcGroupArgs &g, cudaStream_t stream) {
    if (g.k < kTcBK || g.k % kTcBK || g.experts < 1 || g.rows_upper < 1) return fail(ctx, NNQ_ERR_UNSUPPORTED, "grouped tensor product: unsupported shape");
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
    // Small grids (few rows, few output tiles) split K over CTAs so that every SM works; the f32
    // partial sums go through a scratch buffer owned by the context and are added in slice order.
    int ksplit = 1;
    {
        const int64_t ctas = ((a.n + 127) / 128) * ((a.m + 127) / 128);
        const int64_t nkb = a.k / kTcBK;
        // aim at two CTAs per SM for very few rows (the partial sums are small), one otherwise
        const int64_t target = a.m <= 64 ? 2 * ctx->sm_count : ctx->sm_count;
        if (a.m <= 256 && ctas * 2 <= target) {
            ksplit = (int)(target / ctas);
            if (ksplit > 8) ksplit = 8;
            if (ksplit > nkb / 4) ksplit = (int)(nkb / 4);
            if (ksplit < 1) ksplit = 1;
        }
        // the scratch is sized once, at context creation, for the largest split this rule can ask
        // for (ksplit * ctas <= 2 * SMs tiles of 128 x 128 f32): nothing is allocated here
        while (ksplit > 1 && (size_t)ksplit * a.m * a.n * sizeof(float) > ctx->partials_bytes) ksplit--;
    }
    switch (a.fmt) {
        case NNQ_Q4_0: e = launch_fmt<NNQ_Q4_0>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q4_1: e = launch_fmt<NNQ_Q4_1>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q8_0: e = launch_fmt<NNQ_Q8_0>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q4_K: e = launch_fmt<NNQ_Q4_K>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q4_K_GGML: e = launch_fmt<NNQ_Q4_K_GGML>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q6_K: e = launch_fmt<NNQ_Q6_K>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_MXFP4_CORE: e = launch_fmt<NNQ_MXFP4_CORE>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_MXFP4_SPLIT: e = launch_fmt<NNQ_MXFP4_SPLIT>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_MXFP4_GPTOSS: e = launch_fmt<NNQ_MXFP4_GPTOSS>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q5_0: e = launch_fmt<NNQ_Q5_0>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q5_1: e = launch_fmt<NNQ_Q5_1>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q2_K: e = launch_fmt<NNQ_Q2_K>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q3_K: e = launch_fmt<NNQ_Q3_K>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_Q5_K: e = launch_fmt<NNQ_Q5_K>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_F32_DENSE: e = launch_fmt<NNQ_F32_DENSE>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        case NNQ_BF16_DENSE: e = launch_fmt<NNQ_BF16_DENSE>(a, ctx->d_status, ctx->sm_count, ksplit, ctx->d_partials, stream); break;
        default: return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", a.fmt);
    }
    ctx->launches += ksplit > 1 ? 2 : 1;
    return check_cuda(ctx, e, "tensor-core GEMM launch");
}

}  // namespace nnq
