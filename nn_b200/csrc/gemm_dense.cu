// Large-prefill product (M >= 256 tokens): decode the weight once to bf16, then a plain bf16 GEMM
// on the 5th-generation tensor cores.
//
// With hundreds of activation rows per weight row the decode is a small part of the work: one pass
// over the raw blocks writes bf16 [N, K] into a scratch buffer owned by the context (0.56 + 2 bytes
// per weight at HBM speed; weights up to ~60 MB stay in L2 for the GEMM), and the GEMM main loop
// then does nothing but move tiles and issue MMAs:
//   * persistent CTAs (one per SM), output tiles of 128 x 256, k steps of 64 (one 128-byte swizzle
//     row of bf16), a 4-stage ring of (16 KB activation tile + 32 KB weight tile);
//   * warp 0: one thread issues the TMA loads of both tiles (cp.async.bulk.tensor.2d, 128-byte
//     swizzle, zero fill beyond M / N) onto the stage's "full" barrier;
//   * warp 1: one thread issues tcgen05.mma (M 128, N 256, K 16, bf16 x bf16 -> f32) into one of
//     two 256-column accumulators in tensor memory and commits the stage's "empty" barrier;
//   * warps 2..5: epilogue -- tcgen05.ld of the finished accumulator (each warp its quarter of
//     the 128 lanes), bias, conversion, stores -- while the MMA warp already fills the other
//     accumulator with the next tile.
// Tiles are numbered m-fastest, so the CTAs running at one time share a few weight tiles and the
// activation matrix stays in L2. Weights and activations are bf16: the 1e-2 tolerance class.
// Every barrier wait is bounded; a wait that runs out sets the context's status word, every role
// leaves its loop and the tensor memory is freed.
#include <cuda.h>
#include <cuda_bf16.h>
#include <string.h>

#include "decode.cuh"
#include "gemm_tc.h"
#include "sync.cuh"

namespace nnq {

// ---------------------------------------------------------------------------------
// raw blocks -> bf16 [N, K]
// ---------------------------------------------------------------------------------

constexpr int kDbThreads = 128;

// MXFP4 straight to bf16 bits, no f32 detour: a magnitude code m >= 2 is (1 + (m & 1) / 2) * 2^((m >> 1) - 1),
// m == 1 is 0.5, and the block scale is 2^(e - 127), so the product is the bf16 number with exponent field
// e - 1 + (m >> 1) and top mantissa bit (m & 1): bits = ((e - 1) << 7) + (m' << 6) with m' = m (0 for m == 1),
// zero for m == 0, sign on bit 15. Exact, hence equal to rounding the f32 decode; valid for 1 <= e <= 251
// (other exponents take the f32 path).
__device__ __forceinline__ uint32_t mx_bf16_one(uint32_t nib, uint32_t base) {
    const uint32_t m = nib & 7u;
    const uint32_t mp = m == 1u ? 0u : m;
    const uint32_t mag = m == 0u ? 0u : base + (mp << 6);
    return mag | ((nib & 8u) << 12);
}

template <bool HIGH_FIRST>
__device__ __forceinline__ void mx_chunk_bf16(const uint4 q, uint32_t e, uint4 *out4) {
    const uint32_t base = (e - 1u) << 7;
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int v = 0; v < 4; v++) {
        uint32_t p[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t byte = (qw[v] >> (8 * i)) & 0xFFu;
            const uint32_t even = HIGH_FIRST ? byte >> 4 : byte & 15u, odd = HIGH_FIRST ? byte & 15u : byte >> 4;
            p[i] = mx_bf16_one(even, base) | (mx_bf16_one(odd, base) << 16);
        }
        out4[v] = make_uint4(p[0], p[1], p[2], p[3]);
    }
}

template <int FMT>
__global__ void __launch_bounds__(kDbThreads)
dequant_bf16_kernel(const uint8_t *__restrict__ src, const uint8_t *__restrict__ scales, int64_t nchunks,
                    uint4 *__restrict__ dst, int cpr, int half_rows) {
    if (FMT == NNQ_MXFP4_SPLIT || FMT == NNQ_MXFP4_GPTOSS) {
        // a thread owns one 32-weight chunk: 64 contiguous output bytes (two whole 32-byte sectors), written
        // with four 16-byte stores -- the integer decode needs no staging (measured: 366 -> 320 us for the
        // 282 MB of a gpt-oss gate / up tensor; the f32 decoders below are faster with the staged store)
        auto emit = [&](int64_t c, uint32_t e, const uint4 q) {
            uint4 o4[4];
            if (e >= 1u && e <= 251u) {
                mx_chunk_bf16<FMT == NNQ_MXFP4_GPTOSS>(q, e, o4);
            } else {
                float o[32];
                Decode<FMT>::chunk(src, scales, c, o);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint32_t p[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        __nv_bfloat162 v = __floats2bfloat162_rn(o[8 * j + 2 * i], o[8 * j + 2 * i + 1]);
                        p[i] = *reinterpret_cast<uint32_t *>(&v);
                    }
                    o4[j] = make_uint4(p[0], p[1], p[2], p[3]);
                }
            }
            // half_rows > 0: every group of 2 * half_rows weight rows (one expert's gate rows, then its up
            // rows) is written interleaved, gate row j to row 2j and up row j to row 2j + 1, so that a GEMM
            // tile holds both halves of an output column pair (the fused SwiGLU epilogue)
            int64_t oc = c;
            if (half_rows > 0) {   // nchunks < 2^31 here (checked by the launcher): 32-bit divisions
                const uint32_t c32 = (uint32_t)c, row = c32 / (uint32_t)cpr, cin = c32 - row * (uint32_t)cpr;
                const uint32_t ex = row / (2u * half_rows), r = row - ex * 2u * half_rows;
                const uint32_t r2 = r < (uint32_t)half_rows ? 2u * r : 2u * (r - half_rows) + 1u;
                oc = (int64_t)(ex * 2u * half_rows + r2) * cpr + cin;
            }
#pragma unroll
            for (int j = 0; j < 4; j++) dst[oc * 4 + j] = o4[j];
        };
        // two chunks per iteration: both loads are in flight before either is decoded
        const int64_t stride = (int64_t)gridDim.x * kDbThreads;
        int64_t c = (int64_t)blockIdx.x * kDbThreads + threadIdx.x;
        for (; c + stride < nchunks; c += 2 * stride) {
            const uint32_t e0 = __ldg(scales + c), e1 = __ldg(scales + c + stride);
            const uint4 q0 = __ldg(reinterpret_cast<const uint4 *>(src + c * 16));
            const uint4 q1 = __ldg(reinterpret_cast<const uint4 *>(src + (c + stride) * 16));
            emit(c, e0, q0);
            emit(c + stride, e1, q1);
        }
        if (c < nchunks) emit(c, __ldg(scales + c), __ldg(reinterpret_cast<const uint4 *>(src + c * 16)));
        return;
    }
    __shared__ uint4 tile[kDbThreads * 4 + 4];
    for (int64_t base = (int64_t)blockIdx.x * kDbThreads; base < nchunks; base += (int64_t)gridDim.x * kDbThreads) {
        const int64_t c = base + threadIdx.x;
        if (c < nchunks) {
            float o[32];
            Decode<FMT>::chunk(src, scales, c, o);   // the bit-exact decode, then round to nearest even
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t p[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(o[8 * j + 2 * i], o[8 * j + 2 * i + 1]);
                    p[i] = *reinterpret_cast<uint32_t *>(&v);
                }
                // chunk-local XOR swizzle: for a fixed j the 16-byte stores of a quarter warp fall into
                // eight different bank groups (unswizzled, threads 64 bytes apart share two of them)
                tile[threadIdx.x * 4 + (j ^ ((threadIdx.x >> 1) & 3))] = make_uint4(p[0], p[1], p[2], p[3]);
            }
        }
        __syncthreads();
        const int64_t remaining = nchunks - base;
        const int live = remaining < kDbThreads ? (int)remaining : kDbThreads;
        uint4 *out = dst + base * 4;
        for (int idx = threadIdx.x; idx < live * 4; idx += kDbThreads) out[idx] = tile[(idx & ~3) | ((idx & 3) ^ ((idx >> 3) & 3))];
        __syncthreads();
    }
}

// nn-gptoss expert tensors [E, K, N] (MXFP4, 32-weight blocks along N, the even column in the high
// nibble) -> bf16 [E, N, K]: a CTA turns a 64 x 64 tile through shared memory. Reads are 16 bytes per
// thread (one block), writes 128 contiguous bytes per output row. half_rows > 0 interleaves the output
// rows of every expert (row j -> 2j, row half_rows + j -> 2j + 1), as the fused SwiGLU epilogue wants.
constexpr int kKnTile = 64;
__global__ void __launch_bounds__(128)
dequant_kn_bf16_kernel(const uint8_t *__restrict__ data, const uint8_t *__restrict__ scales, __nv_bfloat16 *__restrict__ dst,
                       int K, int N, int half_rows) {
    __shared__ __align__(16) uint16_t tile[kKnTile][kKnTile + 8];   // [n][k]; 144-byte rows keep 16-byte reads aligned
    const int e = blockIdx.z, k0 = blockIdx.y * kKnTile, n0 = blockIdx.x * kKnTile;
    const int kk = threadIdx.x & 63, blk = threadIdx.x >> 6;          // this thread's k row and which 32 of the 64 columns
    const size_t row = (size_t)e * K + k0 + kk;
    const uint4 q = __ldg(reinterpret_cast<const uint4 *>(data + row * (size_t)(N / 2) + n0 / 2 + blk * 16));
    const uint32_t ex = __ldg(scales + row * (size_t)(N / 32) + n0 / 32 + blk);
    const bool direct = ex >= 1u && ex <= 251u;
    const uint32_t base = (ex - 1u) << 7;
    const float scale = mx_scale_gptoss(ex);
    auto one = [&](uint32_t nib) -> uint16_t {
        if (direct) return (uint16_t)mx_bf16_one(nib, base);
        return __bfloat16_as_ushort(__float2bfloat16_rn(e2m1_value(nib, scale)));
    };
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int v = 0; v < 4; v++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t byte = (qw[v] >> (8 * i)) & 0xFFu;
            const int col = blk * 32 + v * 8 + i * 2;
            tile[col][kk] = one(byte >> 4);
            tile[col + 1][kk] = one(byte & 15u);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kKnTile * 8; i += 128) {
        const int r = i >> 3, c = i & 7, n = n0 + r;
        const int nn = half_rows > 0 ? (n < half_rows ? 2 * n : 2 * (n - half_rows) + 1) : n;
        *reinterpret_cast<uint4 *>(dst + ((size_t)e * N + nn) * K + k0 + c * 8) = *reinterpret_cast<const uint4 *>(&tile[r][c * 8]);
    }
}

template <int FMT>
static cudaError_t launch_dequant_bf16(const uint8_t *src, const uint8_t *scales, int64_t nchunks, void *dst, int sm_count,
                                       cudaStream_t stream, int cpr = 1, int half_rows = 0) {
    const int64_t want = (nchunks + kDbThreads - 1) / kDbThreads;
    const int64_t cap = (int64_t)sm_count * 16;
    int grid = (int)(want < cap ? want : cap);
    if (grid < 1) grid = 1;
    dequant_bf16_kernel<FMT><<<grid, kDbThreads, 0, stream>>>(src, scales, nchunks, reinterpret_cast<uint4 *>(dst), cpr, half_rows);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// bf16 GEMM: y[M, N] = x[M, K] * Wd[N, K]^T (+ bias)
// ---------------------------------------------------------------------------------

// Tile 128 x BN x 64 with BN = 256, or 128 where 256-wide tiles would leave SMs without a tile.
constexpr int kDgBM = 128, kDgBK = 64, kDgStages = 4;
constexpr int kDgABytes = kDgBM * 128;
constexpr int kDgThreads = 192;
__host__ __device__ constexpr int dg_stage_bytes(int bn) { return kDgABytes + bn * 128; }

__device__ __forceinline__ void dg_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void dg_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t dg_smem_desc(uint32_t addr) {
    const uint32_t lo = ((addr >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void dg_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void dg_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void dg_tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}

__device__ __forceinline__ void dg_tmem_ld32(uint32_t addr, uint32_t (&v)[32]) {
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

// Grouped mode (expert products): the rows of x are sorted by expert (offsets[e] .. offsets[e+1]
// on the device), expert e multiplies its rows with rows [e * N, (e + 1) * N) of the decoded
// weights and adds bias + e * N. Row tiles are numbered expert by expert; rows of the next expert
// inside a tile are computed but not stored. offsets == NULL: a plain product.
constexpr int kDgMaxGroups = 64;

template <int BN>
__global__ void __launch_bounds__(kDgThreads, 1)
gemm_dense_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                  const float *__restrict__ bias, void *__restrict__ y, int M, int N, int K, int y_dt, int *status,
                  const int *__restrict__ offsets, int groups, __nv_bfloat16 *__restrict__ h_out, float swiglu_limit) {
    constexpr int kDgBN = BN, kDgStageBytes = dg_stage_bytes(BN);
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * kDgStages + 4];   // full[4], empty[4], acc_full[2], acc_empty[2]
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t full_s = smem_u32(bars), empty_s = full_s + 8 * kDgStages;
    const uint32_t accf_s = empty_s + 8 * kDgStages, acce_s = accf_s + 16;
    __shared__ int tile_begin[kDgMaxGroups + 1], row_begin[kDgMaxGroups + 1];
    if (tid == 0) {
        if (offsets) {
            int acc = 0;
            for (int e = 0; e < groups; e++) {
                tile_begin[e] = acc;
                row_begin[e] = offsets[e];
                acc += (offsets[e + 1] - offsets[e] + kDgBM - 1) / kDgBM;
            }
            tile_begin[groups] = acc;
            row_begin[groups] = offsets[groups];
        } else {
            tile_begin[0] = 0;
            tile_begin[1] = (M + kDgBM - 1) / kDgBM;
            row_begin[0] = 0;
            row_begin[1] = M;
        }
    }
    __syncthreads();
    const int ngroups = offsets ? groups : 1;
    const int m_tiles = tile_begin[ngroups], n_tiles = (N + kDgBN - 1) / kDgBN;
    const int tiles = m_tiles * n_tiles;
    const int nkb = K / kDgBK;
    // tile t -> (group, first row, end of the group's rows, first weight row)
    auto locate = [&](int t, int &e, int &m0, int &m_end, int &n0) {
        const int mt = t % m_tiles;
        e = 0;
        while (e + 1 < ngroups && mt >= tile_begin[e + 1]) e++;
        m0 = row_begin[e] + (mt - tile_begin[e]) * kDgBM;
        m_end = row_begin[e + 1];
        n0 = (t / m_tiles) * kDgBN;
    };

    if (tid == 0) {
        for (int s = 0; s < kDgStages; s++) {
            mbar_init(full_s + 8 * s, 1);
            mbar_init(empty_s + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(accf_s + 8 * a, 1);
            mbar_init(acce_s + 8 * a, 4);
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    dg_fence_before();
    __syncthreads();
    dg_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    bool ok = true;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            long long filled = 0;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                int e, m0, m_end, n0;
                locate(t, e, m0, m_end, n0);
                const int w0 = e * N + n0;   // weight rows of this group in the decoded [groups * N, K] matrix
                for (int kb = 0; kb < nkb; kb++) {
                    if (filled >= kDgStages && !mbar_wait_fast(empty_s + 8 * slot, phase ^ 1u)) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_s = smem_u32(smem + (size_t)slot * kDgStageBytes);
                    mbar_expect_tx(full_s + 8 * slot, kDgStageBytes);
                    dg_tma_2d(a_s, &xmap, kb * kDgBK, m0, full_s + 8 * slot);
                    dg_tma_2d(a_s + kDgABytes, &wmap, kb * kDgBK, w0, full_s + 8 * slot);
                    filled++;
                    if (++slot == kDgStages) {
                        slot = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // f32 accumulate, bf16 x bf16, both K-major, N = BN, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (((uint32_t)BN >> 3) << 17) | ((128u >> 4) << 24);
            int slot = 0;
            uint32_t phase = 0;
            int it = 0;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, it++) {
                const int a = it & 1;
                // the epilogue has read this accumulator's previous tile
                if (it >= 2 && !mbar_wait_fast(acce_s + 8 * a, (uint32_t)(((it >> 1) - 1) & 1))) {
                    ok = false;
                    break;
                }
                dg_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(a * kDgBN);
                for (int kb = 0; kb < nkb; kb++) {
                    if (!mbar_wait_fast(full_s + 8 * slot, phase)) {
                        ok = false;
                        break;
                    }
                    dg_fence_after();
                    const uint32_t a_s = smem_u32(smem + (size_t)slot * kDgStageBytes);
                    const uint64_t da = dg_smem_desc(a_s), db = dg_smem_desc(a_s + kDgABytes);
#pragma unroll
                    for (int k = 0; k < 4; k++) dg_mma(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    dg_commit(empty_s + 8 * slot);
                    if (++slot == kDgStages) {
                        slot = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) dg_commit(accf_s + 8 * a);
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;   // the quarter of the 128 TMEM lanes this warp may read
        int it = 0;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, it++) {
            const int a = it & 1;
            int e, m0, m_end, n0;
            locate(t, e, m0, m_end, n0);
            const float *gbias = bias ? bias + (size_t)e * N : nullptr;
            if (!mbar_wait_fast(accf_s + 8 * a, (uint32_t)((it >> 1) & 1))) {
                ok = false;
                break;
            }
            dg_fence_after();
            const int row = m0 + q * 32 + lane;
#pragma unroll 1
            for (int cc = 0; cc < kDgBN / 32; cc++) {
                uint32_t v[32];
                dg_tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * kDgBN + cc * 32), v);
                const int col0 = n0 + cc * 32;
                if (h_out) {
                    // interleaved gate / up columns (2j, 2j + 1): h[row, j] = clamp(silu(g), +-limit) * u in bf16,
                    // the input of the second expert product; the bias of column c is the gate bias of c / 2 for
                    // even c and the up bias (second half of the expert's bias row) for odd c
                    if (row < m_end && col0 < N) {
                        const int I = N >> 1;
                        uint32_t packed[8];
#pragma unroll
                        for (int p = 0; p < 16; p += 2) {
                            float hv[2];
#pragma unroll
                            for (int q2 = 0; q2 < 2; q2++) {
                                const int j = (col0 >> 1) + p + q2;
                                float gv = __uint_as_float(v[2 * (p + q2)]), uv = __uint_as_float(v[2 * (p + q2) + 1]);
                                if (gbias && j < I) {
                                    gv += __ldg(gbias + j);
                                    uv += __ldg(gbias + I + j);
                                }
                                // fast exponential and division (2^-22 relative): far below the bf16 rounding of h,
                                // and cheap enough for the epilogue to stay hidden behind the next tile's MMAs
                                float sv = __fdividef(gv, 1.0f + __expf(-gv));
                                sv = fminf(fmaxf(sv, -swiglu_limit), swiglu_limit);
                                hv[q2] = sv * uv;
                            }
                            __nv_bfloat162 b2 = __floats2bfloat162_rn(hv[0], hv[1]);
                            packed[p >> 1] = *reinterpret_cast<uint32_t *>(&b2);
                        }
                        __nv_bfloat16 *dstp = h_out + (size_t)row * I + (col0 >> 1);
                        if (col0 + 32 <= N && (I & 7) == 0) {
                            reinterpret_cast<uint4 *>(dstp)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                            reinterpret_cast<uint4 *>(dstp)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        } else {
                            const __nv_bfloat16 *pk = reinterpret_cast<const __nv_bfloat16 *>(packed);
                            for (int i = 0; i < 16; i++)
                                if ((col0 >> 1) + i < I) dstp[i] = pk[i];
                        }
                    }
                } else if (row < m_end && col0 < N) {
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; i++) f[i] = __uint_as_float(v[i]) + (gbias && col0 + i < N ? __ldg(gbias + col0 + i) : 0.0f);
                    if (col0 + 32 <= N && (N & 7) == 0) {
                        if (y_dt == NNQ_F32) {
                            float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(y) + (size_t)row * N + col0);
#pragma unroll
                            for (int i = 0; i < 8; i++) dst[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
                        } else {
                            uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(y) + (size_t)row * N + col0);
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                uint32_t p[4];
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    __nv_bfloat162 b2 = __floats2bfloat162_rn(f[8 * i + 2 * j], f[8 * i + 2 * j + 1]);
                                    p[j] = *reinterpret_cast<uint32_t *>(&b2);
                                }
                                dst[i] = make_uint4(p[0], p[1], p[2], p[3]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            if (col0 + i < N) {
                                if (y_dt == NNQ_F32) reinterpret_cast<float *>(y)[(size_t)row * N + col0 + i] = f[i];
                                else reinterpret_cast<__nv_bfloat16 *>(y)[(size_t)row * N + col0 + i] = __float2bfloat16_rn(f[i]);
                            }
                        }
                    }
                }
            }
            dg_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_s + 8 * a);
        }
    }
    if (!ok) {
        abort_s = 1;
        atomicExch(status, 1);
    }
    __syncthreads();
    if (warp == 1) {
        // with an aborted CTA, MMAs may still be in flight: give the last accumulator a bounded chance
        if (abort_s) {
            mbar_wait(accf_s, 0);
            mbar_wait(accf_s + 8, 0);
        }
        dg_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------

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

// bf16 [rows, k] row-major -> boxes of 64 x box_rows elements, 128-byte swizzle, zero fill outside
static bool make_map(const void *base, int64_t rows, int64_t k, int box_rows, CUtensorMap *map) {
    EncodeFn fn = encode_fn();
    if (!fn || ((uintptr_t)base & 15u) || (k * 2) % 16) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kDgBK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool gemm_dense_shape_ok(const nnq_ctx *ctx, int64_t m, int64_t n, int64_t k, int x_dt) {
    static const char *env_min = diag_env("NNQ_DENSE_MIN_M");   // tuning aid
    const int64_t min_m = env_min ? atoll(env_min) : 256;
    return ctx->d_dense && x_dt == NNQ_BF16 && m >= min_m && k >= kDgBK && k % kDgBK == 0 && n >= 1 &&
           (size_t)n * (size_t)k * 2 <= ctx->dense_bytes && m < (1ll << 31) && n < (1ll << 31) && encode_fn() != nullptr;
}
bool gemm_dense_supported(const nnq_ctx *ctx, const nnq_weight *w, int64_t m, int x_dt) {
    // Formats whose fused decode reads its raw blocks through the TMA ring keep it for longer. Measured on
    // 4096 x 4096, 12288 x 4096 and 4096 x 12288 (us, fused / decoded once): Q4_K (either element order)
    // 26 / 34, 53 / 68, 50 / 97 at 256 rows, 38 / 37, 75 / 95, 69 / 99 at 512 rows, 64 / 41, 142 / 122,
    // 127 / 113 at 1024 rows; Q8_0 29 / 42, 58 / 84, 55 / 113 at 256 rows, 47 / 43, 113 / 111, 100 / 115 at
    // 512 rows (its 512-row tile has no room for the ring).
    if (w) {
        const bool q4k = w->fmt == NNQ_Q4_K || w->fmt == NNQ_Q4_K_GGML;
        const bool q8 = w->fmt == NNQ_Q8_0 && w->k % 256 == 0;
        if ((q4k && m <= 512) || (q8 && m < 384)) return false;
    }
    return w && w->d_raw && gemm_dense_shape_ok(ctx, m, w->n, w->k, x_dt);
}

nnq_status dense_scratch_reserve(nnq_ctx *ctx, int64_t n, int64_t k) {
    if (k < kDgBK || k % kDgBK) return NNQ_OK;
    const size_t need = (size_t)n * (size_t)k * 2;
    if (need <= ctx->dense_bytes) return NNQ_OK;
    cudaFree(ctx->d_dense);   // load time: synchronising here is fine
    ctx->d_dense = nullptr;
    ctx->dense_bytes = 0;
    nnq_status s = check_cuda(ctx, cudaMalloc(&ctx->d_dense, need), "cudaMalloc bf16 weight scratch");
    if (s != NNQ_OK) return s;
    ctx->dense_bytes = need;
    return NNQ_OK;
}

// 256-wide tiles unless they would leave more than half of the SMs without a tile (few row tiles,
// narrow weights): then twice as many 128-wide tiles still fit one wave. (Measured: 4096 x 4096 at
// 512 rows 64 -> 128 tiles, +13 %; 1024 x 5120 at 4096 rows, 128 tiles of 256 beat 256 of 128.)
static int dg_pick_bn(const nnq_ctx *ctx, int64_t m_tiles, int64_t n) {
    return 2 * m_tiles * ((n + 255) / 256) <= ctx->sm_count ? 128 : 256;
}

static nnq_status dg_configure(nnq_ctx *ctx, int bn) {
    static bool configured[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int which = bn == 256 ? 0 : 1;
    if (dev >= 0 && dev < 64 && !configured[dev][which]) {
        const int smem_bytes = kDgStages * dg_stage_bytes(bn) + 1024;
        nnq_status s = check_cuda(ctx, bn == 256 ? cudaFuncSetAttribute(gemm_dense_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes)
                                                 : cudaFuncSetAttribute(gemm_dense_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes),
                                  "GEMM attribute");
        if (s != NNQ_OK) return s;
        configured[dev][which] = true;
    }
    return NNQ_OK;
}

// The GEMM alone: w_bf16 is a bf16 [n, k] weight in device memory (16-byte aligned).
nnq_status launch_gemm_dense_bf16(nnq_ctx *ctx, const void *w_bf16, const TcArgs &a, cudaStream_t stream) {
    CUtensorMap xmap, wmap;
    memset(&xmap, 0, sizeof(xmap));
    memset(&wmap, 0, sizeof(wmap));
    const int64_t m_tiles = (a.m + kDgBM - 1) / kDgBM;
    const int bn = dg_pick_bn(ctx, m_tiles, a.n);
    if (!make_map(a.x, a.m, a.k, kDgBM, &xmap) || !make_map(w_bf16, a.n, a.k, bn, &wmap))
        return fail(ctx, NNQ_ERR_DISPATCH_FAILED, "tensor map creation failed");
    nnq_status s = dg_configure(ctx, bn);
    if (s != NNQ_OK) return s;
    const int smem_bytes = kDgStages * dg_stage_bytes(bn) + 1024;
    const int64_t tiles = m_tiles * ((a.n + bn - 1) / bn);
    const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
    if (bn == 256)
        gemm_dense_kernel<256><<<grid, kDgThreads, smem_bytes, stream>>>(xmap, wmap, a.bias, a.y, (int)a.m, (int)a.n, (int)a.k, a.y_dt, ctx->d_status, nullptr, 0, nullptr, 0.0f);
    else
        gemm_dense_kernel<128><<<grid, kDgThreads, smem_bytes, stream>>>(xmap, wmap, a.bias, a.y, (int)a.m, (int)a.n, (int)a.k, a.y_dt, ctx->d_status, nullptr, 0, nullptr, 0.0f);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "bf16 GEMM launch");
}

nnq_status launch_gemm_dense(nnq_ctx *ctx, const TcArgs &a, cudaStream_t stream) {
    // a bf16 weight is its own decoded form
    if (a.fmt == NNQ_BF16_DENSE && !((uintptr_t)a.w & 15u)) return launch_gemm_dense_bf16(ctx, a.w, a, stream);
    Geometry g = geometry(a.fmt);
    const int64_t nchunks = a.n * (a.k / g.elems) * (g.elems / 32);
    cudaError_t e;
    switch (a.fmt) {
#define NNQ_DB(F) case F: e = launch_dequant_bf16<F>(a.w, a.scales, nchunks, ctx->d_dense, ctx->sm_count, stream); break
        NNQ_DB(NNQ_Q4_0); NNQ_DB(NNQ_Q4_1); NNQ_DB(NNQ_Q8_0); NNQ_DB(NNQ_Q4_K); NNQ_DB(NNQ_Q4_K_GGML); NNQ_DB(NNQ_Q6_K);
        NNQ_DB(NNQ_MXFP4_CORE); NNQ_DB(NNQ_MXFP4_SPLIT); NNQ_DB(NNQ_MXFP4_GPTOSS); NNQ_DB(NNQ_Q5_0); NNQ_DB(NNQ_Q5_1);
        NNQ_DB(NNQ_Q2_K); NNQ_DB(NNQ_Q3_K); NNQ_DB(NNQ_Q5_K);
        NNQ_DB(NNQ_F32_DENSE); NNQ_DB(NNQ_BF16_DENSE);
#undef NNQ_DB
        default: return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", a.fmt);
    }
    ctx->launches++;
    nnq_status s = check_cuda(ctx, e, "bf16 decode launch");
    if (s != NNQ_OK) return s;
    return launch_gemm_dense_bf16(ctx, ctx->d_dense, a, stream);
}

bool gemm_dense_grouped_supported(const nnq_ctx *ctx, const TcGroupArgs &g) {
    if (g.kn && (g.fmt != NNQ_MXFP4_GPTOSS || g.n % kKnTile || g.k % kKnTile || ((uintptr_t)g.w & 15u))) return false;
    return ctx->d_dense && g.k >= kDgBK && g.k % kDgBK == 0 && g.experts >= 1 && g.experts <= kDgMaxGroups && g.rows_upper >= 1 &&
           (size_t)g.experts * (size_t)g.n * (size_t)g.k * 2 <= ctx->dense_bytes && g.rows_upper < (1ll << 30) &&
           (int64_t)g.experts * g.n < (1ll << 31) && encode_fn() != nullptr;
}

bool gemm_dense_grouped_fuses_swiglu(const TcGroupArgs &g) {
    return g.h_out != nullptr && (g.fmt == NNQ_MXFP4_SPLIT || g.fmt == NNQ_MXFP4_GPTOSS) && g.n % 2 == 0 &&
           (int64_t)g.experts * g.n * (g.k / 32) < (1ll << 31);
}

nnq_status launch_gemm_dense_grouped(nnq_ctx *ctx, const TcGroupArgs &g, cudaStream_t stream) {
    // the experts' raw blocks are one contiguous [experts, N, K] tensor: one decode launch
    Geometry geo = geometry(g.fmt);
    const int64_t nchunks = (int64_t)g.experts * g.n * (g.k / geo.elems) * (geo.elems / 32);
    cudaError_t e;
    // SwiGLU in the GEMM's epilogue (g.h_out given): needs the gate / up rows interleaved in the decoded copy,
    // which the direct MXFP4 decode can write at no cost
    const bool fuse = gemm_dense_grouped_fuses_swiglu(g);
    const int cpr = (int)(g.k / 32), half = fuse ? (int)(g.n / 2) : 0;
    if (g.kn) {
        dequant_kn_bf16_kernel<<<dim3((unsigned)(g.n / kKnTile), (unsigned)(g.k / kKnTile), (unsigned)g.experts), 128, 0, stream>>>(
            g.w, g.scales, static_cast<__nv_bfloat16 *>(ctx->d_dense), (int)g.k, (int)g.n, half);
        e = cudaGetLastError();
    } else
    switch (g.fmt) {
#define NNQ_DB(F) case F: e = launch_dequant_bf16<F>(g.w, g.scales, nchunks, ctx->d_dense, ctx->sm_count, stream, cpr, half); break
        NNQ_DB(NNQ_Q4_0); NNQ_DB(NNQ_Q4_1); NNQ_DB(NNQ_Q8_0); NNQ_DB(NNQ_Q4_K); NNQ_DB(NNQ_Q4_K_GGML); NNQ_DB(NNQ_Q6_K);
        NNQ_DB(NNQ_MXFP4_CORE); NNQ_DB(NNQ_MXFP4_SPLIT); NNQ_DB(NNQ_MXFP4_GPTOSS); NNQ_DB(NNQ_Q5_0); NNQ_DB(NNQ_Q5_1);
        NNQ_DB(NNQ_Q2_K); NNQ_DB(NNQ_Q3_K); NNQ_DB(NNQ_Q5_K);
        NNQ_DB(NNQ_F32_DENSE); NNQ_DB(NNQ_BF16_DENSE);
#undef NNQ_DB
        default: return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown format %d", g.fmt);
    }
    ctx->launches++;
    nnq_status s = check_cuda(ctx, e, "bf16 decode launch");
    if (s != NNQ_OK) return s;
    CUtensorMap xmap, wmap;
    memset(&xmap, 0, sizeof(xmap));
    memset(&wmap, 0, sizeof(wmap));
    // row tiles of all experts: at most rows / 128 + one ragged tile per expert
    const int bn = dg_pick_bn(ctx, g.rows_upper / kDgBM + g.experts, g.n);
    if (!make_map(g.x_bf16, g.rows_upper, g.k, kDgBM, &xmap) || !make_map(ctx->d_dense, (int64_t)g.experts * g.n, g.k, bn, &wmap))
        return fail(ctx, NNQ_ERR_DISPATCH_FAILED, "tensor map creation failed");
    s = dg_configure(ctx, bn);
    if (s != NNQ_OK) return s;
    const int smem_bytes = kDgStages * dg_stage_bytes(bn) + 1024;
    if (bn == 256)
        gemm_dense_kernel<256><<<ctx->sm_count, kDgThreads, smem_bytes, stream>>>(xmap, wmap, g.bias, g.y, (int)g.rows_upper, (int)g.n, (int)g.k, NNQ_F32,
                                                                                  ctx->d_status, g.offsets, g.experts, fuse ? g.h_out : nullptr, g.swiglu_limit);
    else
        gemm_dense_kernel<128><<<ctx->sm_count, kDgThreads, smem_bytes, stream>>>(xmap, wmap, g.bias, g.y, (int)g.rows_upper, (int)g.n, (int)g.k, NNQ_F32,
                                                                                  ctx->d_status, g.offsets, g.experts, fuse ? g.h_out : nullptr, g.swiglu_limit);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "grouped bf16 GEMM launch");
}

}  // namespace nnq
