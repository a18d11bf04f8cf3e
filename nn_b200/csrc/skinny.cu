// Host side of the skinny (decode) kernels: tiled copies of the weights, choice of kernel and
// launch geometry. The kernels live in skinny_m1.cuh (Q4_K, one token), skinny_mn.cuh (token-column
// and grouped kernels) and skinny_repack.cuh.
#include <stdlib.h>
#include <string.h>

#include "skinny_repack.cuh"

namespace nnq {

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------

nnq_status skinny_init(nnq_ctx *) { return NNQ_OK; }

size_t tiled_bytes_kn(int64_t n, int64_t k, int *sb_out) {
    const int sb = k % 256 == 0 ? 8 : (k % 192 == 0 ? 6 : 0);
    if (sb_out) *sb_out = sb;
    if (sb == 0 || n <= 0 || n % 32 != 0 || n > (1 << 24) || k > (1 << 24)) return 0;
    return (size_t)(n / 16) * (size_t)(k / (32 * sb)) * (size_t)(288 * sb);
}

nnq_status repack_kn_into(nnq_ctx *ctx, const uint8_t *d_codes, const uint8_t *d_scales, int64_t n, int64_t k, uint8_t *dst) {
    int sb = 0;
    if (tiled_bytes_kn(n, k, &sb) == 0) return fail(ctx, NNQ_ERR_UNSUPPORTED, "no tiled layout for a [K, N] expert tensor with K = %lld, N = %lld", (long long)k, (long long)n);
    const int64_t total = n * (k / 32);
    const int grid = (int)((total + 255) / 256);
    const int ktiles = (int)(k / (32 * sb));
    if (sb == 8) repack_mxfp4_kn_kernel<8><<<grid, 256>>>(d_codes, d_scales, dst, (int)n, (int)k, ktiles);
    else repack_mxfp4_kn_kernel<6><<<grid, 256>>>(d_codes, d_scales, dst, (int)n, (int)k, ktiles);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "repack launch");
}

static int tile_bytes_of(int fmt, int sb) {
    switch (fmt) {
        case NNQ_Q4_K: case NNQ_Q4_K_GGML: return TileFmt<NNQ_Q4_K>::kBytes;
        case NNQ_Q8_0: return TileFmt<NNQ_Q8_0>::kBytes;
        case NNQ_Q6_K: return TileFmt<NNQ_Q6_K>::kBytes;
        case NNQ_Q4_0: return TileFmt<NNQ_Q4_0>::kBytes;
        case NNQ_Q4_1: return TileFmt<NNQ_Q4_1>::kBytes;
        case NNQ_MXFP4_CORE: case NNQ_MXFP4_SPLIT: return 128 + 256 * sb;
        default: return 0;
    }
}

// Sub-blocks per tile row for this format and K; 0 = no tiled layout.
static int tile_sb_of(int fmt, int64_t k) {
    switch (fmt) {
        case NNQ_Q4_K: case NNQ_Q4_K_GGML: case NNQ_Q8_0: case NNQ_Q6_K: case NNQ_Q4_0: case NNQ_Q4_1: return k % 256 == 0 ? 8 : 0;
        case NNQ_MXFP4_CORE: case NNQ_MXFP4_SPLIT: return k % 256 == 0 ? 8 : (k % 192 == 0 ? 6 : 0);
        default: return 0;
    }
}

size_t tiled_bytes_for(int fmt, int64_t n, int64_t k, int *sb_out) {
    const int sb = tile_sb_of(fmt, k);
    if (sb_out) *sb_out = sb;
    if (sb == 0 || n <= 0 || k <= 0 || n > (1 << 24) || k > (1 << 24)) return 0;
    return (size_t)((n + 15) / 16) * (size_t)(k / (32 * sb)) * tile_bytes_of(fmt, sb);
}

nnq_status repack_into(nnq_ctx *ctx, int fmt, const uint8_t *d_raw, const uint8_t *d_scales, int64_t n, int64_t k,
                       uint8_t *d) {
    int sb = 0;
    const size_t bytes = tiled_bytes_for(fmt, n, k, &sb);
    if (bytes == 0) return fail(ctx, NNQ_ERR_UNSUPPORTED, "no tiled layout for format %d with K = %lld", fmt, (long long)k);
    const int ktiles = (int)(k / (32 * sb));
    nnq_status s = NNQ_OK;
    if (n % 16) s = check_cuda(ctx, cudaMemset(d, 0, bytes), "cudaMemset tiled weight");
    if (s != NNQ_OK) return s;
    const int64_t total = fmt == NNQ_MXFP4_CORE || fmt == NNQ_MXFP4_SPLIT ? n * (k / 32) : n * ktiles * 8;
    const int grid = (int)((total + 255) / 256);
    const int split = fmt == NNQ_MXFP4_SPLIT;
    switch (fmt) {
        case NNQ_Q4_K: repack_q4k_kernel<false><<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        case NNQ_Q4_K_GGML: repack_q4k_kernel<true><<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        case NNQ_Q8_0: repack_q8_0_kernel<<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        case NNQ_Q6_K: repack_q6_k_kernel<<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        case NNQ_Q4_0: repack_q4x_kernel<false><<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        case NNQ_Q4_1: repack_q4x_kernel<true><<<grid, 256>>>(d_raw, d, (int)n, ktiles); break;
        default:
            if (sb == 8) repack_mxfp4_kernel<8><<<grid, 256>>>(d_raw, d_scales, d, (int)n, ktiles, split);
            else repack_mxfp4_kernel<6><<<grid, 256>>>(d_raw, d_scales, d, (int)n, ktiles, split);
            break;
    }
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "repack launch");
}

nnq_status build_tiled_buffer(nnq_ctx *ctx, int fmt, const uint8_t *d_raw, const uint8_t *d_scales, int64_t n,
                              int64_t k, uint8_t **out, size_t *out_bytes, int *out_sb) {
    *out = nullptr;
    *out_bytes = 0;
    *out_sb = 0;
    int sb = 0;
    const size_t bytes = tiled_bytes_for(fmt, n, k, &sb);
    if (bytes == 0) return NNQ_OK;
    uint8_t *d = nullptr;
    nnq_status s = check_cuda(ctx, cudaMalloc(&d, bytes), "cudaMalloc tiled weight");
    if (s != NNQ_OK) return s;
    s = repack_into(ctx, fmt, d_raw, d_scales, n, k, d);
    if (s == NNQ_OK) s = check_cuda(ctx, cudaDeviceSynchronize(), "repack");
    if (s != NNQ_OK) {
        cudaFree(d);
        return s;
    }
    *out = d;
    *out_bytes = bytes;
    *out_sb = sb;
    return NNQ_OK;
}

static int layout_of(int fmt) {
    switch (fmt) {
        case NNQ_Q4_K: case NNQ_Q4_K_GGML: return kTiledQ4K;
        case NNQ_Q8_0: return kTiledQ8_0;
        case NNQ_Q6_K: return kTiledQ6K;
        case NNQ_MXFP4_CORE: case NNQ_MXFP4_SPLIT: return kTiledMxfp4;
        case NNQ_Q4_0: return kTiledQ4_0;
        case NNQ_Q4_1: return kTiledQ4_1;
        default: return kTiledNone;
    }
}

nnq_status build_tiled(nnq_ctx *ctx, nnq_weight *w) {
    nnq_status s = build_tiled_buffer(ctx, w->fmt, w->d_raw, w->d_scales, w->n, w->k, &w->d_tiled, &w->tiled_bytes, &w->tile_sb);
    if (s != NNQ_OK) return s;
    w->tiled_layout = w->d_tiled ? layout_of(w->fmt) : kTiledNone;
    return NNQ_OK;
}

// Ring depth and CTAs per SM that fit shared memory for this K. More resident warps beat a
// deeper ring (the kernel is bound by instruction latency, not by bytes in flight), so: three
// CTAs per SM with a 2-deep ring when that fits, else two with up to 4 stages, else one;
// stages = 0 when K is too large altogether.
static void pick_stages(int kblocks, bool f32x, int *stages, int *ctas_per_sm) {
    static const char *env_st = diag_env("NNQ_SKINNY_STAGES");  // tuning aid
    const int forced = env_st ? atoi(env_st) : 0;
    static const char *env_ctas = diag_env("NNQ_SKINNY_CTAS");  // tuning aid
    int max_ctas = f32x ? 2 : 3;   // register budget of the two instantiations
    if (env_ctas && atoi(env_ctas) > 0 && atoi(env_ctas) < max_ctas) max_ctas = atoi(env_ctas);
    for (int ctas = max_ctas; ctas >= 1; ctas--) {
        const int budget = kSmemMax / ctas - 1024;
        const int hi = forced > 0 ? forced : (ctas == 3 ? 2 : kMaxStages);
        const int lo = forced > 0 ? forced : 2;
        for (int st = hi; st >= lo; st--)
            if (smem_plan(kblocks, st, f32x).total <= budget) {
                *stages = st;
                *ctas_per_sm = ctas;
                return;
            }
    }
    *stages = 0;
    *ctas_per_sm = 0;
}

bool skinny_supported(const nnq_weight *w, int64_t m, int x_dt) {
    if (!w || w->tiled_layout == kTiledNone || m < 1 || m > kSkinnyMaxM) return false;
    // token-column kernel: f32 activations (two MMAs per product) up to 8 tokens only
    if (m > 1 || w->tiled_layout != kTiledQ4K) return x_dt == NNQ_BF16 || m <= 8;
    int st, cps;
    pick_stages((int)(w->k / 256), x_dt == NNQ_F32, &st, &cps);
    return st > 0;
}

template <bool F32X, int KS, bool FUSED = false>
static cudaError_t launch_kernel(const SkinnyParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(skinny_q4k_m1_kernel<F32X, KS, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax - 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    // programmatic dependent launch: the kernel prefetches weights while its predecessor in
    // the stream drains, and waits (griddepcontrol.wait) before reading activations
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const char *env_pdl = diag_env("NNQ_SKINNY_PDL");  // tuning aid
    cfg.numAttrs = env_pdl && atoi(env_pdl) == 0 ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, skinny_q4k_m1_kernel<F32X, KS, FUSED>, P);
}

template <bool F32X, bool FUSED>
static cudaError_t launch_ks_f(int ksplit, const SkinnyParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    switch (ksplit) {
        case 1: return launch_kernel<F32X, 1, FUSED>(P, grid, smem_bytes, stream);
        case 2: return launch_kernel<F32X, 2, FUSED>(P, grid, smem_bytes, stream);
        case 4: return launch_kernel<F32X, 4, FUSED>(P, grid, smem_bytes, stream);
        default: return launch_kernel<F32X, 8, FUSED>(P, grid, smem_bytes, stream);
    }
}

template <bool F32X>
static cudaError_t launch_ks(int ksplit, const SkinnyParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    return P.fr.enabled ? launch_ks_f<F32X, true>(ksplit, P, grid, smem_bytes, stream)
                        : launch_ks_f<F32X, false>(ksplit, P, grid, smem_bytes, stream);
}

template <int FMT, int SB, int NT, bool F32X>
static cudaError_t launch_mn(const SkinnyParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(skinny_mn_kernel<FMT, SB, NT, F32X>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, skinny_mn_kernel<FMT, SB, NT, F32X>, P);
}

template <int FMT, int SB = 8>
static cudaError_t launch_mn_fmt(const SkinnyParams &P, int nt, bool f32x, int grid, int smem_bytes, cudaStream_t stream) {
    if (f32x) return launch_mn<FMT, SB, 1, true>(P, grid, smem_bytes, stream);
    return nt == 1 ? launch_mn<FMT, SB, 1, false>(P, grid, smem_bytes, stream) : launch_mn<FMT, SB, 2, false>(P, grid, smem_bytes, stream);
}

#ifdef NNQ_DIAG
// Diagnostic only (NNQ_SKINNY_DIAG=4): read the tiled weights of the jobs with plain coalesced
// 16-byte loads and nothing else -- the read bandwidth a launch of this size can reach.
__global__ void __launch_bounds__(256) stream_read_kernel(const SkinnyParams P, int *sink) {
    uint32_t acc = 0;
    for (int j = 0; j < P.njobs; j++) {
        const uint4 *p = reinterpret_cast<const uint4 *>(P.job[j].tiled);
        size_t n16 = (size_t)P.job[j].row_tiles * P.kblocks * (kTileBytes / 16);
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
            uint4 v = __ldg(p + i);
            acc ^= v.x ^ v.y ^ v.z ^ v.w;
        }
    }
    if (acc == 0x12345678u && sink) *sink = 1;   // keeps the loads alive; sink is NULL
}
#endif

// One launch: jobs that share their activations (same x pointer, same K).
static nnq_status launch_group(nnq_ctx *ctx, const SkinnyJob *jobs, int count, int x_dt, int m, int y_dt,
                               cudaStream_t stream, const FusedReduce *fr = nullptr) {
    SkinnyParams P;
    memset(&P, 0, sizeof(P));
    if (fr) P.fr = *fr;
    P.njobs = count;
    P.m = m;
    P.y_dt = y_dt;
    P.x = jobs[0].x;
    const int tile_sb = jobs[0].w->tile_sb;
    P.kblocks = (int)(jobs[0].w->k / (32 * tile_sb));
    P.status = ctx->d_status;
    static const char *env_diag = diag_env("NNQ_SKINNY_DIAG");
    P.diag = env_diag ? atoi(env_diag) : 0;
    static const char *env_l2 = diag_env("NNQ_SKINNY_L2PF");
    P.l2_prefetch = env_l2 ? atoi(env_l2) : 0;
    const bool f32x = x_dt == NNQ_F32;
    int ctas_per_sm = 0;
    const int layout = jobs[0].w->tiled_layout;
    // One token of bf16 activations on few row tiles (one wave of the token-column kernel, e.g. the
    // 4096-row o / down projections): the token-column kernel has no activation staging after the
    // dependency wait and wins by a few percent; larger launches keep the M = 1 kernel.
    static const char *env_tc = diag_env("NNQ_SKINNY_TOKCOL");  // tuning aid: the row-tile limit of that rule
    int64_t job_tiles = 0;
    for (int i = 0; i < count; i++) job_tiles += (jobs[i].w->n + 15) / 16;
    const int64_t tokcol_limit = env_tc ? atoi(env_tc) : 2 * ctx->sm_count;
    const bool token_columns = m > 1 || layout != kTiledQ4K || (!f32x && !fr && job_tiles <= tokcol_limit);
    if (!token_columns) pick_stages(P.kblocks, f32x, &P.stages, &ctas_per_sm);
    else P.stages = 2;
    if (fr && ctas_per_sm > 2) ctas_per_sm = 2;   // register budget of the fused variant
    if (P.stages == 0) return fail(ctx, NNQ_ERR_UNSUPPORTED, "K = %lld is too large for the skinny kernel", (long long)jobs[0].w->k);
    int tiles = 0;
    for (int i = 0; i < count; i++) {
        const nnq_weight *w = jobs[i].w;
        SkinnyJobDev &J = P.job[i];
        J.tiled = w->d_tiled;
        J.bias = jobs[i].bias;
        J.y = jobs[i].y;
        J.n = (int)w->n;
        J.row_tiles = (int)((w->n + 15) / 16);
        J.tile_begin = tiles;
        tiles += J.row_tiles;
    }
    P.total_tiles = tiles;
    if (token_columns) {
        // a unit is one row tile, its K split over the 8 warps
        const int nt = m <= 8 ? 1 : 2;
        const int smem_bytes = mn_plan(tile_bytes_of(jobs[0].w->fmt, tile_sb), P.stages, nt).total;
        int per_sm = kSmemMax / (smem_bytes + 1024);
        if (per_sm > 2) per_sm = 2;   // register budget of the kernel
        int grid = tiles < ctx->sm_count * per_sm ? tiles : ctx->sm_count * per_sm;
        cudaError_t e;
        if (layout == kTiledQ4K) e = launch_mn_fmt<NNQ_Q4_K>(P, nt, f32x, grid, smem_bytes, stream);
        else if (layout == kTiledQ8_0) e = launch_mn_fmt<NNQ_Q8_0>(P, nt, f32x, grid, smem_bytes, stream);
        else if (layout == kTiledQ6K) e = launch_mn_fmt<NNQ_Q6_K>(P, nt, f32x, grid, smem_bytes, stream);
        else if (layout == kTiledQ4_0) e = launch_mn_fmt<NNQ_Q4_0>(P, nt, f32x, grid, smem_bytes, stream);
        else if (layout == kTiledQ4_1) e = launch_mn_fmt<NNQ_Q4_1>(P, nt, f32x, grid, smem_bytes, stream);
        else if (tile_sb == 8) e = launch_mn_fmt<NNQ_MXFP4_SPLIT, 8>(P, nt, f32x, grid, smem_bytes, stream);
        else e = launch_mn_fmt<NNQ_MXFP4_SPLIT, 6>(P, nt, f32x, grid, smem_bytes, stream);
        ctx->launches++;
        return check_cuda(ctx, e, "skinny launch");
    }
#ifdef NNQ_DIAG
    if (P.diag == 4) {
        stream_read_kernel<<<ctx->sm_count * 8, 256, 0, stream>>>(P, nullptr);
        ctx->launches++;
        return check_cuda(ctx, cudaGetLastError(), "diag launch");
    }
#endif
    // K split over the warps of a CTA: all 8 warps share a row tile when K allows, so that even
    // the smallest projections spread over every SM
    const int slots = ctx->sm_count * ctas_per_sm;
    int ksplit = 1;
    while (ksplit < kWarps && P.kblocks >= 2 * ksplit) ksplit *= 2;
    static const char *env_ks = diag_env("NNQ_SKINNY_KS");  // tuning aid
    if (env_ks && atoi(env_ks) > 0) ksplit = atoi(env_ks);
    // persistent grid: every CTA resident
    const int rg = kWarps / ksplit;
    const int units = (tiles + rg - 1) / rg;
    int grid = units < slots ? units : slots;
    static const char *env_grid = diag_env("NNQ_SKINNY_GRID");  // tuning aid
    if (env_grid && atoi(env_grid) > 0) grid = atoi(env_grid);
    if (grid > units) grid = units;
    if (grid < 1) grid = 1;
    int smem_bytes = smem_plan(P.kblocks, P.stages, f32x).total;
    cudaError_t e = f32x ? launch_ks<true>(ksplit, P, grid, smem_bytes, stream) : launch_ks<false>(ksplit, P, grid, smem_bytes, stream);
    ctx->launches++;
    return check_cuda(ctx, e, "skinny launch");
}

template <int FMT, int SB, int NT, bool F32X>
static cudaError_t launch_grouped_t(const GroupedParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(skinny_grouped_kernel<FMT, SB, NT, F32X>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemMax - 1024);   // the kernel also has a small static table
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    skinny_grouped_kernel<FMT, SB, NT, F32X><<<grid, kWarps * 32, smem_bytes, stream>>>(P);
    return cudaGetLastError();
}

template <int FMT, int SB>
static cudaError_t launch_grouped_x(const GroupedParams &P, bool f32x, int nt, int grid, int smem_bytes, cudaStream_t stream) {
    if (f32x) return launch_grouped_t<FMT, SB, 1, true>(P, grid, smem_bytes, stream);   // two MMAs per product: 8 rows
    return nt == 2 ? launch_grouped_t<FMT, SB, 2, false>(P, grid, smem_bytes, stream)
                   : launch_grouped_t<FMT, SB, 1, false>(P, grid, smem_bytes, stream);
}

nnq_status launch_grouped(nnq_ctx *ctx, const GroupedArgs &a, cudaStream_t stream) {
    if (a.experts < 1 || a.experts > kMoeMaxExperts) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad expert count %d", a.experts);
    int sb = 0;
    if ((a.kn_gptoss ? tiled_bytes_kn(a.n, a.k, &sb) : tiled_bytes_for(a.fmt, a.n, a.k, &sb)) == 0)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "no tiled layout for the grouped product");
    GroupedParams P;
    memset(&P, 0, sizeof(P));
    P.tiled = a.tiled;
    P.expert_stride = a.expert_stride;
    P.bias = a.bias;
    P.x = a.x;
    P.rowtok = a.rowtok;
    P.offset = a.offset;
    P.out = a.out;
    P.experts = a.experts;
    P.top_k = a.top_k;
    P.n = (int)a.n;
    P.row_tiles = (int)((a.n + 15) / 16);
    P.kblocks = (int)(a.k / (32 * sb));
    P.stages = 2;
    P.status = ctx->d_status;
    const bool f32x = a.x_dt == NNQ_F32;
    // 16-row groups once the experts see 5 or more rows on average (bf16 activations only)
    const int nt = !f32x && a.max_rows >= 5 * (int64_t)a.experts ? 2 : 1;
    const int smem_bytes = mn_plan(a.kn_gptoss ? 288 * sb : tile_bytes_of(a.fmt, sb), P.stages, nt).total;
    // every expert may end with a partly filled row group
    const int64_t max_units = (a.max_rows / (8 * nt) + a.experts) * P.row_tiles;
    int64_t grid = 2 * (int64_t)ctx->sm_count;
    if (grid > max_units) grid = max_units;
    if (grid < 1) grid = 1;
    cudaError_t e;
    if (a.kn_gptoss) {
        e = sb == 8 ? launch_grouped_x<NNQ_MXFP4_GPTOSS, 8>(P, f32x, nt, (int)grid, smem_bytes, stream)
                    : launch_grouped_x<NNQ_MXFP4_GPTOSS, 6>(P, f32x, nt, (int)grid, smem_bytes, stream);
        ctx->launches++;
        return check_cuda(ctx, e, "grouped product launch");
    }
    switch (layout_of(a.fmt)) {
        case kTiledQ4K: e = launch_grouped_x<NNQ_Q4_K, 8>(P, f32x, nt, (int)grid, smem_bytes, stream); break;
        case kTiledQ8_0: e = launch_grouped_x<NNQ_Q8_0, 8>(P, f32x, nt, (int)grid, smem_bytes, stream); break;
        case kTiledQ6K: e = launch_grouped_x<NNQ_Q6_K, 8>(P, f32x, nt, (int)grid, smem_bytes, stream); break;
        case kTiledQ4_0: e = launch_grouped_x<NNQ_Q4_0, 8>(P, f32x, nt, (int)grid, smem_bytes, stream); break;
        case kTiledQ4_1: e = launch_grouped_x<NNQ_Q4_1, 8>(P, f32x, nt, (int)grid, smem_bytes, stream); break;
        default:
            e = sb == 8 ? launch_grouped_x<NNQ_MXFP4_SPLIT, 8>(P, f32x, nt, (int)grid, smem_bytes, stream)
                        : launch_grouped_x<NNQ_MXFP4_SPLIT, 6>(P, f32x, nt, (int)grid, smem_bytes, stream);
            break;
    }
    ctx->launches++;
    return check_cuda(ctx, e, "grouped product launch");
}

bool skinny_fused_supported(const nnq_weight *w, int64_t m, int x_dt) {
    return m == 1 && w && w->tiled_layout == kTiledQ4K && skinny_supported(w, m, x_dt);
}

nnq_status launch_skinny_fused(nnq_ctx *ctx, const SkinnyJob &job, int x_dt, int y_dt, const FusedReduce &fr,
                               cudaStream_t stream) {
    if (!skinny_fused_supported(job.w, 1, x_dt)) return fail(ctx, NNQ_ERR_UNSUPPORTED, "fused product + all-reduce needs the M = 1 Q4_K kernel");
    return launch_group(ctx, &job, 1, x_dt, 1, y_dt, stream, &fr);
}

nnq_status launch_skinny(nnq_ctx *ctx, const SkinnyJob *jobs, int count, int x_dt, int64_t m, int y_dt,
                         cudaStream_t stream) {
    if (count < 1 || count > kSkinnyMaxJobs) return fail(ctx, NNQ_ERR_INVALID_ARG, "bad job count %d", count);
    if (m < 1 || m > kSkinnyMaxM) return fail(ctx, NNQ_ERR_UNSUPPORTED, "skinny kernels cover 1 <= M <= %d", kSkinnyMaxM);
    // consecutive jobs with the same activations and K go out together
    int i = 0;
    while (i < count) {
        int jn = i + 1;
        while (jn < count && jobs[jn].x == jobs[i].x && jobs[jn].w->k == jobs[i].w->k && jobs[jn].w->tiled_layout == jobs[i].w->tiled_layout) jn++;
        nnq_status s = launch_group(ctx, jobs + i, jn - i, x_dt, (int)m, y_dt, stream);
        if (s != NNQ_OK) return s;
        i = jn;
    }
    return NNQ_OK;
}

}  // namespace nnq
