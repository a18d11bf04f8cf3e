// Host side of the compiled product plan (nnq_plan_*): records a sequence of M = 1 products as a
// decoder issues them, lays out the device-side descriptors and counters once, and runs the whole
// sequence as one cooperative launch of plan_q4k_kernel (plan.cuh).
#include <string.h>

#include <new>
#include <vector>

#include "plan.cuh"

namespace nnq {
nnq_status comm_view(nnq_comm *c, CommView *out);   // comm.cu
}

struct nnq_plan {
    nnq_ctx *ctx;
    int x_dt, y_dt, flags;
    std::vector<nnq::PlanGroupDev> groups;
    std::vector<size_t> x_bytes;                 // per group: bytes of activations read
    std::vector<std::vector<size_t>> y_bytes;    // per group and job: bytes written
    bool finalized;
    nnq_comm *comm;
    nnq::CommView cv;
    int nfused;
    int nc, stages, kt_max, acc_slots, smem_bytes;
    unsigned spin_limit;
    nnq::PlanGroupDev *d_groups;
    unsigned *d_words;     // [0] epoch, then done[ngroups], then the row-tile counters
    size_t words;
    float *d_scratch;
    size_t scratch_floats;
    unsigned *d_prof;      // builds with -DNNQ_PLAN_PROF only
};

namespace nnq {

// Largest per-CTA tile count and the most parts any row tile is spread over, for a group of
// `row_tiles` x `kt` tiles on `nc` CTAs.
static void group_geometry(int row_tiles, int kt, int nc, int *max_tiles, int *pmax) {
    const int tiles = row_tiles * kt;
    int mt = 0, pm = 1;
    for (int c = 0; c < nc; c++) {
        const int n = plan_lo(c + 1, nc, row_tiles, kt) - plan_lo(c, nc, row_tiles, kt);
        if (n > mt) mt = n;
    }
    if (row_tiles < nc) {   // tiles dealt out evenly: row tiles straddle CTAs
        if (tiles < nc) {
            pm = kt;
        } else {
            for (int rt = 0; rt < row_tiles; rt++) {
                const int p = plan_owner((rt + 1) * kt - 1, nc, tiles) - plan_owner(rt * kt, nc, tiles) + 1;
                if (p > pm) pm = p;
            }
        }
    }
    *max_tiles = mt;
    *pmax = pm;
}

static bool overlap(const void *a, size_t an, const void *b, size_t bn) {
    const uintptr_t a0 = (uintptr_t)a, b0 = (uintptr_t)b;
    return an && bn && a0 < b0 + bn && b0 < a0 + an;
}

template <bool F32X>
static cudaError_t launch_plan(const PlanParams &P, int grid, int smem_bytes, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(plan_q4k_kernel<F32X>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kPlanWarps * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    // the CTAs wait for one another on the group counters: all of them must be resident
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, plan_q4k_kernel<F32X>, P);
}

}  // namespace nnq

using namespace nnq;

extern "C" {

nnq_status nnq_plan_geometry(int row_tiles, int k_tiles, int ctas, int *max_tiles_per_cta, int *max_parts) {
    if (row_tiles < 1 || k_tiles < 1 || ctas < 1 || (long long)row_tiles * k_tiles * ctas >= (1ll << 31)) return NNQ_ERR_INVALID_ARG;
    int mt = 0, pm = 0;
    group_geometry(row_tiles, k_tiles, ctas, &mt, &pm);
    if (max_tiles_per_cta) *max_tiles_per_cta = mt;
    if (max_parts) *max_parts = pm;
    return NNQ_OK;
}

nnq_status nnq_plan_create(nnq_ctx *ctx, nnq_dtype x_dt, nnq_dtype y_dt, int flags, nnq_plan **out) {
    if (!ctx || !out) return NNQ_ERR_INVALID_ARG;
    *out = nullptr;
    if ((int)x_dt < 0 || x_dt > NNQ_BF16 || (int)y_dt < 0 || y_dt > NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown dtype");
    if (flags & ~NNQ_PLAN_ANALYZE_DEPS) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown plan flags %d", flags);
    nnq_plan *p = new (std::nothrow) nnq_plan();
    if (!p) return fail(ctx, NNQ_ERR_OUT_OF_MEMORY, "host allocation failed");
    p->ctx = ctx;
    p->x_dt = x_dt;
    p->y_dt = y_dt;
    p->flags = flags;
    p->finalized = false;
    p->comm = nullptr;
    p->nfused = 0;
    p->spin_limit = 1u << 21;
    p->d_groups = nullptr;
    p->d_words = nullptr;
    p->d_scratch = nullptr;
    p->d_prof = nullptr;
    *out = p;
    return NNQ_OK;
}

static nnq_status plan_add(nnq_plan *p, int count, const nnq_weight *const *w, const void *x_dev, const float *const *bias_dev,
                           void *const *y_dev, nnq_comm *comm) {
    if (!p) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = p->ctx;
    if (p->finalized) return fail(ctx, NNQ_ERR_INVALID_ARG, "the plan has been finalized");
    if (count < 1 || count > kPlanMaxJobs || !w || !y_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "a group holds 1..%d products", kPlanMaxJobs);
    if (!x_dev || ((uintptr_t)x_dev & 15u)) return fail(ctx, NNQ_ERR_INVALID_ARG, "x must be a 16-byte aligned device pointer");
    PlanGroupDev G;
    memset(&G, 0, sizeof(G));
    G.x = x_dev;
    G.njobs = count;
    std::vector<size_t> yb;
    const size_t es_y = p->y_dt == NNQ_F32 ? 4 : 2;
    int rt = 0;
    for (int i = 0; i < count; i++) {
        const nnq_weight *wi = w[i];
        if (!wi) return fail(ctx, NNQ_ERR_NOT_QUANTIZED, "weight tensor is not quantized");
        if (wi->ctx != ctx) return fail(ctx, NNQ_ERR_INVALID_ARG, "weight belongs to another context");
        if (wi->tiled_layout != kTiledQ4K || !wi->d_tiled)
            return fail(ctx, NNQ_ERR_UNSUPPORTED, "a plan takes Q4_K weights with K a multiple of 256 (format %d, K = %lld)", wi->fmt, (long long)wi->k);
        if (wi->k != w[0]->k) return fail(ctx, NNQ_ERR_SHAPE_MISMATCH, "the products of a group share their activations: K must agree");
        if (wi->n < 1) return fail(ctx, NNQ_ERR_INVALID_SHAPE, "empty weight");
        if (!y_dev[i] || ((uintptr_t)y_dev[i] & 15u)) return fail(ctx, NNQ_ERR_INVALID_ARG, "y must be a 16-byte aligned device pointer");
        PlanJobDev &J = G.job[i];
        J.tiled = wi->d_tiled;
        J.bias = bias_dev ? bias_dev[i] : nullptr;
        J.y = y_dev[i];
        J.n = (int)wi->n;
        J.rt_begin = rt;
        rt += (int)((wi->n + 15) / 16);
        yb.push_back((size_t)wi->n * es_y);
    }
    G.kt = (int)(w[0]->k / 256);
    G.row_tiles = rt;
    if ((long long)rt * G.kt >= (1ll << 22)) return fail(ctx, NNQ_ERR_UNSUPPORTED, "group of %d x %d tiles is too large for a plan", rt, G.kt);
    G.tiles = rt * G.kt;
    if (comm) {
        if (count != 1) return fail(ctx, NNQ_ERR_INVALID_ARG, "an exchanged group holds one product");
        nnq::CommView cv;
        nnq_status s = comm_view(comm, &cv);
        if (s != NNQ_OK) return s;
        if (p->comm && p->comm != comm) return fail(ctx, NNQ_ERR_INVALID_ARG, "a plan uses one communicator");
        if ((size_t)w[0]->n * 8 > cv.slot_bytes)
            return fail(ctx, NNQ_ERR_UNSUPPORTED, "the communicator's slots hold %zu bytes, %lld rows need %lld", cv.slot_bytes,
                        (long long)w[0]->n, (long long)w[0]->n * 8);
        p->comm = comm;
        p->cv = cv;
        G.fused = ++p->nfused;
    }
    p->groups.push_back(G);
    p->x_bytes.push_back((size_t)w[0]->k * (p->x_dt == NNQ_F32 ? 4 : 2));
    p->y_bytes.push_back(yb);
    return NNQ_OK;
}

nnq_status nnq_plan_add(nnq_plan *p, int count, const nnq_weight *const *w, const void *x_dev, const float *const *bias_dev,
                        void *const *y_dev) {
    return plan_add(p, count, w, x_dev, bias_dev, y_dev, nullptr);
}

nnq_status nnq_plan_add_reduced(nnq_plan *p, nnq_comm *comm, const nnq_weight *w, const void *x_dev, const float *bias_dev,
                                void *y_dev) {
    if (!p) return NNQ_ERR_INVALID_ARG;
    if (!comm) return fail(p->ctx, NNQ_ERR_INVALID_ARG, "NULL communicator");
    const nnq_weight *ws[1] = {w};
    const float *bs[1] = {bias_dev};
    void *ys[1] = {y_dev};
    return plan_add(p, 1, ws, x_dev, bias_dev ? bs : nullptr, ys, comm);
}

nnq_status nnq_plan_finalize(nnq_plan *p) {
    if (!p) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = p->ctx;
    if (p->finalized) return NNQ_OK;
    if (p->groups.empty()) return fail(ctx, NNQ_ERR_INVALID_ARG, "the plan is empty");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    const bool f32x = p->x_dt == NNQ_F32;
    const int ng = (int)p->groups.size();

    // dependencies: by default every group waits for the one before it (what issuing the products
    // one after another on a stream guarantees); with NNQ_PLAN_ANALYZE_DEPS a group waits for the
    // latest earlier group whose buffers overlap its own (read after write, write after read,
    // write after write), and for nothing when there is none. An exchanged group and its successor
    // always wait for their predecessor: the exchange slots are reused every second exchange.
    int last_fused = -1;
    for (int g = 0; g < ng; g++) {
        PlanGroupDev &G = p->groups[g];
        int dep = g - 1;
        if (p->flags & NNQ_PLAN_ANALYZE_DEPS) {
            dep = -1;
            for (int e = 0; e < g; e++) {
                const PlanGroupDev &E = p->groups[e];
                bool hit = false;
                for (int j = 0; j < E.njobs && !hit; j++) hit = overlap(E.job[j].y, p->y_bytes[e][j], G.x, p->x_bytes[g]);
                for (int j = 0; j < G.njobs && !hit; j++) {
                    hit = overlap(E.x, p->x_bytes[e], G.job[j].y, p->y_bytes[g][j]);
                    for (int i = 0; i < E.njobs && !hit; i++) hit = overlap(E.job[i].y, p->y_bytes[e][i], G.job[j].y, p->y_bytes[g][j]);
                }
                if (hit) dep = e;
            }
            if (G.fused && dep < g - 1) dep = g - 1;
            if (dep < last_fused) dep = last_fused;
        }
        G.dep = dep;
        if (G.fused) last_fused = g;
    }

    // grid: one CTA per SM, all resident (cooperative launch); ring depth from what shared memory is left
    int kt_max = 0;
    for (const PlanGroupDev &G : p->groups) kt_max = G.kt > kt_max ? G.kt : kt_max;
    int nc = ctx->sm_count;
    int acc_slots = 0;
    size_t fix_floats = 0, counters = 0;
    for (PlanGroupDev &G : p->groups) {
        int mt = 0, pm = 0;
        group_geometry(G.row_tiles, G.kt, nc, &mt, &pm);
        if (mt > acc_slots) acc_slots = mt;
        G.pmax = pm;
        if (fix_floats + (size_t)G.row_tiles * pm * 16 >= ((size_t)1 << 31)) return fail(ctx, NNQ_ERR_UNSUPPORTED, "the plan's partial-sum area would exceed 8 GiB");
        G.fix_off = (int)fix_floats;
        fix_floats += (size_t)G.row_tiles * pm * 16;
        G.cnt_off = (int)counters;
        counters += (size_t)G.row_tiles;
    }
    int stages = 0;
    for (int st = kPlanMaxStages; st >= 2; st--)
        if (plan_smem(kt_max, acc_slots, st, f32x).total <= kSmemMax) {
            stages = st;
            break;
        }
    if (stages == 0)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "K = %d or a group of %d tiles per SM does not fit the plan kernel's shared memory", kt_max * 256, acc_slots);
    const int smem_bytes = plan_smem(kt_max, acc_slots, stages, f32x).total;
    cudaError_t e = f32x ? cudaFuncSetAttribute(plan_q4k_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax)
                         : cudaFuncSetAttribute(plan_q4k_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
    if ((s = check_cuda(ctx, e, "plan kernel attribute")) != NNQ_OK) return s;
    int per_sm = 0;
    e = f32x ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, plan_q4k_kernel<true>, kPlanWarps * 32, smem_bytes)
             : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, plan_q4k_kernel<false>, kPlanWarps * 32, smem_bytes);
    if ((s = check_cuda(ctx, e, "plan kernel occupancy")) != NNQ_OK) return s;
    if (per_sm < 1) return fail(ctx, NNQ_ERR_UNSUPPORTED, "the plan kernel does not fit an SM (%d bytes of shared memory)", smem_bytes);

    p->nc = nc;
    p->stages = stages;
    p->kt_max = kt_max;
    p->acc_slots = acc_slots;
    p->smem_bytes = smem_bytes;
    p->words = 1 + (size_t)ng + counters;
    p->scratch_floats = fix_floats ? fix_floats : 16;
    s = check_cuda(ctx, cudaMalloc(&p->d_groups, sizeof(PlanGroupDev) * ng), "cudaMalloc plan groups");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMalloc(&p->d_words, p->words * 4), "cudaMalloc plan counters");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMalloc(&p->d_scratch, p->scratch_floats * 4), "cudaMalloc plan partial sums");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemcpy(p->d_groups, p->groups.data(), sizeof(PlanGroupDev) * ng, cudaMemcpyHostToDevice), "plan upload");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemset(p->d_words, 0, p->words * 4), "plan counters");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaDeviceSynchronize(), "plan set-up");
    if (s != NNQ_OK) {
        cudaFree(p->d_groups);
        cudaFree(p->d_words);
        cudaFree(p->d_scratch);
        p->d_groups = nullptr;
        p->d_words = nullptr;
        p->d_scratch = nullptr;
        return s;
    }
    p->finalized = true;
    return NNQ_OK;
}

nnq_status nnq_plan_run(nnq_plan *p, void *stream) {
    if (!p) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = p->ctx;
    if (!p->finalized) return fail(ctx, NNQ_ERR_INVALID_ARG, "the plan has not been finalized");
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    PlanParams P;
    memset(&P, 0, sizeof(P));
    P.groups = p->d_groups;
    P.ngroups = (int)p->groups.size();
    P.nfused = p->nfused;
    P.epoch = p->d_words;
    P.done = p->d_words + 1;
    P.cnt = p->d_words + 1 + P.ngroups;
    P.scratch = p->d_scratch;
    P.status = ctx->d_status;
    P.y_dt = p->y_dt;
    P.stages = p->stages;
    P.kt_max = p->kt_max;
    P.acc_slots = p->acc_slots;
    P.spin_limit = p->spin_limit;
#ifdef NNQ_PLAN_PROF
    P.prof = p->d_prof;
#endif
    if (p->nfused) {
        P.fr.peers = p->cv.peer_table;
        P.fr.slot_bytes = p->cv.slot_bytes;
        P.fr.rank = p->cv.rank;
        P.fr.world = p->cv.world;
        P.fr.enabled = 1;
    }
    cudaError_t e = p->x_dt == NNQ_F32 ? launch_plan<true>(P, p->nc, p->smem_bytes, (cudaStream_t)stream)
                                       : launch_plan<false>(P, p->nc, p->smem_bytes, (cudaStream_t)stream);
    ctx->launches++;
    return check_cuda(ctx, e, "plan launch");
}

nnq_status nnq_plan_reset(nnq_plan *p, void *stream) {
    if (!p) return NNQ_ERR_INVALID_ARG;
    if (!p->finalized) return NNQ_OK;
    nnq_status s = check_cuda(p->ctx, cudaSetDevice(p->ctx->device), "cudaSetDevice");
    if (s == NNQ_OK) s = check_cuda(p->ctx, cudaMemsetAsync(p->d_words, 0, p->words * 4, (cudaStream_t)stream), "plan counters");
    return s;
}

nnq_status nnq_plan_set_spin_limit(nnq_plan *p, unsigned polls) {
    if (!p || polls == 0) return NNQ_ERR_INVALID_ARG;
    p->spin_limit = polls;
    return NNQ_OK;
}

nnq_status nnq_plan_info(const nnq_plan *p, int *groups, int *ctas, int *stages, size_t *smem_bytes, size_t *scratch_bytes) {
    if (!p) return NNQ_ERR_INVALID_ARG;
    if (groups) *groups = (int)p->groups.size();
    if (ctas) *ctas = p->finalized ? p->nc : 0;
    if (stages) *stages = p->finalized ? p->stages : 0;
    if (smem_bytes) *smem_bytes = p->finalized ? (size_t)p->smem_bytes : 0;
    if (scratch_bytes) *scratch_bytes = p->finalized ? p->scratch_floats * 4 + p->words * 4 : 0;
    return NNQ_OK;
}

nnq_status nnq_plan_dependency(const nnq_plan *p, int group, int *dep) {
    if (!p || !dep || group < 0 || group >= (int)p->groups.size() || !p->finalized) return NNQ_ERR_INVALID_ARG;
    *dep = p->groups[group].dep;
    return NNQ_OK;
}

#ifdef NNQ_PLAN_PROF
// diagnostic build: per group and CTA, eight clock stamps of thread 0 (phase boundaries)
NNQ_API nnq_status nnq_plan_profile(nnq_plan *p, unsigned *host_out, size_t words) {
    if (!p || !p->finalized) return NNQ_ERR_INVALID_ARG;
    const size_t need = p->groups.size() * (size_t)p->nc * 8;
    if (!p->d_prof) {
        cudaMalloc(&p->d_prof, need * 4);
        cudaMemset(p->d_prof, 0, need * 4);
        return NNQ_OK;
    }
    cudaDeviceSynchronize();
    cudaMemcpy(host_out, p->d_prof, (words < need ? words : need) * 4, cudaMemcpyDeviceToHost);
    return NNQ_OK;
}
#endif

void nnq_plan_destroy(nnq_plan *p) {
    if (!p) return;
    cudaSetDevice(p->ctx->device);
    cudaDeviceSynchronize();
    cudaFree(p->d_groups);
    cudaFree(p->d_words);
    cudaFree(p->d_scratch);
    cudaGetLastError();
    delete p;
}

}  // extern "C"
