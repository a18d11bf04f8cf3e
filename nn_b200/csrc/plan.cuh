// A compiled sequence of M = 1 products run by ONE persistent kernel.
//
// A decode step is a chain of small matrix-vector products (per layer: q/k/v, o, gate/up, down),
// each reading a few tens of MB of weights. Launched one by one, every product pays a ramp (first
// tiles arrive) and a tail (the last SM finishes), which together cost a third of the HBM peak.
// Weights never depend on activations, so this kernel keeps every SM's copy ring full ACROSS the
// products: one CTA per SM walks the groups of the plan in order, and only the activations wait
// for the group that produces them (a device-wide arrival counter per group).
//
// Work split. A group is up to kPlanMaxJobs products that share their activations; its tiles
// (16 rows x 256 weights, 2304 bytes, stored contiguously by (row tile, k tile)) are numbered
// 0 .. tiles-1 and CTA c owns a contiguous range of them. With at least one row tile per CTA the
// ranges are whole row tiles (row tiles c*R/C .. (c+1)*R/C): every row is finished inside one CTA
// and nothing crosses CTAs (a hand-over through global memory costs more than the few percent of
// imbalance). With fewer row tiles than CTAs the tiles themselves are dealt out evenly and a row
// tile that straddles CTAs goes through a global partial-sum slot per (row tile, CTA) and an
// arrival counter: the last CTA to arrive adds the parts in CTA order and writes the rows.
// Inside the CTA, warp w takes tiles lo+w, lo+w+W, ... through a private ring of bulk copies, so
// no warp ever waits for another on the data path. Each tile's 16 partial sums go to a
// shared-memory slot; after the group's last tile the CTA adds the slots of every row tile in k
// order (fixed order: deterministic). Counters only ever count up (a row tile with n parts is
// complete when its counter is a multiple of n), so nothing is reset between launches.
#pragma once
#include "skinny_m1.cuh"

namespace nnq {

#ifndef NNQ_PLAN_WARPS
#define NNQ_PLAN_WARPS 16
#endif
constexpr int kPlanWarps = NNQ_PLAN_WARPS;
constexpr int kPlanMaxJobs = 4;
constexpr int kPlanMaxStages = 6;

struct PlanJobDev {
    const uint8_t *tiled;
    const float *bias;
    void *y;
    int n;          // real rows
    int rt_begin;   // first row tile of this job in the group's numbering
};

struct PlanGroupDev {
    const void *x;      // activations shared by the group's jobs, [kt * 256]
    int kt;             // tiles along K
    int row_tiles;      // of all jobs
    int tiles;          // row_tiles * kt
    int njobs;
    int dep;            // group whose completion the activations wait for; -1 = ready at launch
    int fix_off;        // first float of this group's cross-CTA partial sums
    int cnt_off;        // first arrival counter of this group's row tiles
    int pmax;           // most CTAs any row tile of the group is spread over
    int fused;          // 0, or 1 + index of this group among the plan's exchanged (row-parallel) groups
    int pad[3];
    PlanJobDev job[kPlanMaxJobs];
};

struct PlanParams {
    const PlanGroupDev *groups;
    int ngroups;
    int nfused;          // exchanged groups in the plan
    unsigned *done;      // [ngroups] CTAs that have finished the group, all launches so far
    unsigned *cnt;       // arrival counters of the row tiles
    float *scratch;      // cross-CTA partial sums
    unsigned *epoch;     // completed launches of this plan
    int *status;
    int y_dt;
    int stages;
    int kt_max;          // largest kt of any group (size of the activation image)
    int acc_slots;       // largest per-CTA tile count of any group
    unsigned spin_limit; // bound of a dependency wait (polls)
    FusedReduce fr;
    unsigned *prof;      // builds with -DNNQ_PLAN_PROF only: [group][cta][8] clock stamps of thread 0
};

// First tile of CTA c (its range ends where CTA c + 1 begins) for a group of row_tiles x kt tiles
// over nc CTAs: whole row tiles when there is at least one per CTA, else an even deal of tiles.
__host__ __device__ inline int plan_lo(int c, int nc, int row_tiles, int kt) {
    if (row_tiles >= nc) return (int)(((long long)c * row_tiles) / nc) * kt;
    return (int)(((long long)c * row_tiles * kt) / nc);
}
// The CTA that owns tile i under the even deal of `tiles` tiles (fewer row tiles than CTAs).
__host__ __device__ inline int plan_owner(int i, int nc, int tiles) { return (int)((((long long)i + 1) * nc - 1) / tiles); }

// A row tile whose k range is spread over several CTAs: how many parts it has and which of them
// CTA `c` (whose range starts at tile `lo`) holds. With at least one tile per CTA the parts are
// the CTAs from the owner of the row tile's first tile to the owner of its last; with fewer tiles
// than CTAs every tile sits in a CTA of its own.
struct PlanParts {
    int parts, part;
};
__host__ __device__ inline PlanParts plan_parts(int rt, int kt, int tiles, int nc, int c, int lo) {
    PlanParts p;
    if (tiles >= nc) {
        const int c_first = plan_owner(rt * kt, nc, tiles), c_last = plan_owner((rt + 1) * kt - 1, nc, tiles);
        p.parts = c_last - c_first + 1;
        p.part = c - c_first;
    } else {
        p.parts = kt;
        p.part = lo - rt * kt;
    }
    return p;
}

struct PlanSmem {
    int ring_off, xs_off, xs_lo_off, tab_off, xinv_off, acc_off, bar_off, flag_off, desc_off, total;
};

__host__ __device__ inline PlanSmem plan_smem(int kt_max, int acc_slots, int stages, bool f32x) {
    PlanSmem p;
    p.ring_off = 0;
    p.xs_off = kPlanWarps * stages * kTileBytes;
    p.xs_lo_off = p.xs_off + kt_max * 1024;
    p.tab_off = p.xs_lo_off + (f32x ? kt_max * 1024 : 0);
    p.xinv_off = p.tab_off + kt_max * 64;
    p.acc_off = (p.xinv_off + kt_max * 4 + 15) & ~15;
    p.bar_off = p.acc_off + acc_slots * 64;
    p.flag_off = p.bar_off + kPlanWarps * kPlanMaxStages * 8;
    p.desc_off = p.flag_off + 16;
    p.total = p.desc_off + (int)sizeof(PlanGroupDev);
    return p;
}

// read-only load of a pointer field of a descriptor
template <typename T>
__device__ __forceinline__ T *ldg_ptr(T *const *p) {
    return reinterpret_cast<T *>(__ldg(reinterpret_cast<const unsigned long long *>(p)));
}

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <bool F32X>
__global__ void __launch_bounds__(kPlanWarps * 32, 1)
plan_q4k_kernel(const __grid_constant__ PlanParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int stages = P.stages;
    const PlanSmem L = plan_smem(P.kt_max, P.acc_slots, stages, F32X);
    uint8_t *xs = smem + L.xs_off;
    uint8_t *xs_lo = smem + L.xs_lo_off;
    float *tab = reinterpret_cast<float *>(smem + L.tab_off);
    float *xinv = reinterpret_cast<float *>(smem + L.xinv_off);
    float *acc = reinterpret_cast<float *>(smem + L.acc_off);
    volatile int *dead = reinterpret_cast<volatile int *>(smem + L.flag_off);
    PlanGroupDev *gd = reinterpret_cast<PlanGroupDev *>(smem + L.desc_off);   // the current group's descriptor

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
    const int g = lane >> 2, t = lane & 3;
    const int cta = blockIdx.x, nc = gridDim.x;
    uint8_t *ring = smem + warp * stages * kTileBytes;
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t bar_s = smem_u32(smem + L.bar_off) + warp * kPlanMaxStages * 8;

    if (tid == 0) *dead = 0;
    if (lane == 0) {
        for (int d = 0; d < stages; d++) mbar_init(bar_s + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // every launch of the plan adds nc arrivals to each group's counter
    const unsigned epoch = *reinterpret_cast<volatile unsigned *>(P.epoch);
    const unsigned target = (epoch + 1u) * (unsigned)nc;
    unsigned ar_base = 0, ar_limit = 0;
    if (P.nfused) {
        ar_base = *reinterpret_cast<volatile unsigned *>(P.fr.peers[P.fr.rank]);
        ar_limit = comm_spin_limit(P.fr.peers[P.fr.rank]);
    }

    // ---- weight stream of this warp: runs ahead of the compute, across group boundaries ----
    int pf_g = -1, pf_i = 0, pf_hi = 0, pf_job_end = 0, pf_slot = 0;
    const uint8_t *pf_src = nullptr;
    bool pf_done = false;
    unsigned issued = 0, consumed = 0;
    auto pf_locate = [&]() {   // job of tile pf_i in group pf_g
        const PlanGroupDev *G = P.groups + pf_g;
        const int kt = __ldg(&G->kt), nj = __ldg(&G->njobs);
        int j = 0;
        for (int q = 1; q < nj; q++)
            if (pf_i >= __ldg(&G->job[q].rt_begin) * kt) j = q;
        const int tb = __ldg(&G->job[j].rt_begin) * kt;
        const int te = j + 1 < nj ? __ldg(&G->job[j + 1].rt_begin) * kt : __ldg(&G->tiles);
        pf_src = ldg_ptr(&G->job[j].tiled) + (size_t)(pf_i - tb) * kTileBytes;
        pf_job_end = te < pf_hi ? te : pf_hi;
    };
    auto pf_next_group = [&]() {
        for (;;) {
            if (++pf_g >= P.ngroups) {
                pf_done = true;
                return;
            }
            const int rts = __ldg(&P.groups[pf_g].row_tiles), kt = __ldg(&P.groups[pf_g].kt);
            pf_i = plan_lo(cta, nc, rts, kt) + warp;
            pf_hi = plan_lo(cta + 1, nc, rts, kt);
            if (pf_i < pf_hi) {
                pf_locate();
                return;
            }
        }
    };
    pf_next_group();
    const int is_lane0 = lane == 0;
    auto issue = [&]() {
        if (!pf_done) {
            issue_tile(ring_s + pf_slot * kTileBytes, pf_src, bar_s + 8 * pf_slot, is_lane0);
            issued++;
            pf_slot = pf_slot + 1 == stages ? 0 : pf_slot + 1;
            pf_i += kPlanWarps;
            pf_src += (size_t)kPlanWarps * kTileBytes;
            if (pf_i >= pf_job_end) {
                if (pf_i < pf_hi) pf_locate();
                else pf_next_group();
            }
        }
    };
    for (int d = 0; d < stages; d++) issue();

    Consts K;
    K.init();
    BRegs B, BL;
#pragma unroll
    for (int p = 0; p < 4; p++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            B.v[p][h] = make_uint4(0, 0, 0, 0);
            BL.v[p][h] = make_uint4(0, 0, 0, 0);
        }
    const uint32_t xs_s = smem_u32(xs) + lane * 32, xs_lo_s = smem_u32(xs_lo) + lane * 32;
    int slot = 0;
    uint32_t phase = 0;
    bool warp_failed = false;

    // Writes one finished row tile: lanes 0..15 hold its 16 sums. With an exchanged group the sums
    // are this rank's share: every value travels to each peer as one 8-byte (value, sequence
    // number) store, the lane then waits (bounded) for the peers' pairs of its row and adds all
    // shares in rank order, so every rank ends up with the same bits.
    auto store_rows = [&](int rt, float v) {
        const int nj = gd->njobs;
        int j = 0;
        for (int q = 1; q < nj; q++)
            if (rt >= gd->job[q].rt_begin) j = q;
        const int row = (rt - gd->job[j].rt_begin) * 16 + (lane & 15);
        if (lane >= 16 || row >= gd->job[j].n) return;
        const int fused = gd->fused;
        if (fused) {
            const unsigned seq = ar_base + (unsigned)fused;
            const int par = (int)(seq & 1u);
            const size_t mine = comm_data_offset(par, P.fr.rank, P.fr.world, P.fr.slot_bytes) + (size_t)row * 8;
            for (int p = 0; p < P.fr.world; p++)
                if (p != P.fr.rank)
                    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(P.fr.peers[p] + mine),
                                 "r"(__float_as_uint(v)), "r"(seq) : "memory");
            const uint8_t *local = P.fr.peers[P.fr.rank];
            float sum = 0.0f;
            bool ok = true;
            for (int r = 0; r < P.fr.world; r++) {
                if (r == P.fr.rank) {
                    sum += v;
                    continue;
                }
                const uint8_t *src = local + comm_data_offset(par, r, P.fr.world, P.fr.slot_bytes) + (size_t)row * 8;
                uint32_t bits = 0, tag = 0;
                unsigned spins = 0;
                do {
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(bits), "=r"(tag) : "l"(src) : "memory");
                } while (tag != seq && ++spins <= ar_limit);
                ok = ok && tag == seq;
                sum += __uint_as_float(bits);
            }
            if (!ok) {
                atomicExch(P.status, 1);
                *dead = 1;
            }
            v = sum;
        }
        const float *bias = gd->job[j].bias;
        if (bias) v += __ldg(bias + row);
        void *y = gd->job[j].y;
        if (P.y_dt == NNQ_F32) reinterpret_cast<float *>(y)[row] = v;
        else reinterpret_cast<__nv_bfloat16 *>(y)[row] = __float2bfloat16_rn(v);
    };

#pragma unroll 1
    for (int gi = 0; gi < P.ngroups; gi++) {
        const PlanGroupDev *G = P.groups + gi;
        const int kt = __ldg(&G->kt), tiles = __ldg(&G->tiles);
        const int row_tiles = __ldg(&G->row_tiles);
        const int lo = plan_lo(cta, nc, row_tiles, kt), hi = plan_lo(cta + 1, nc, row_tiles, kt);
#ifdef NNQ_PLAN_PROF
        unsigned *pr = P.prof ? P.prof + ((size_t)gi * nc + cta) * 8 : nullptr;
        if (pr && tid == 0) pr[0] = (unsigned)clock64();
#define PLAN_STAMP(i) if (pr && tid == 0) pr[i] = (unsigned)clock64();
#else
#define PLAN_STAMP(i)
#endif

        // the group's descriptor goes to shared memory (the previous group is done with its copy:
        // every thread has passed the barrier that follows the previous group's last use)
        if (tid >= 32 && tid < 32 + (int)(sizeof(PlanGroupDev) / 4))
            reinterpret_cast<uint32_t *>(gd)[tid - 32] = __ldg(reinterpret_cast<const uint32_t *>(G) + (tid - 32));
        // ---- the activations wait for the group that writes them ----
        if (tid == 0) {
            const int dep = __ldg(&G->dep);
            if (dep >= 0) {
                unsigned spins = 0;
                while ((int)(ld_acquire_u32(P.done + dep) - target) < 0) {
                    if (++spins > P.spin_limit) {
                        atomicExch(P.status, 1);
                        *dead = 1;
                        break;
                    }
                }
            }
        }
        __syncthreads();
        if (*dead) break;   // uniform: nobody writes the flag between this barrier and the next
        PLAN_STAMP(1)
        const void *gx = gd->x;
        stage_x_warp_batched<F32X, true, F32X ? 1 : 3>(gx, warp, kt, kPlanWarps, xs, xs_lo, tab, xinv, lane);
        __syncthreads();
        PLAN_STAMP(2)

        // ---- this warp's tiles of the group ----
        {
            int i = lo + warp;
            int kb = i % kt;
            const int kstep = kPlanWarps % kt;
#pragma unroll 1
            for (; i < hi; i += kPlanWarps) {
                if (!warp_failed && !mbar_wait_fast(bar_s + 8 * slot, phase)) {
                    // the copy never landed: record it and stop touching the ring (the copies
                    // still in flight are waited for, bounded, before the kernel returns)
                    warp_failed = true;
                    if (lane == 0) {
                        atomicExch(P.status, 1);
                        *dead = 1;
                    }
                }
                if (warp_failed) continue;
                float yg = 0.0f, yg8 = 0.0f;
                tile_mac<F32X>(ring + slot * kTileBytes, xs_s + kb * 1024, xs_lo_s + kb * 1024, tab + kb * 16, xinv[kb],
                               lane, g, t, K, B, BL, yg, yg8);
                yg += __shfl_xor_sync(0xFFFFFFFFu, yg, 1);
                yg8 += __shfl_xor_sync(0xFFFFFFFFu, yg8, 1);
                yg += __shfl_xor_sync(0xFFFFFFFFu, yg, 2);
                yg8 += __shfl_xor_sync(0xFFFFFFFFu, yg8, 2);
                if (t == 0) {
                    float *a = acc + (i - lo) * 16;
                    a[g] = yg;
                    a[8 + g] = yg8;
                }
                consumed++;
                if (++slot == stages) {
                    slot = 0;
                    phase ^= 1u;
                }
                __syncwarp();   // all lanes have read the slot before it is refilled
                issue();
                kb += kstep;
                if (kb >= kt) kb -= kt;
            }
        }
        PLAN_STAMP(6)
        __syncthreads();
        PLAN_STAMP(3)

        // ---- row tiles of this CTA's range: 32 lanes per row tile (two halves of its k range) ----
        if (lo < hi) {
            const int rt_first = lo / kt, rt_last = (hi - 1) / kt;
            const int l16 = lane & 15, q = lane >> 4;
            for (int rt = rt_first + warp; rt <= rt_last; rt += kPlanWarps) {
                const int a = max(lo, rt * kt), b = min(hi, (rt + 1) * kt);
                const int mid = a + ((b - a + 1) >> 1);
                const int s = q ? mid : a, e = q ? b : mid;
                float v0 = 0.0f, v1 = 0.0f, v2 = 0.0f, v3 = 0.0f;   // fixed order, four chains
                const float *ap = acc + (s - lo) * 16 + l16;
                int i = s;
                for (; i + 3 < e; i += 4, ap += 64) {
                    v0 += ap[0];
                    v1 += ap[16];
                    v2 += ap[32];
                    v3 += ap[48];
                }
                for (; i < e; i++, ap += 16) v0 += ap[0];
                float v = (v0 + v1) + (v2 + v3);
                v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
                if (a == rt * kt && b == (rt + 1) * kt) {
                    store_rows(rt, v);
                } else {
                    // the row tile is spread over several CTAs: hand in this part, the last one adds
                    const PlanParts pp = plan_parts(rt, kt, tiles, nc, cta, lo);
                    const unsigned parts = (unsigned)pp.parts;
                    float *slots = P.scratch + __ldg(&G->fix_off) + (size_t)rt * __ldg(&G->pmax) * 16;
                    if (q == 0) {
                        __stcg(slots + pp.part * 16 + l16, v);
                        __threadfence();
                    }
                    __syncwarp();
                    unsigned old = 0;
                    if (lane == 0) old = atomicAdd(P.cnt + __ldg(&G->cnt_off) + rt, 1u);
                    old = __shfl_sync(0xFFFFFFFFu, old, 0);
                    if ((old + 1u) % parts == 0u) {
                        __threadfence();
                        float sum = 0.0f;
                        if (q == 0)
                            for (unsigned p = 0; p < parts; p++) sum += __ldcg(slots + p * 16 + l16);
                        store_rows(rt, sum);
                    }
                }
            }
        }
        __syncthreads();
        PLAN_STAMP(4)
        if (tid == 0) {
            __threadfence();
            if (gi < P.ngroups - 1) {
                // nobody needs the old value: the thread goes on to the next group at once
                asm volatile("red.relaxed.gpu.global.add.u32 [%0], 1;" ::"l"(P.done + gi) : "memory");
            } else if (atomicAdd(P.done + gi, 1u) + 1u == target) {
                // the last CTA of the launch: the next launch counts from here
                *reinterpret_cast<volatile unsigned *>(P.epoch) = epoch + 1u;
                if (P.nfused) *reinterpret_cast<volatile unsigned *>(P.fr.peers[P.fr.rank]) = ar_base + (unsigned)P.nfused;
            }
        }
        PLAN_STAMP(5)
    }

    // a failed launch: give the copies still in flight a bounded chance to land before the
    // CTA's shared memory goes away
    if (consumed < issued) {
        for (unsigned n = consumed; n < issued; n++) {
            if (!mbar_wait(bar_s + 8 * slot, phase)) break;
            if (++slot == stages) {
                slot = 0;
                phase ^= 1u;
            }
        }
    }
}

}  // namespace nnq
