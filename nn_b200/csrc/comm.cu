// One-shot all-reduce for the small messages of tensor-parallel decode (the [M, hidden] partial
// outputs of the row-parallel o_proj / down_proj: 8-16 KB at M = 1), over peer-mapped buffers on
// one NVLink/NVSwitch box. The reference has no counterpart (it is single-device).
//
// Every rank owns a buffer with one slot per (source rank, parity) and one flag per source rank;
// peers map it through CUDA IPC. A call with sequence number s (kept on the device, so that a
// captured graph can be replayed):
//   1. each rank stores its vector into slot[rank][s & 1] of every peer's buffer (plain peer stores),
//   2. fences, then stores s into flag[rank] of every peer,
//   3. waits (bounded) until its own flags from all peers show s,
//   4. sums the slots in rank order (bit-identical on every rank) and writes the result in place.
// Parity double-buffering is enough: a peer can be at most one call ahead, because call s + 1
// cannot finish without this rank's flag for s + 1. A wait that runs out sets the context's
// status word and the kernel returns (the result is then meaningless); nothing spins forever.
// Only plain loads / stores to peer memory are used: no multimem, no bulk copies.
#include <cuda_bf16.h>
#include <string.h>

#include <new>

#include "comm.cuh"
#include "nnq_internal.h"
#include "skinny.h"

struct nnq_comm {
    nnq_ctx *ctx;
    int rank, world;
    size_t slot_bytes;          // capacity of one message
    uint8_t *d_local;           // this rank's buffer
    uint8_t *peer[8];           // every rank's buffer as seen from here (peer[rank] == d_local)
    bool opened[8];
    uint8_t **d_peer_table;     // device copy of peer[]
};

namespace nnq {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
// loads that bypass L1, so that data a peer has just stored is seen
__device__ __forceinline__ float ld_fresh(const float *p) { return __ldcv(p); }
__device__ __forceinline__ __nv_bfloat16 ld_fresh(const __nv_bfloat16 *p) {
    unsigned short u = __ldcv(reinterpret_cast<const unsigned short *>(p));
    return __ushort_as_bfloat16(u);
}
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(uint8_t *const *peers, int rank, int world, size_t slot_bytes, T *buf, int count, int *status) {
    // let the next kernel of the stream start (it only prefetches weights until this kernel has
    // completed), and wait for the producer of `buf`
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint8_t *local = peers[rank];
    __shared__ unsigned seq_s, limit_s;
    __shared__ int failed_s;
    if (threadIdx.x == 0) {
        seq_s = *reinterpret_cast<volatile unsigned *>(local) + 1u;
        limit_s = comm_spin_limit(local);
        failed_s = 0;
    }
    __syncthreads();
    const unsigned seq = seq_s, limit = limit_s;
    const int parity = (int)(seq & 1u);
    // 1. push this rank's vector into every peer (and into its own slot)
    for (int p = 0; p < world; p++) {
        T *dst = reinterpret_cast<T *>(peers[p] + comm_data_offset(parity, rank, world, slot_bytes));
        for (int i = threadIdx.x; i < count; i += blockDim.x) dst[i] = buf[i];
    }
    __threadfence_system();
    __syncthreads();
    // 2. publish, 3. wait for everybody else's publication (one thread per peer)
    if (threadIdx.x < world) {
        const int p = threadIdx.x;
        volatile unsigned *remote_flag = reinterpret_cast<volatile unsigned *>(peers[p] + 64) + rank;
        *remote_flag = seq;
        volatile unsigned *my_flag = reinterpret_cast<volatile unsigned *>(local + 64) + p;
        unsigned spins = 0;
        while ((int)(*my_flag - seq) < 0) {
            if (++spins > limit) {
                failed_s = 1;
                break;
            }
        }
    }
    __syncthreads();
    __threadfence_system();
    if (failed_s) {
        if (threadIdx.x == 0) atomicExch(status, 1);
    } else {
        // 4. sum in rank order
        for (int i = threadIdx.x; i < count; i += blockDim.x) {
            float acc = 0.0f;
            for (int r = 0; r < world; r++) {
                const T *src = reinterpret_cast<const T *>(local + comm_data_offset(parity, r, world, slot_bytes));
                acc += to_f32<T>(ld_fresh(src + i));
            }
            buf[i] = from_f32<T>(acc);
        }
    }
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned *>(local) = seq;
}

// The same exchange for messages of tens of KB to MB (the [rows, hidden] partial sums of a prompt
// pass): up to 64 CTAs, each owning a contiguous run of 16-byte units. A CTA pushes its run to every
// peer; the last CTA of the rank to have pushed publishes the rank's flags; every CTA waits (bounded)
// for every peer's flag and sums its run in rank order; the last CTA to finish advances the epoch. No
// CTA waits for another CTA of its own grid, so the grid need not be resident at once. The two arrival
// counters live at bytes 132 and 136 of the buffer header and are left at zero.
template <typename T>
__global__ void __launch_bounds__(512)
allreduce_multi_kernel(uint8_t *const *peers, int rank, int world, size_t slot_bytes, T *buf, int64_t units, int *status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint8_t *local = peers[rank];
    __shared__ unsigned seq_s, limit_s;
    __shared__ int failed_s, last_s;
    if (threadIdx.x == 0) {
        seq_s = *reinterpret_cast<volatile unsigned *>(local) + 1u;
        limit_s = comm_spin_limit(local);
        failed_s = 0;
    }
    __syncthreads();
    const unsigned seq = seq_s, limit = limit_s;
    const int parity = (int)(seq & 1u);
    const int64_t per = (units + gridDim.x - 1) / gridDim.x;
    const int64_t lo = (int64_t)blockIdx.x * per, hi = lo + per < units ? lo + per : units;
    const uint4 *src = reinterpret_cast<const uint4 *>(buf);
    for (int p = 0; p < world; p++) {
        uint4 *dst = reinterpret_cast<uint4 *>(peers[p] + comm_data_offset(parity, rank, world, slot_bytes));
        for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    unsigned *pushed = reinterpret_cast<unsigned *>(local + 132), *done = reinterpret_cast<unsigned *>(local + 136);
    if (threadIdx.x == 0) {
        last_s = atomicAdd(pushed, 1u) == gridDim.x - 1;
        if (last_s) *pushed = 0;
    }
    __syncthreads();
    if (last_s && threadIdx.x < world) {
        __threadfence_system();
        *(reinterpret_cast<volatile unsigned *>(peers[threadIdx.x] + 64) + rank) = seq;
    }
    if (threadIdx.x < world) {
        volatile unsigned *my_flag = reinterpret_cast<volatile unsigned *>(local + 64) + threadIdx.x;
        unsigned spins = 0;
        while ((int)(*my_flag - seq) < 0) {
            if (++spins > limit) {
                failed_s = 1;
                break;
            }
        }
    }
    __syncthreads();
    __threadfence_system();
    if (failed_s) {
        if (threadIdx.x == 0) atomicExch(status, 1);
    } else {
        constexpr int PER = 16 / (int)sizeof(T);
        for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            float acc[PER];
#pragma unroll
            for (int j = 0; j < PER; j++) acc[j] = 0.0f;
            for (int r = 0; r < world; r++) {
                const uint4 *slot = reinterpret_cast<const uint4 *>(local + comm_data_offset(parity, r, world, slot_bytes));
                uint4 v;
                asm volatile("ld.global.cv.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(slot + i));
                const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
                for (int j = 0; j < PER; j++) acc[j] += to_f32<T>(e[j]);
            }
            uint4 o;
            T *oe = reinterpret_cast<T *>(&o);
#pragma unroll
            for (int j = 0; j < PER; j++) oe[j] = from_f32<T>(acc[j]);
            reinterpret_cast<uint4 *>(buf)[i] = o;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(done, 1u) == gridDim.x - 1) {
        *done = 0;
        *reinterpret_cast<volatile unsigned *>(local) = seq;
    }
}

nnq_status comm_view(nnq_comm *c, CommView *out) {
    if (!c || !out) return NNQ_ERR_INVALID_ARG;
    for (int p = 0; p < c->world; p++)
        if (!c->peer[p]) return fail(c->ctx, NNQ_ERR_INVALID_ARG, "peer %d has not been opened", p);
    out->peer_table = c->d_peer_table;
    out->slot_bytes = c->slot_bytes;
    out->rank = c->rank;
    out->world = c->world;
    return NNQ_OK;
}

}  // namespace nnq

using namespace nnq;

extern "C" {

nnq_status nnq_comm_create(nnq_ctx *ctx, int rank, int world, size_t max_bytes, nnq_comm **out) {
    if (!ctx || !out) return NNQ_ERR_INVALID_ARG;
    *out = nullptr;
    if (world < 1 || world > kCommMaxWorld || rank < 0 || rank >= world || max_bytes == 0 || max_bytes > ((size_t)1 << 24))
        return fail(ctx, NNQ_ERR_INVALID_ARG, "bad communicator spec rank=%d world=%d bytes=%zu", rank, world, max_bytes);
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    nnq_comm *c = new (std::nothrow) nnq_comm();
    if (!c) return fail(ctx, NNQ_ERR_OUT_OF_MEMORY, "host allocation failed");
    memset(c, 0, sizeof(*c));
    c->ctx = ctx;
    c->rank = rank;
    c->world = world;
    c->slot_bytes = (max_bytes + 255) & ~(size_t)255;
    const size_t total = comm_data_offset(2, 0, world, c->slot_bytes);
    s = check_cuda(ctx, cudaMalloc(&c->d_local, total), "cudaMalloc comm buffer");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemset(c->d_local, 0, total), "cudaMemset comm buffer");
    const unsigned default_limit = kCommSpins;
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMemcpy(c->d_local + kCommSpinLimitOffset, &default_limit, 4, cudaMemcpyHostToDevice), "comm wait bound");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaMalloc(&c->d_peer_table, sizeof(uint8_t *) * kCommMaxWorld), "cudaMalloc peer table");
    if (s == NNQ_OK) s = check_cuda(ctx, cudaDeviceSynchronize(), "comm init");
    if (s != NNQ_OK) {
        nnq_comm_destroy(c);
        return s;
    }
    c->peer[rank] = c->d_local;
    if (world == 1) s = check_cuda(ctx, cudaMemcpy(c->d_peer_table, c->peer, sizeof(c->peer), cudaMemcpyHostToDevice), "peer table");
    if (s != NNQ_OK) {
        nnq_comm_destroy(c);
        return s;
    }
    *out = c;
    return NNQ_OK;
}

nnq_status nnq_comm_get_handle(nnq_comm *c, void *handle64) {
    if (!c || !handle64) return NNQ_ERR_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaSetDevice(c->ctx->device);
    cudaIpcMemHandle_t h;
    nnq_status s = check_cuda(c->ctx, cudaIpcGetMemHandle(&h, c->d_local), "cudaIpcGetMemHandle");
    if (s != NNQ_OK) return s;
    memcpy(handle64, &h, 64);
    return NNQ_OK;
}

nnq_status nnq_comm_open_peers(nnq_comm *c, const void *handles) {
    if (!c || !handles) return NNQ_ERR_INVALID_ARG;
    cudaSetDevice(c->ctx->device);
    for (int p = 0; p < c->world; p++) {
        if (p == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)handles + 64 * p, 64);
        void *ptr = nullptr;
        nnq_status s = check_cuda(c->ctx, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
        if (s != NNQ_OK) return s;
        c->peer[p] = (uint8_t *)ptr;
        c->opened[p] = true;
    }
    return check_cuda(c->ctx, cudaMemcpy(c->d_peer_table, c->peer, sizeof(c->peer), cudaMemcpyHostToDevice), "peer table");
}

nnq_status nnq_comm_set_spin_limit(nnq_comm *c, unsigned polls) {
    if (!c || polls == 0) return NNQ_ERR_INVALID_ARG;
    cudaSetDevice(c->ctx->device);
    nnq_status s = check_cuda(c->ctx, cudaDeviceSynchronize(), "comm wait bound");
    if (s == NNQ_OK) s = check_cuda(c->ctx, cudaMemcpy(c->d_local + kCommSpinLimitOffset, &polls, 4, cudaMemcpyHostToDevice), "comm wait bound");
    return s;
}

nnq_status nnq_comm_local_buffer(nnq_comm *c, void **dev_ptr) {
    if (!c || !dev_ptr) return NNQ_ERR_INVALID_ARG;
    *dev_ptr = c->d_local;
    return NNQ_OK;
}

nnq_status nnq_comm_open_local_peers(nnq_comm *c, void *const *peer_dev_ptrs) {
    if (!c || !peer_dev_ptrs) return NNQ_ERR_INVALID_ARG;
    cudaSetDevice(c->ctx->device);
    for (int p = 0; p < c->world; p++) {
        if (p == c->rank) continue;
        if (!peer_dev_ptrs[p]) return fail(c->ctx, NNQ_ERR_INVALID_ARG, "peer %d: NULL buffer", p);
        c->peer[p] = (uint8_t *)peer_dev_ptrs[p];
        c->opened[p] = false;   // not an IPC mapping: nothing to close
    }
    return check_cuda(c->ctx, cudaMemcpy(c->d_peer_table, c->peer, sizeof(c->peer), cudaMemcpyHostToDevice), "peer table");
}

nnq_status nnq_comm_all_reduce(nnq_comm *c, void *buf_dev, nnq_dtype dt, int64_t count, void *stream) {
    if (!c) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = c->ctx;
    if ((int)dt < 0 || dt > NNQ_BF16) return fail(ctx, NNQ_ERR_INVALID_ARG, "unknown dtype");
    const size_t es = dt == NNQ_F32 ? 4 : 2;
    if (count < 0 || (size_t)count * es > c->slot_bytes)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "message of %lld elements exceeds the communicator's %zu-byte slots", (long long)count, c->slot_bytes);
    if (count == 0) return NNQ_OK;
    if (!buf_dev) return fail(ctx, NNQ_ERR_INVALID_ARG, "NULL buffer");
    for (int p = 0; p < c->world; p++)
        if (!c->peer[p]) return fail(ctx, NNQ_ERR_INVALID_ARG, "peer %d has not been opened", p);
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    // large, 16-byte granular messages: the multi-CTA form
    const size_t bytes = (size_t)count * es;
    const bool multi = bytes >= 32 * 1024 && bytes % 16 == 0 && !((uintptr_t)buf_dev & 15u) && c->slot_bytes % 16 == 0;
    const int64_t units = (int64_t)(bytes / 16);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(multi ? (unsigned)(units / 1024 < 64 ? (units / 1024 < 1 ? 1 : units / 1024) : 64) : 1u);
    cfg.blockDim = dim3(512);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may become resident early; waits inside
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    uint8_t *const *table = c->d_peer_table;
    int *status = ctx->d_status;
    int cnt = (int)count;
    cudaError_t e;
    if (dt == NNQ_F32) {
        float *b = (float *)buf_dev;
        e = multi ? cudaLaunchKernelEx(&cfg, allreduce_multi_kernel<float>, table, c->rank, c->world, c->slot_bytes, b, units, status)
                  : cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<float>, table, c->rank, c->world, c->slot_bytes, b, cnt, status);
    } else {
        __nv_bfloat16 *b = (__nv_bfloat16 *)buf_dev;
        e = multi ? cudaLaunchKernelEx(&cfg, allreduce_multi_kernel<__nv_bfloat16>, table, c->rank, c->world, c->slot_bytes, b, units, status)
                  : cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<__nv_bfloat16>, table, c->rank, c->world, c->slot_bytes, b, cnt, status);
    }
    ctx->launches++;
    return check_cuda(ctx, e, "all-reduce launch");
}

nnq_status nnq_comm_linear(nnq_comm *c, const nnq_weight *w, const void *x_dev, nnq_dtype x_dt, int64_t m,
                           const float *bias_dev, void *y_dev, nnq_dtype y_dt, void *stream) {
    if (!c || !w) return NNQ_ERR_INVALID_ARG;
    nnq_ctx *ctx = c->ctx;
    if (w->ctx != ctx) return fail(ctx, NNQ_ERR_INVALID_ARG, "weight belongs to another context");
    for (int p = 0; p < c->world; p++)
        if (!c->peer[p]) return fail(ctx, NNQ_ERR_INVALID_ARG, "peer %d has not been opened", p);
    if (m >= 1 && (size_t)m * (size_t)w->n * 4 > c->slot_bytes)
        return fail(ctx, NNQ_ERR_UNSUPPORTED, "output of %lld x %lld exceeds the communicator's %zu-byte slots",
                    (long long)m, (long long)w->n, c->slot_bytes);
    const bool slots_fit_pairs = (size_t)w->n * 8 <= c->slot_bytes;   // (value, sequence number) per row
    nnq_status s = check_cuda(ctx, cudaSetDevice(ctx->device), "cudaSetDevice");
    if (s != NNQ_OK) return s;
    if (m == 1 && slots_fit_pairs && ctx->path == NNQ_PATH_AUTO && skinny_fused_supported(w, m, x_dt)) {
        FusedReduce fr = {c->d_peer_table, c->slot_bytes, c->rank, c->world, 1};
        SkinnyJob job = {w, x_dev, bias_dev, y_dev};
        return launch_skinny_fused(ctx, job, x_dt, y_dt, fr, (cudaStream_t)stream);
    }
    // two steps: the product (bias on rank 0 only, so that the sum holds it once), then the exchange
    s = nnq_linear(ctx, w, x_dev, x_dt, m, c->rank == 0 ? bias_dev : nullptr, y_dev, y_dt, stream);
    if (s != NNQ_OK) return s;
    return nnq_comm_all_reduce(c, y_dev, y_dt, m * w->n, stream);
}

void nnq_comm_destroy(nnq_comm *c) {
    if (!c) return;
    cudaSetDevice(c->ctx->device);
    cudaDeviceSynchronize();
    for (int p = 0; p < c->world; p++)
        if (c->opened[p]) cudaIpcCloseMemHandle(c->peer[p]);
    cudaFree(c->d_local);
    cudaFree(c->d_peer_table);
    cudaGetLastError();
    delete c;
}

}  // extern "C"
