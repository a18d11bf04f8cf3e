// Layout of a communicator's peer-mapped buffer, shared by the all-reduce kernel and by the
// product kernel that pushes its partial outputs straight into the peers' slots.
//   [0, 64)     epoch: sequence number of the last completed exchange
//   [64, 128)   flags: u32 per source rank, the sequence number that rank has published
//   [128, 192)  arrival counters: u32 at 128 of the fused product kernel (CTAs that finished pushing),
//               at 132 / 136 of the multi-CTA all-reduce (CTAs that pushed / that finished)
//   [192, 196)  bound of every flag wait of kernels that use this communicator, in polls
//   [256, ...)  data[parity][source rank][slot_bytes]
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace nnq {

constexpr int kCommMaxWorld = 8;
constexpr unsigned kCommSpins = 1u << 22;   // default bound of every flag wait (nnq_comm_set_spin_limit changes it)
constexpr size_t kCommSpinLimitOffset = 192;

// the wait bound of the communicator whose buffer is `local`
__device__ __forceinline__ unsigned comm_spin_limit(const uint8_t *local) {
    return *reinterpret_cast<const volatile unsigned *>(local + kCommSpinLimitOffset);
}

__host__ __device__ inline size_t comm_data_offset(int parity, int src, int world, size_t slot_bytes) {
    return 256 + ((size_t)parity * world + src) * slot_bytes;
}

// What the fused product kernel needs to know about the exchange (enabled = 0: plain product).
struct FusedReduce {
    uint8_t *const *peers;   // device table of every rank's buffer (peers[rank] = own)
    size_t slot_bytes;
    int rank, world;
    int enabled;
};

// What a kernel outside comm.cu needs to know about an opened communicator.
struct CommView {
    uint8_t *const *peer_table;   // device table of every rank's buffer
    size_t slot_bytes;
    int rank, world;
};

}  // namespace nnq
