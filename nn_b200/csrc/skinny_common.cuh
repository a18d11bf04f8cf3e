// Constants and launch parameter blocks shared by the skinny (decode) kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "decode.cuh"
#include "skinny.h"
#include "sync.cuh"

namespace nnq {

constexpr int kTileBytes = 2304;
constexpr int kWarps = 8;          // compute warps per CTA; they split K of one row tile
constexpr int kMaxStages = 4;      // bulk-copy ring depth per warp (tiles in flight)
constexpr int kSmemMax = 227 * 1024;         // one CTA per SM
constexpr int kMoeMaxExperts = 64;

struct SkinnyJobDev {
    const uint8_t *tiled;
    const float *bias;
    void *y;
    int n;              // real rows
    int row_tiles;      // ceil(n / 16)
    int tile_begin;     // first row tile of this job in the launch-wide numbering
};

struct SkinnyParams {
    SkinnyJobDev job[kSkinnyMaxJobs];
    const void *x;      // activations shared by all jobs, [K]
    int njobs;
    int m;              // tokens (1 for the M = 1 kernel, 2..16 for the token-column kernel)
    int y_dt;
    int kblocks;        // tiles along K (K / 256; K / 192 for six-block MXFP4 tiles)
    int total_tiles;    // row tiles of all jobs
    int stages;         // ring depth per warp
    int diag;           // builds with -DNNQ_DIAG only: bit 0 = skip the arithmetic (stream only),
                        // bit 1 = do not wait for the previous kernel; 4 = plain streaming read
    int l2_prefetch;    // 1 = ask L2 for the warp's whole weight stream at kernel start
    int *status;
    FusedReduce fr;     // row-parallel product + all-reduce in one kernel (M = 1 kernel, one job)
};

}  // namespace nnq
