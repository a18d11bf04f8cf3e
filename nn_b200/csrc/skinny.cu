#include "skinny.h"
namespace nnq {
nnq_status skinny_init(nnq_ctx *) { return NNQ_OK; }
nnq_status build_tiled(nnq_ctx *, nnq_weight *) { return NNQ_OK; }
bool skinny_supported(const nnq_weight *, int64_t) { return false; }
nnq_status launch_skinny(nnq_ctx *ctx, const SkinnyJob *, int, int, int64_t, int, cudaStream_t) {
    return fail(ctx, NNQ_ERR_UNSUPPORTED, "skinny kernels not built");
}
}  // namespace nnq
