// Programmatic dependent launch for the small kernels around the quantized products.
#pragma once
#include <cuda_runtime.h>

namespace nnq {

// Every kernel of the step is launched with programmatic stream serialization and waits for its
// predecessor before touching any data, so that its launch overlaps the predecessor's tail. The
// small kernels do NOT release their successor early: a quantized product that became resident
// while they run would hold most of the registers of every SM and starve them (measured: slower).
__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace nnq
