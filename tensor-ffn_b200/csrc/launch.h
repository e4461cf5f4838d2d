// Kernel launch helper: optional programmatic-dependent-launch attribute. A kernel launched with it
// may start before the previous kernel of the stream has finished, so it must execute
// griddepcontrol.wait (pdl_wait) before it touches anything an earlier kernel wrote.
#pragma once
#include <cuda_runtime.h>

namespace tffn {

template <typename Kern, typename... Args>
inline cudaError_t launch_k(Kern k, dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = cudaLaunchConfig_t{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, k, args...);
}

}  // namespace tffn
