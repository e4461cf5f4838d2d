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

// Ask for the largest shared-memory carveout for a kernel, whatever it uses itself. The kernels of a
// decode step are resident together (dependent launches let the next ones start early and fetch their
// weights). An SM cannot change its L1 / shared-memory split while CTAs are resident on it: if the small
// kernels ran with a small carveout, a CTA that needs 200 KB of shared memory could only start once the
// SM had drained, i.e. without its head start. With one common carveout they co-reside.
template <typename Kern>
inline cudaError_t prefer_max_shared(Kern k) {
    return cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}

}  // namespace tffn
