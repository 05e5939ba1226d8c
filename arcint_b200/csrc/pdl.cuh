// pdl.cuh -- programmatic dependent launch for the decode chain (quantize -> GEMV -> quantize -> ...).
//
// A decode-width product is a few microseconds of kernel time, so the gap between two kernels in a
// stream (drain, launch, ramp) is a large part of a token. Launched with the programmatic-serialization
// attribute, a kernel may start while its predecessor is still running; it must not touch anything the
// predecessor produces before pdl_wait() (which returns once every prerequisite grid has completed and its
// writes are visible). The GEMV uses the head start to put its first weight stages in flight -- weights
// do not depend on the predecessor -- and the quantizer to get its blocks resident. pdl_trigger() lets the
// next kernel be scheduled: the small quantizers call it first thing, the GEMV when a block has finished its
// rows (triggered at its start, the blocks of later kernels would occupy the places of its own wave: measured
// 40 % slower). Both calls do nothing in a kernel
// launched the plain way. Stream capture keeps the edges, so CUDA graphs replay with them.
#pragma once

#include <cuda_runtime.h>

namespace b200q {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(bool pdl, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

}  // namespace b200q
