// Programmatic dependent launch and the warp-level MMA shared by the packed-weight-stream kernels
// (forward: lq_fused.cu, backward: lq_bwd_small.cu).
//
// A site of the <= 16-token regime is two short launches (weight kernel, finalize) whose launch
// latency is comparable to their run time; both kernels therefore let their successor in the stream
// start launching at once (`launch_dependents`) and wait for their predecessor's completion and
// memory flush (`wait`) before touching any global memory.  Launched without the attribute (or after
// a kernel that never triggers) both are no-ops.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <utility>

#include <cuda_runtime.h>

#include "lq_internal.cuh"

namespace lqstream {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("LQ_NO_PDL");
        return !(e && e[0] == '1');
    }();
    return on;
}

// <<<grid, block, smem, st>>> with the programmatic-stream-serialization attribute.
template <typename... KArgs, typename... Args>
void launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    LQ_CUDA(cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...));
}

// D[16 x 8] += A[16 x 16] . B[16 x 8], bf16 operands, f32 accumulators
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

}  // namespace lqstream
