// lm_device.cuh - device helpers and the launch helper shared by the language-model kernels (lm_kernels.cu,
// lm_mixers.cu).  Everything here has internal linkage.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

namespace lm {
namespace {

__device__ __forceinline__ float bf(const __nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float dyt(float x, float alpha, float w, float b) { return fmaf(tanhf(alpha * x), w, b); }

// Programmatic dependent launch: a kernel of a short step lets the next one start as soon as it runs itself
// (pdl_release) and reads what earlier kernels wrote - or writes anything - only after pdl_wait.  Before the wait a
// kernel may fetch weights, which no kernel writes.  Launched without the attribute both are no-ops.
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// fixed-tree block reductions (red: one float per warp); every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; ++i) t += red[i];
    return t;
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float siluf_(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// activation of a gated unit on its gate g and up u products.  kGluSilu: silu(g) u.  kGluClamped: both are clamped first
// (g from above, u on both sides), the gate's sigmoid is 1.702 times steeper and the up branch is offset by one:
// g' sigmoid(1.702 g') (u' + 1)
constexpr int kGluSilu = 0, kGluClamped = 1;
__device__ __forceinline__ float glu_act(int kind, float g, float u, float limit) {
    if (kind == kGluClamped) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g * sigmoidf_(1.702f * g) * (u + 1.0f);
    }
    return siluf_(g) * u;
}

// the kernels of a short step are launched with programmatic stream serialization (see pdl_release / pdl_wait)
// early == false: a plain launch, which starts when its predecessor has ended.  For a kernel of few, long-running CTAs
// behind a kernel of thousands of short ones (a recurrence scan behind its per-row preparation) that is the faster
// order: CTAs that arrive while the predecessor drains are placed wherever a slot frees first, several to an SM, and
// stay there for the whole scan.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl_if(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = early ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    return launch_pdl_if(true, kernel, grid, block, smem, st, args...);
}

}  // namespace
}  // namespace lm
