// Helpers shared by every kernel file of the engine.  Each .cu file is built into a shared
// library of its own with plain C entry points (no torch headers): the Python side loads it with
// ctypes, passes device pointers and the current CUDA stream, and checks the returned code.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TNX_EXPORT extern "C" __attribute__((visibility("default")))

// Entry points return 0 on success, a CUDA error code (>0) if a launch failed, or a negative
// code of their own for an argument they refuse.
#define TNX_ERR_BAD_ARG (-1)
#define TNX_ERR_UNSUPPORTED (-2)
#define TNX_ERR_TIMEOUT (-3)

static inline int tnx_launch_status() {
    cudaError_t e = cudaGetLastError();
    return (int)e;
}

// The 16-bit floating type of this build.  Every library is compiled once with bfloat16 as `h16` and,
// when a model asks for it, once more with TNX_F16 defined, where `h16` is IEEE half precision
// (float16): the same kernels, other conversions, other operand formats of the tensor-core instructions.
// An entry point's `*_h16` flags say "this tensor holds h16" (0: 32-bit floats).
#ifdef TNX_F16
typedef __half h16;
typedef __half2 h16x2;
#define TNX_H16_NAME "float16"
__device__ __forceinline__ float h16_to_float(h16 v) { return __half2float(v); }
__device__ __forceinline__ h16 float_to_h16(float v) { return __float2half_rn(v); }
__device__ __forceinline__ float2 h16x2_to_float2(h16x2 v) { return __half22float2(v); }
__device__ __forceinline__ h16x2 floats_to_h16x2(float a, float b) { return __floats2half2_rn(a, b); }
#else
typedef __nv_bfloat16 h16;
typedef __nv_bfloat162 h16x2;
#define TNX_H16_NAME "bfloat16"
__device__ __forceinline__ float h16_to_float(h16 v) { return __bfloat162float(v); }
__device__ __forceinline__ h16 float_to_h16(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float2 h16x2_to_float2(h16x2 v) { return __bfloat1622float2(v); }
__device__ __forceinline__ h16x2 floats_to_h16x2(float a, float b) { return __floats2bfloat162_rn(a, b); }
#endif
// 1 when this library was built with float16 as its 16-bit type, 0 for bfloat16.
TNX_EXPORT int tnx_h16_is_float16() {
#ifdef TNX_F16
    return 1;
#else
    return 0;
#endif
}

// Programmatic dependent launch.  The matrix products and LayerNorm are launched with the attribute that
// lets a kernel start while the kernel before it in the stream is still running (tnx_launch_ex with
// early = 1); the other kernels are launched in stream order (tnx_launch_in_order).  The rules every kernel
// keeps, so that either launch is right for it: it calls pdl_launch_dependents() at its start (the next kernel
// may begin its own set-up and prefetch data that no kernel writes, i.e. weights), and it calls pdl_wait()
// before it reads anything a preceding kernel wrote and before it writes anything at all.  pdl_wait() returns
// when the preceding kernel has completed and its writes are visible; since every kernel waits before
// it finishes, completion is transitive along the stream.  (In a kernel launched in stream order the wait
// returns at once; its call of pdl_launch_dependents() still lets a following kernel with the attribute in.)
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// early != 0: the kernel may start before the kernel ahead of it has finished (it must keep the
// rules above).  early == 0: an ordinary launch, after the kernel ahead of it.
template <typename... KArgs, typename... Args>
static inline int tnx_launch_ex(int early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = early ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return 0;
}
// The same with the thread blocks grouped into clusters of `cluster` (which must divide the grid).
template <typename... KArgs, typename... Args>
static inline int tnx_launch_cluster(int early, dim3 cluster, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x; attr[0].val.clusterDim.y = cluster.y; attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = early ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return 0;
}
template <typename... KArgs, typename... Args>
static inline int tnx_launch_in_order(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
    return tnx_launch_ex(0, kernel, grid, block, smem, stream, args...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(h16 v) { return h16_to_float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ h16 from_float<h16>(float v) { return float_to_h16(v); }

// Activations that a product's epilogue applies to (sum + bias), by code: the names of
// src/transformers_neuronx/activations.py (relu :43-48, gelu_new :17-41 with its tanh form, sigmoid
// :66-67, silu :70-72) plus the exact (erf) gelu.  The code travels to the kernel as a number, so
// another activation is one more case here and one more name in kernels/ops.py.
#define TNX_ACT_NONE 0
#define TNX_ACT_RELU 1
#define TNX_ACT_GELU_NEW 2
#define TNX_ACT_SILU 3
#define TNX_ACT_SIGMOID 4
#define TNX_ACT_GELU 5
#define TNX_ACT_COUNT 6
// The two cheap cases are inline; everything else is one call into a function that is compiled once.
// (With every case expanded inline, the epilogues of the tensor-core products, which apply the
// activation to several accumulators per loop turn, grew so much that a 2,048-token prefill of the
// 6.7B sizes took 32 ms instead of 26: also for the products that use no activation at all.)
__device__ __noinline__ float apply_activation_other(float v, int act) {
    switch (act) {
        case TNX_ACT_GELU_NEW: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case TNX_ACT_SILU: return v / (1.f + expf(-v));
        case TNX_ACT_SIGMOID: return 1.f / (1.f + expf(-v));
        case TNX_ACT_GELU: return 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
        default: return v;
    }
}
__device__ __forceinline__ float apply_activation(float v, int act) {
    if (act == TNX_ACT_NONE) return v;
    if (act == TNX_ACT_RELU) return fmaxf(v, 0.f);
    return apply_activation_other(v, act);
}

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

// Sum over a thread block; `scratch` holds at least 32 floats of shared memory.  Every thread
// receives the result.  The order of the additions is fixed by the block size alone.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}
