// Helpers shared by every kernel file of the engine.  Each .cu file is built into a shared
// library of its own with plain C entry points (no torch headers): the Python side loads it with
// ctypes, passes device pointers and the current CUDA stream, and checks the returned code.
#pragma once
#include <cuda_bf16.h>
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

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch.  Every kernel of the engine is launched with the attribute that
// lets it start while the kernel before it in the stream is still running.  The rules each kernel
// keeps: it calls pdl_launch_dependents() at its start (the next kernel may begin its own set-up
// and prefetch data that no kernel writes, i.e. weights), and it calls pdl_wait() before it reads
// anything a preceding kernel wrote and before it writes anything at all.  pdl_wait() returns when
// the preceding kernel has completed and its writes are visible; since every kernel waits before
// it finishes, completion is transitive along the stream.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// early != 0: the kernel may start before the kernel ahead of it has finished (it must keep the
// rules above).  early == 0: an ordinary launch; the calls above are then no-ops.
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
static inline int tnx_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
    return tnx_launch_ex(0, kernel, grid, block, smem, stream, args...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

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
