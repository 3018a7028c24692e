// LayerNorm over the hidden axis, statistics in 32-bit from the 32-bit residual stream:
//   y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * gamma + beta
// One thread block per row; the row is held in shared memory between the two passes, so the
// variance is that of the formula (two passes), not E[x^2] - mean^2.
// Outputs: the activation type for the next matrix product, and/or 32-bit (the residual stream of
// a post-norm block).  `rows`, when given, picks the input rows (the rows whose logits are wanted).
#include "common.cuh"

template <typename TA>
__global__ void layer_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                  const float* __restrict__ gamma, const float* __restrict__ beta,
                                  float eps, float* __restrict__ out_f32, TA* __restrict__ out_act, int H) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[r] : r) * H;
    float s = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = src[c];
        row[c] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)H;
    float q = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float d = row[c] - mean;
        q += d * d;
    }
    const float var = block_sum(q, scratch) / (float)H;
    const float rstd = 1.0f / sqrtf(var + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float y = (row[c] - mean) * rstd;
        if (gamma) y *= gamma[c];
        if (beta) y += beta[c];
        if (out_f32) out_f32[(size_t)r * H + c] = y;
        if (out_act) out_act[(size_t)r * H + c] = from_float<TA>(y);
    }
}

// The same with the row held in registers: four consecutive elements per load, NV loads per
// thread (H == 4 * NV * threads exactly is not required: pieces beyond the row are skipped; NV = 5
// is there for rows of 5,120, which 8 loads per thread served a seventh slower).
// Launched so that it may start while the kernel ahead still runs: it waits for that kernel's
// results before its first load (measured: 1 % of a decode step).
template <typename TA, int NV, bool EARLY>
__global__ void layer_norm_reg_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                      const float* __restrict__ gamma, const float* __restrict__ beta,
                                      float eps, float* __restrict__ out_f32, TA* __restrict__ out_act, int H) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int n4 = H / 4;
    // The scale and the shift are weights: no kernel writes them.  EARLY (few rows, where the kernel is a chain of
    // round trips): they are fetched before the wait for the preceding kernel and are not a second round trip to
    // the second-level cache behind the statistics.  With many rows they are read where they are used, which
    // keeps the registers few and the blocks an SM many.
    float4 g[EARLY ? NV : 1], b[EARLY ? NV : 1];
    if (EARLY) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            g[i] = (gamma && c < n4) ? __ldg((const float4*)gamma + c) : make_float4(1.f, 1.f, 1.f, 1.f);
            b[i] = (beta && c < n4) ? __ldg((const float4*)beta + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    pdl_wait();
    const float4* src = (const float4*)(x + (size_t)(rows ? rows[r] : r) * H);
    float4 v[NV];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        v[i] = c < n4 ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = block_sum(s, scratch) / (float)H;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n4) {
            const float a = v[i].x - mean, b = v[i].y - mean, cc = v[i].z - mean, d = v[i].w - mean;
            q += (a * a + b * b) + (cc * cc + d * d);
        }
    }
    const float var = block_sum(q, scratch) / (float)H;
    const float rstd = 1.0f / sqrtf(var + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c >= n4) continue;
        float4 y = make_float4((v[i].x - mean) * rstd, (v[i].y - mean) * rstd, (v[i].z - mean) * rstd, (v[i].w - mean) * rstd);
        if (EARLY) {
            if (gamma) { y.x *= g[i].x; y.y *= g[i].y; y.z *= g[i].z; y.w *= g[i].w; }
            if (beta) { y.x += b[i].x; y.y += b[i].y; y.z += b[i].z; y.w += b[i].w; }
        } else {
            if (gamma) { const float4 gg = ((const float4*)gamma)[c]; y.x *= gg.x; y.y *= gg.y; y.z *= gg.z; y.w *= gg.w; }
            if (beta) { const float4 bb = ((const float4*)beta)[c]; y.x += bb.x; y.y += bb.y; y.z += bb.z; y.w += bb.w; }
        }
        if (out_f32) ((float4*)(out_f32 + (size_t)r * H))[c] = y;
        if (out_act) {
            TA* dst = out_act + (size_t)r * H + 4 * c;
            if constexpr (sizeof(TA) == 2) {
                h16x2 lo = floats_to_h16x2(y.x, y.y), hi = floats_to_h16x2(y.z, y.w);
                uint2 u;
                u.x = *(uint32_t*)&lo; u.y = *(uint32_t*)&hi;
                *(uint2*)dst = u;
            } else {
                *(float4*)dst = y;
            }
        }
    }
}

// Copies (and converts) picked rows without normalising: the head of a model with no final norm.
template <typename TA>
__global__ void pick_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                 float* __restrict__ out_f32, TA* __restrict__ out_act, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[r] : r) * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = src[c];
        if (out_f32) out_f32[(size_t)r * H + c] = v;
        if (out_act) out_act[(size_t)r * H + c] = from_float<TA>(v);
    }
}

TNX_EXPORT int tnx_layer_norm(const float* x, const int* rows, const float* gamma, const float* beta,
                              float eps, float* out_f32, void* out_act, int n_rows, int H,
                              int act_h16, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || (size_t)H * sizeof(float) > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    // Rows of a multiple of four elements, 16-byte aligned, up to 8,192 elements: the register kernel.
    const bool aligned = H % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)gamma % 16) == 0 &&
                         ((uintptr_t)beta % 16) == 0 && ((uintptr_t)out_f32 % 16) == 0 && ((uintptr_t)out_act % 16) == 0;
    if (aligned && H <= 8192) {
        const int n4 = H / 4;
        const int threads = n4 >= 1024 ? 256 : (n4 >= 256 ? 128 : 64);
        const int nv = (n4 + threads - 1) / threads;
        const bool early = n_rows <= 256;
#define LN_LAUNCH(TA, NV)                                                                                      \
    (early ? tnx_launch_ex(1, layer_norm_reg_kernel<TA, NV, true>, dim3(n_rows), dim3(threads), 0, stream, x, rows, gamma, beta, \
                           eps, out_f32, (TA*)out_act, H)                                                       \
           : tnx_launch_ex(1, layer_norm_reg_kernel<TA, NV, false>, dim3(n_rows), dim3(threads), 0, stream, x, rows, gamma, beta, \
                           eps, out_f32, (TA*)out_act, H))
#define LN_PICK(TA)                                                                        \
    (nv <= 1 ? LN_LAUNCH(TA, 1) : nv <= 2 ? LN_LAUNCH(TA, 2) : nv <= 4 ? LN_LAUNCH(TA, 4) : nv <= 5 ? LN_LAUNCH(TA, 5) : LN_LAUNCH(TA, 8))
        if (act_h16) return LN_PICK(h16);
        return LN_PICK(float);
#undef LN_PICK
#undef LN_LAUNCH
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const size_t smem = (size_t)H * sizeof(float);
    if (act_h16) {
        if (smem + 1024 > 48 * 1024) cudaFuncSetAttribute(layer_norm_kernel<h16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tnx_launch_in_order(layer_norm_kernel<h16>, dim3(n_rows), dim3(threads), smem, stream, x, rows, gamma, beta, eps, out_f32, (h16*)out_act, H);
    } else {
        if (smem + 1024 > 48 * 1024) cudaFuncSetAttribute(layer_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tnx_launch_in_order(layer_norm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, rows, gamma, beta, eps, out_f32, (float*)out_act, H);
    }
}

TNX_EXPORT int tnx_pick_rows(const float* x, const int* rows, float* out_f32, void* out_act,
                             int n_rows, int H, int act_h16, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (act_h16) return tnx_launch_in_order(pick_rows_kernel<h16>, dim3(n_rows), dim3(threads), 0, stream, x, rows, out_f32, (h16*)out_act, H);
    return tnx_launch_in_order(pick_rows_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, rows, out_f32, (float*)out_act, H);
}
