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
                              int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || (size_t)H * sizeof(float) > 200 * 1024) return TNX_ERR_UNSUPPORTED;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const size_t smem = (size_t)H * sizeof(float);
    if (act_bf16) {
        if (smem + 1024 > 48 * 1024) cudaFuncSetAttribute(layer_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tnx_launch_pdl(layer_norm_kernel<bf16>, dim3(n_rows), dim3(threads), smem, stream, x, rows, gamma, beta, eps, out_f32, (bf16*)out_act, H);
    } else {
        if (smem + 1024 > 48 * 1024) cudaFuncSetAttribute(layer_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tnx_launch_pdl(layer_norm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, rows, gamma, beta, eps, out_f32, (float*)out_act, H);
    }
}

TNX_EXPORT int tnx_pick_rows(const float* x, const int* rows, float* out_f32, void* out_act,
                             int n_rows, int H, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (act_bf16) return tnx_launch_pdl(pick_rows_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, rows, out_f32, (bf16*)out_act, H);
    return tnx_launch_pdl(pick_rows_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, rows, out_f32, (float*)out_act, H);
}
