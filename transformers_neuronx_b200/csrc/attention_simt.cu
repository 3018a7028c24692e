// Attention over the paged cache on CUDA cores, scores and softmax in 32-bit: the true 32-bit
// path, and the path for head sizes that the tensor-core kernels refuse.
//
// One warp per (query token, head).  The query at position p of its request reads the keys at
// positions max(0, p - window + 1) .. p, all of which are in the cache when the kernel runs (this
// step's keys and values are written before it).  Keys are visited in ascending position, 32 at a
// time, with an online softmax; the result for a token therefore does not depend on how the
// request was cut into steps or on what else is in the batch.
//
//   s_j = scale * <q, k_j>;  out = sum_j exp(s_j - max) v_j / sum_j exp(s_j - max)
#include "common.cuh"

namespace {
constexpr int MAX_DIMS_PER_LANE = 8;   // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(128)
attention_simt_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ cache,
                      const int* __restrict__ block_tables, int bt_stride,
                      const int* __restrict__ token_request, const int* __restrict__ positions,
                      T* __restrict__ out, int out_stride, int n_tokens, int n_heads, int n_kv_heads,
                      int head_dim, int page_size, int window, float scale) {
    extern __shared__ float qsm[];                  // [warps per block][head_dim]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (pair >= (long long)n_tokens * n_heads) return;
    const int n = (int)(pair / n_heads), h = (int)(pair % n_heads);
    const int req = token_request[n];
    if (req < 0) return;                            // a padded row of a captured batch
    const int pos = positions[n];
    const int kvh = h / (n_heads / n_kv_heads);
    const int* bt = block_tables + (size_t)req * bt_stride;
    float* qs = qsm + warp * head_dim;
    const T* qrow = q + (size_t)n * q_stride + (size_t)h * head_dim;
    for (int c = lane; c < head_dim; c += 32) qs[c] = to_float(qrow[c]);
    __syncwarp();

    const size_t head_block = (size_t)page_size * head_dim;
    float m = -INFINITY, l = 0.f;
    float acc[MAX_DIMS_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) acc[i] = 0.f;
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    for (int c0 = first; c0 <= pos; c0 += 32) {
        const int j = c0 + lane;
        float s = -INFINITY;
        if (j <= pos) {
            const int page = bt[j / page_size];
            const T* krow = cache + (((size_t)page * 2 + 0) * n_kv_heads + kvh) * head_block +
                            (size_t)(j % page_size) * head_dim;
            float dot = 0.f;
            for (int c = 0; c < head_dim; ++c) dot = fmaf(qs[c], to_float(krow[c]), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = (j <= pos) ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) acc[i] *= corr;
        const int cnt = min(32, pos - c0 + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int jk = c0 + jj;
            const int page = bt[jk / page_size];
            const T* vrow = cache + (((size_t)page * 2 + 1) * n_kv_heads + kvh) * head_block +
                            (size_t)(jk % page_size) * head_dim;
#pragma unroll
            for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
                const int c = lane + 32 * i;
                if (c < head_dim) acc[i] = fmaf(pj, to_float(vrow[c]), acc[i]);
            }
        }
    }
    const float inv = 1.0f / l;
    T* orow = out + (size_t)n * out_stride + (size_t)h * head_dim;
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < head_dim) orow[c] = from_float<T>(acc[i] * inv);
    }
}
}  // namespace

TNX_EXPORT int tnx_attention_simt(const void* q, int q_stride, const void* cache, const int* block_tables,
                                  int bt_stride, const int* token_request, const int* positions, void* out,
                                  int out_stride, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                  int page_size, int window, float scale, int is_h16, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > 32 * MAX_DIMS_PER_LANE || n_kv_heads <= 0 || n_heads % n_kv_heads)
        return TNX_ERR_UNSUPPORTED;
    const int warps = 4;
    const long long pairs = (long long)n_tokens * n_heads;
    const int blocks = (int)((pairs + warps - 1) / warps);
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
    if (is_h16)
        return tnx_launch_in_order(attention_simt_kernel<h16>, dim3(blocks), dim3(warps * 32), smem, stream,
                              (const h16*)q, q_stride, (const h16*)cache, block_tables, bt_stride, token_request,
                              positions, (h16*)out, out_stride, n_tokens, n_heads, n_kv_heads, head_dim, page_size,
                              window, scale);
    return tnx_launch_in_order(attention_simt_kernel<float>, dim3(blocks), dim3(warps * 32), smem, stream,
                          (const float*)q, q_stride, (const float*)cache, block_tables, bt_stride, token_request,
                          positions, (float*)out, out_stride, n_tokens, n_heads, n_kv_heads, head_dim, page_size,
                          window, scale);
}
