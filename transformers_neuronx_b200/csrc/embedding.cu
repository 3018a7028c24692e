// Token embedding gather + learned position embedding.
//
//   x[n, :] = (tok_table ? tok_table[ids[n], :] : pre[n, :]) + (pos_table ? pos_table[positions[n] + offset, :] : 0)
//
// written as the 32-bit residual stream and, when asked, also in the activation type for a block
// that reads its input un-normalised.  `pre` is the 32-bit output of project_in when the embedding
// width differs from the hidden width.  gather_rows copies table rows in the activation type (the
// input of project_in).
#include "common.cuh"

template <typename TT, typename TA>
__global__ void embed_kernel(const TT* __restrict__ tok_table, const float* __restrict__ pre,
                             const int* __restrict__ ids, const TT* __restrict__ pos_table,
                             const int* __restrict__ positions, int pos_offset,
                             float* __restrict__ out_f32, TA* __restrict__ out_act, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    const TT* trow = tok_table ? tok_table + (size_t)ids[n] * H : nullptr;
    const TT* prow = pos_table ? pos_table + (size_t)(positions[n] + pos_offset) * H : nullptr;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = trow ? to_float(trow[c]) : pre[(size_t)n * H + c];
        if (prow) v += to_float(prow[c]);
        if (out_f32) out_f32[(size_t)n * H + c] = v;
        if (out_act) out_act[(size_t)n * H + c] = from_float<TA>(v);
    }
}

template <typename TT, typename TA>
__global__ void gather_rows_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                   TA* __restrict__ out, int E) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    const TT* row = table + (size_t)ids[n] * E;
    for (int c = threadIdx.x; c < E; c += blockDim.x) out[(size_t)n * E + c] = from_float<TA>(to_float(row[c]));
}

// tokens[i] = sampled[src[i]] where src[i] >= 0: a request's next input is the id that the sampling
// kernel left on the device in the step before, so the host need not wait for it.
__global__ void patch_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src,
                                    const int* __restrict__ sampled, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && src[i] >= 0) tokens[i] = sampled[src[i]];
}

TNX_EXPORT int tnx_patch_tokens(int* tokens, const int* src, const int* sampled, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    return tnx_launch_in_order(patch_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tokens, src, sampled, n);
}

// table_h16 / act_h16: 1 when the tables / the activation output are bfloat16, 0 for float.
TNX_EXPORT int tnx_embed(const void* tok_table, const float* pre, const int* ids, const void* pos_table,
                         const int* positions, int pos_offset, float* out_f32, void* out_act,
                         int N, int H, int table_h16, int act_h16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || (!tok_table && !pre)) return TNX_ERR_BAD_ARG;
    const int threads = H >= 1024 ? 256 : 128;
#define LAUNCH(TT, TA)                                                                                        \
    tnx_launch_in_order(embed_kernel<TT, TA>, dim3(N), dim3(threads), 0, stream, (const TT*)tok_table, pre, ids,   \
                   (const TT*)pos_table, positions, pos_offset, out_f32, (TA*)out_act, H)
    if (table_h16 && act_h16) return LAUNCH(h16, h16);
    if (table_h16 && !act_h16) return LAUNCH(h16, float);
    if (!table_h16 && act_h16) return LAUNCH(float, h16);
    return LAUNCH(float, float);
#undef LAUNCH
}

TNX_EXPORT int tnx_gather_rows(const void* table, const int* ids, void* out, int N, int E,
                               int table_h16, int act_h16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (E <= 0) return TNX_ERR_BAD_ARG;
    const int threads = E >= 1024 ? 256 : 128;
    if (table_h16 && act_h16) return tnx_launch_in_order(gather_rows_kernel<h16, h16>, dim3(N), dim3(threads), 0, stream, (const h16*)table, ids, (h16*)out, E);
    if (table_h16) return tnx_launch_in_order(gather_rows_kernel<h16, float>, dim3(N), dim3(threads), 0, stream, (const h16*)table, ids, (float*)out, E);
    if (act_h16) return tnx_launch_in_order(gather_rows_kernel<float, h16>, dim3(N), dim3(threads), 0, stream, (const float*)table, ids, (h16*)out, E);
    return tnx_launch_in_order(gather_rows_kernel<float, float>, dim3(N), dim3(threads), 0, stream, (const float*)table, ids, (float*)out, E);
}
