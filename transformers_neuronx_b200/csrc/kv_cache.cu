// Writing this step's keys and values into the pages of a cache.
//
// A cache is one tensor [num_pages, 2 (key, value), n_kv_heads, page_size, head_dim]: for one
// head the page_size rows of a page are contiguous.  `slot_mapping[n]` = page * page_size + row
// for token n, made on the host from the request's block table.
#include "common.cuh"

template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src, int src_stride,
                                 const int* __restrict__ slot_mapping, T* __restrict__ cache,
                                 int n_kv_heads, int head_dim, int page_size) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x, h = blockIdx.y;
    const int slot = slot_mapping[n];
    if (slot < 0) return;                       // a padded row of a captured batch
    const int page = slot / page_size, row = slot % page_size;
    const size_t head_block = (size_t)page_size * head_dim;
    T* kdst = cache + (((size_t)page * 2 + 0) * n_kv_heads + h) * head_block + (size_t)row * head_dim;
    T* vdst = cache + (((size_t)page * 2 + 1) * n_kv_heads + h) * head_block + (size_t)row * head_dim;
    const T* ks = k_src + (size_t)n * src_stride + (size_t)h * head_dim;
    const T* vs = v_src + (size_t)n * src_stride + (size_t)h * head_dim;
    for (int c = threadIdx.x; c < head_dim; c += blockDim.x) {
        kdst[c] = ks[c];
        vdst[c] = vs[c];
    }
}

TNX_EXPORT int tnx_kv_append(const void* k_src, const void* v_src, int src_stride, const int* slot_mapping,
                             void* cache, int N, int n_kv_heads, int head_dim, int page_size,
                             int is_bf16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_kv_heads <= 0 || head_dim <= 0 || page_size <= 0) return TNX_ERR_BAD_ARG;
    dim3 grid(N, n_kv_heads);
    const int threads = head_dim >= 128 ? 128 : (head_dim >= 64 ? 64 : 32);
    if (is_bf16)
        return tnx_launch_pdl(kv_append_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)k_src, (const bf16*)v_src,
                              src_stride, slot_mapping, (bf16*)cache, n_kv_heads, head_dim, page_size);
    return tnx_launch_pdl(kv_append_kernel<float>, grid, dim3(threads), 0, stream, (const float*)k_src, (const float*)v_src,
                          src_stride, slot_mapping, (float*)cache, n_kv_heads, head_dim, page_size);
}
