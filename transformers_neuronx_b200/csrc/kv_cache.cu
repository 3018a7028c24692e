// Writing this step's keys and values into the pages of a cache.
//
// A cache is one tensor [num_pages, 2 (key, value), n_kv_heads, page_size, head_dim]: for one
// head the page_size rows of a page are contiguous.  `slot_mapping[n]` = page * page_size + row
// for token n, made on the host from the request's block table.
#include <type_traits>

#include "common.cuh"

// One block per token; each thread moves 16-byte pieces (VEC elements) of the token's keys and values.
template <typename T, int VEC>
__global__ void kv_append_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src, int src_stride,
                                 const int* __restrict__ slot_mapping, T* __restrict__ cache,
                                 int n_kv_heads, int head_dim, int page_size) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x;
    const int slot = slot_mapping[n];
    if (slot < 0) return;                       // a padded row of a captured batch
    const int page = slot / page_size, row = slot % page_size;
    const size_t head_block = (size_t)page_size * head_dim;
    const int pieces_per_head = head_dim / VEC;
    const int pieces = n_kv_heads * pieces_per_head;
    typedef typename std::conditional<VEC == 1, T, uint4>::type Piece;
    for (int i = threadIdx.x; i < 2 * pieces; i += blockDim.x) {
        const int kv = i / pieces, j = i % pieces;
        const int h = j / pieces_per_head, c = (j % pieces_per_head) * VEC;
        const T* src = (kv ? v_src : k_src) + (size_t)n * src_stride + (size_t)h * head_dim + c;
        T* dst = cache + (((size_t)page * 2 + kv) * n_kv_heads + h) * head_block + (size_t)row * head_dim + c;
        *(Piece*)dst = *(const Piece*)src;
    }
}

TNX_EXPORT int tnx_kv_append(const void* k_src, const void* v_src, int src_stride, const int* slot_mapping,
                             void* cache, int N, int n_kv_heads, int head_dim, int page_size,
                             int is_h16, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_kv_heads <= 0 || head_dim <= 0 || page_size <= 0) return TNX_ERR_BAD_ARG;
    const int esz = is_h16 ? 2 : 4, vec = 16 / esz;
    const bool wide = head_dim % vec == 0 && src_stride % vec == 0 && ((uintptr_t)k_src % 16) == 0 &&
                      ((uintptr_t)v_src % 16) == 0 && ((uintptr_t)cache % 16) == 0;
    const int work = 2 * n_kv_heads * head_dim / (wide ? vec : 1);
    const dim3 grid(N), block(work >= 256 ? 256 : (work >= 128 ? 128 : 64));
#define KV_LAUNCH(T, V)                                                                                          \
    tnx_launch_in_order(kv_append_kernel<T, V>, grid, block, 0, stream, (const T*)k_src, (const T*)v_src, src_stride, \
                   slot_mapping, (T*)cache, n_kv_heads, head_dim, page_size)
    if (is_h16) return wide ? KV_LAUNCH(h16, 8) : KV_LAUNCH(h16, 1);
    return wide ? KV_LAUNCH(float, 4) : KV_LAUNCH(float, 1);
#undef KV_LAUNCH
}

// Whole rows of a tensor copied within it: row dst[i] takes the bytes of row src[i] (pages of a cache,
// or slots of a state tensor, when a request goes on from what another one holds: beam search).  No
// row may be both a source and a destination.  pairs: [n_pairs][2] (source, destination).
__global__ void copy_rows_kernel(uint8_t* __restrict__ base, const int* __restrict__ pairs, long long row_bytes) {
    pdl_launch_dependents();
    pdl_wait();
    const int src = pairs[2 * blockIdx.x], dst = pairs[2 * blockIdx.x + 1];
    if (src < 0 || dst < 0 || src == dst) return;
    const uint8_t* s = base + (size_t)src * row_bytes;
    uint8_t* d = base + (size_t)dst * row_bytes;
    const long long chunk = (row_bytes + gridDim.y - 1) / gridDim.y;
    const long long lo = (long long)blockIdx.y * chunk, hi = lo + chunk < row_bytes ? lo + chunk : row_bytes;
    if ((((uintptr_t)s | (uintptr_t)d | (uintptr_t)chunk) & 15) == 0) {
        for (long long o = lo + 16LL * threadIdx.x; o + 16 <= hi; o += 16LL * blockDim.x) *(uint4*)(d + o) = *(const uint4*)(s + o);
        for (long long o = lo + ((hi - lo) & ~15LL) + threadIdx.x; o < hi; o += blockDim.x) d[o] = s[o];
    } else {
        for (long long o = lo + threadIdx.x; o < hi; o += blockDim.x) d[o] = s[o];
    }
}

TNX_EXPORT int tnx_copy_rows(void* base, const int* pairs, int n_pairs, long long row_bytes, cudaStream_t stream) {
    if (n_pairs <= 0 || row_bytes <= 0) return 0;
    if (!base || !pairs) return TNX_ERR_BAD_ARG;
    long long parts = (row_bytes + 16383) / 16384;                // 16 KB a block
    if (parts > 1024) parts = 1024;
    return tnx_launch_in_order(copy_rows_kernel, dim3(n_pairs, (unsigned)parts), dim3(256), 0, stream, (uint8_t*)base, pairs, row_bytes);
}

