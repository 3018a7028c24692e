// Causal attention of prompt portions over the paged bfloat16 cache (flash style: one pass over the
// keys with an online softmax, nothing of size tokens x tokens is stored).
//
// Work item = (request, tile of 128 of its query rows, head).  The queries of a portion sit at
// positions ctx_len .. ctx_len + q_len - 1 of their request and read the keys 0 .. their own
// position (or the last `window` of them) from the pages of the request's block table: the keys
// and values of this very portion were written to the pages before the kernel runs.
//
// Eight warps, 16 query rows each.  K and V tiles of 64 keys (four pages) are copied to shared
// memory with cp.async (16-byte chunks, XOR-swizzled rows) into two buffers, the next tile while
// the current one is used; S = Q K^T and O += P V run on tensor
// cores (mma.sync m16n8k16, h16 in, 32-bit accumulate); scores, softmax and the running sums are
// 32-bit.  HEAD is the head size rounded up to 64, 128 or 256; the columns beyond the real head
// size are zero in shared memory.
#include "common.cuh"

namespace {

constexpr int BQ = 128, BKV = 64, PAGE = 16, WARPS = 8;

struct PrefillParams {
    const h16* q; int q_stride;
    const h16* cache;
    const int* block_tables; int bt_stride;
    const int* tile_req;             // per work item: request index in the batch
    const int* tile_q0;              // per work item: first query row within the request's portion
    const int* q_start; const int* q_len; const int* ctx_len;
    h16* out; int out_stride;
    int n_heads, n_kv_heads, head_dim;
    int window;
    float scale_log2;                // scale * log2(e)
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_h16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
#ifdef TNX_F16
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
#else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
#endif
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_h16(float lo, float hi) {
    h16x2 h = floats_to_h16x2(lo, hi);
    return *(uint32_t*)&h;
}

// Byte offset of (row, 16-byte chunk) in a tile whose rows hold HEAD h16, chunks XOR-swizzled.
template <int HEAD>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * (HEAD * 2) + ((chunk ^ (row & 7)) << 4));
}

template <int HEAD>
__global__ void __launch_bounds__(WARPS * 32, HEAD <= 128 ? 2 : 1)
attention_prefill_kernel(const PrefillParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int KV_BYTES = BKV * HEAD * 2;
    uint8_t* sQ = smem;
    uint8_t* sKV = sQ + BQ * HEAD * 2;             // [2 buffers][K tile, V tile]
    pdl_launch_dependents();
    pdl_wait();

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Work items are listed in ascending position: the last have the most keys.  Heaviest first, so
    // that the short ones fill the tail.
    const int item = gridDim.y - 1 - blockIdx.y, h = blockIdx.x;      // heaviest tiles first, of all heads
    const int req = p.tile_req[item], q0 = p.tile_q0[item];
    if (req < 0) return;                                     // a padded work item of a captured step
    const int qs = p.q_start[req], ql = p.q_len[req], ctx = p.ctx_len[req];
    const int rows = min(BQ, ql - q0);                       // valid query rows of this tile
    const int d = p.head_dim;
    const int real_chunks = d / 8;
    const int kvh = h / (p.n_heads / p.n_kv_heads);
    const int* bt = p.block_tables + (size_t)req * p.bt_stride;
    const int pos0 = ctx + q0;                               // position of the tile's first query
    const int pos_last = pos0 + rows - 1;
    const int kv_total = ctx + ql;                           // keys of the request that exist

    // zero the padding columns (and everything else) once
    for (int i = tid; i < (BQ + 4 * BKV) * HEAD * 2 / 16; i += WARPS * 32) ((uint4*)smem)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    // Q tile
    for (int i = tid; i < BQ * real_chunks; i += WARPS * 32) {
        const int r = i / real_chunks, c = i % real_chunks;
        if (r < rows)
            cp_async16(sQ + swz<HEAD>(r, c), p.q + (size_t)(qs + q0 + r) * p.q_stride + (size_t)h * d + c * 8);
    }
    cp_async_commit();

    float o[HEAD / 8][4];
#pragma unroll
    for (int i = 0; i < HEAD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int r_lo = warp * 16 + (lane >> 2);                // this thread's two rows within the tile
    const int qpos_lo = pos0 + r_lo, qpos_hi = qpos_lo + 8;

    int key_begin = 0;
    if (p.window > 0) key_begin = max(0, pos0 - p.window + 1) / BKV * BKV;
    const size_t head_block = (size_t)PAGE * d;

    auto load_tile = [&](int k0, int buf) {
        uint8_t* sK = sKV + (size_t)buf * 2 * KV_BYTES;
        uint8_t* sV = sK + KV_BYTES;
        for (int i = tid; i < BKV * real_chunks; i += WARPS * 32) {
            const int r = i / real_chunks, c = i % real_chunks;
            const int key = k0 + r;
            if (key < kv_total) {
                const int page = bt[key / PAGE];
                if (page >= 0) {
                    const h16* kb = p.cache + (((size_t)page * 2 + 0) * p.n_kv_heads + kvh) * head_block +
                                     (size_t)(key % PAGE) * d + c * 8;
                    cp_async16(sK + swz<HEAD>(r, c), kb);
                    cp_async16(sV + swz<HEAD>(r, c), kb + (size_t)p.n_kv_heads * head_block);
                }
            }
        }
        cp_async_commit();
    };
    load_tile(key_begin, 0);
    int tile_no = 0;
    for (int k0 = key_begin; k0 <= pos_last; k0 += BKV, ++tile_no) {
        const int buf = tile_no & 1;
        const bool has_next = k0 + BKV <= pos_last;
        if (has_next) load_tile(k0 + BKV, buf ^ 1);          // its buffer was released by the barrier below
        if (has_next) cp_async_wait_one(); else cp_async_wait_all();
        __syncthreads();
        const uint8_t* sK = sKV + (size_t)buf * 2 * KV_BYTES;
        const uint8_t* sV = sK + KV_BYTES;

        // ---- S = Q K^T for this warp's 16 rows x 64 keys ----------------------------------------
        float s[BKV / 8][4];
#pragma unroll
        for (int i = 0; i < BKV / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < HEAD / 16; ++kk) {
            uint32_t a[4];
            {
                const int row = warp * 16 + (lane & 15), chunk = kk * 2 + (lane >> 4);
                ldmatrix_x4(a, smem_addr(sQ + swz<HEAD>(row, chunk)));
            }
#pragma unroll
            for (int nn = 0; nn < BKV / 16; ++nn) {
                uint32_t b[4];
                const int row = nn * 16 + (lane & 7) + ((lane >> 4) << 3), chunk = kk * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(b, smem_addr(sK + swz<HEAD>(row, chunk)));
                mma_h16(s[2 * nn], a, b[0], b[1]);
                mma_h16(s[2 * nn + 1], a, b[2], b[3]);
            }
        }
        // ---- mask, online softmax ------------------------------------------------------------------
        // The running maximum is kept on the raw scores (the scale is positive); one FMA folds the
        // scale and the maximum into the argument of ex2.  Only tiles that reach past the smallest
        // position of this warp's rows (or fall partly behind the window) need the mask.
        const int warp_pos_lo = pos0 + warp * 16, warp_pos_hi = warp_pos_lo + 15;
        bool need_mask = k0 + BKV - 1 > warp_pos_lo;
        if (p.window > 0) need_mask = need_mask || (k0 <= warp_pos_hi - p.window);
        if (need_mask) {
#pragma unroll
            for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = k0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int qp = (e < 2) ? qpos_lo : qpos_hi;
                    bool ok = key <= qp;
                    if (p.window > 0) ok = ok && key > qp - p.window;
                    if (!ok) s[nt][e] = -INFINITY;
                }
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < BKV / 8; ++nt) {
            mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
        }
        float corr[2], m_scaled[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            m_scaled[r] = (m_new == -INFINITY) ? 0.f : m_new * p.scale_log2;
            corr[r] = (m_run[r] == -INFINITY) ? 0.f : ex2_approx(m_run[r] * p.scale_log2 - m_scaled[r]);
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < HEAD / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = ex2_approx(fmaf(s[nt][e], p.scale_log2, -m_scaled[e >> 1]));   // ex2(-inf) = 0
                s[nt][e] = pv;
                rs[e >> 1] += pv;
            }
        }
        l_run[0] += rs[0];
        l_run[1] += rs[1];
        // ---- O += P V ---------------------------------------------------------------------------------
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_h16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_h16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_h16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_h16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int nn = 0; nn < HEAD / 16; ++nn) {
                uint32_t b[4];
                const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), chunk = nn * 2 + (lane >> 4);
                ldmatrix_x4_trans(b, smem_addr(sV + swz<HEAD>(row, chunk)));
                mma_h16(o[2 * nn], a, b[0], b[1]);
                mma_h16(o[2 * nn + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();                                     // every warp is done with this buffer
    }
    // ---- finish: rows' sums over the quad, normalise, store ------------------------------------------
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
    for (int nt = 0; nt < HEAD / 8; ++nt) {
        const int col = nt * 8 + (lane & 3) * 2;
        if (col < d) {
            if (r_lo < rows)
                *(uint32_t*)(p.out + (size_t)(qs + q0 + r_lo) * p.out_stride + (size_t)h * d + col) =
                    pack_h16(o[nt][0] * inv0, o[nt][1] * inv0);
            if (r_lo + 8 < rows)
                *(uint32_t*)(p.out + (size_t)(qs + q0 + r_lo + 8) * p.out_stride + (size_t)h * d + col) =
                    pack_h16(o[nt][2] * inv1, o[nt][3] * inv1);
        }
    }
}

template <int HEAD>
int launch(const PrefillParams& p, int n_items, cudaStream_t stream) {
    constexpr int smem = (BQ + 4 * BKV) * HEAD * 2;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HEAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(p.n_heads, n_items);        // heads vary fastest: CTAs start in the order of the work items
    return tnx_launch_in_order(attention_prefill_kernel<HEAD>, grid, dim3(WARPS * 32), smem, stream, p);
}

}  // namespace

TNX_EXPORT int tnx_attention_prefill(const void* q, int q_stride, const void* cache, const int* block_tables,
                                     int bt_stride, const int* tile_req, const int* tile_q0, const int* q_start,
                                     const int* q_len, const int* ctx_len, void* out, int out_stride, int n_items,
                                     int n_heads, int n_kv_heads, int head_dim, int page_size, int window,
                                     float scale, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (page_size != PAGE || head_dim % 16 || head_dim < 16 || head_dim > 256 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads || q_stride % 8 || out_stride % 2 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15) ||
        ((uintptr_t)out & 3))
        return TNX_ERR_UNSUPPORTED;
    PrefillParams p;
    p.q = (const h16*)q; p.q_stride = q_stride; p.cache = (const h16*)cache; p.block_tables = block_tables;
    p.bt_stride = bt_stride; p.tile_req = tile_req; p.tile_q0 = tile_q0; p.q_start = q_start; p.q_len = q_len;
    p.ctx_len = ctx_len; p.out = (h16*)out; p.out_stride = out_stride; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads;
    p.head_dim = head_dim; p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
    if (head_dim <= 64) return launch<64>(p, n_items, stream);
    if (head_dim <= 128) return launch<128>(p, n_items, stream);
    return launch<256>(p, n_items, stream);
}
