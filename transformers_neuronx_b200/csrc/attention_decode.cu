// Decode attention over the paged bfloat16 cache: one query token per request, the keys and values
// of its request streamed from the pages named by its block table.  Memory-bound: every key and
// value of the live requests is read once per layer and step.
//
//   s_j = scale * <q, k_j>  (32-bit),  out = sum_j exp(s_j - max) v_j / sum_j exp(s_j - max)
//
// Grid (heads, rows, splits): a CTA takes one (row, head) and one contiguous range of pages; its
// four, eight or sixteen warps take pages of the range in turn and keep an online softmax each (half a page at a
// time, the next half's loads in flight meanwhile).  A lane owns eight
// consecutive dims of the head (one 16-byte load per key) of some of the keys of a page, so a page
// of 16 keys x head_dim is read with fully used 16-byte loads.  The warps' states are merged in
// shared memory.  With more than one split the CTA writes its (max, sum, accumulator) to scratch
// memory, and the CTA of a (row, head) that finishes last merges the splits in split order.
//
// The kernel can also do the cache append of a decode step: given the new keys and values of the
// rows' tokens, the CTA whose range of pages holds a token's own position copies that token's key
// and value (of its key/value head) into the page for later steps, and takes them into its own
// softmax straight from where the projection left them; the pages are read for the earlier keys
// only.  The append kernel and its launch are then not needed.
#include "common.cuh"

namespace {

constexpr int PAGE = 16;

struct DecodeParams {
    const h16* q; int q_stride;
    const h16* cache;
    const int* block_tables; int bt_stride;
    const int* rows;                 // rows of the batch that are decode tokens (null: all rows)
    const int* token_request;
    const int* positions;
    h16* out; int out_stride;
    int n_heads, n_kv_heads, head_dim;
    int window;
    float scale;
    int n_splits, pages_per_split;
    float* scratch;                  // [rows][heads][splits][head_dim + 2]
    int* counters;                   // [rows][heads], zero between calls
    const h16* k_new;               // [rows, kv_heads * head_dim] keys of the rows' own tokens, or null:
    const h16* v_new;               //   then the cache already holds them
    int kv_stride;
    h16* cache_w;
};

// LPK lanes share one key; each of them owns E pieces of 8 dims of the head (piece e * LPK + its place
// among the LPK lanes, so that one warp-wide 16-byte load reads LPK * 16 consecutive bytes of every
// key).  KPL = 32 / LPK keys are read per warp-wide load.  E = 1 serves the head sizes whose number of
// 8-dim pieces is a power of two (and, with idle lanes, any other); E = 3 gives head sizes like 96
// (4 x 3 pieces) a layout without idle lanes.
template <int LPK, int E, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const DecodeParams p) {
    constexpr int KPL = 32 / LPK;
    constexpr int GROUPS = PAGE / KPL;         // key groups (of KPL keys) per page
    constexpr int LOADS = GROUPS * E;          // warp-wide loads per page and tensor (LPK = 32: 16, LPK = 2, E = 1: 1)
    __shared__ float sm_m[WARPS], sm_l[WARPS];
    __shared__ float sm_acc[WARPS][LPK * E * 8];
    __shared__ int last_flag;
    pdl_launch_dependents();
    pdl_wait();

    const int h = blockIdx.x, ri = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The loads a block needs before its first page are a chain (row -> request -> block table -> page);
    // what does not depend on the link before it is asked for at once.
    const int row = p.rows ? p.rows[ri] : ri;
    if (row < 0) return;                                        // a padded entry of the row list of a captured step
    const int req = p.token_request[row];
    const int pos = p.positions[row];
    const int d = p.head_dim;
    const int sub = lane % LPK;                                  // which 8 dims (of each of its E pieces)
    const int kgrp = lane / LPK;                                 // which key of a load
    const bool dim_ok = E > 1 || sub * 8 < d;                    // with E > 1 the head size is exactly LPK * E * 8
    uint4 q_raw[E];
#pragma unroll
    for (int e = 0; e < E; ++e)
        q_raw[e] = dim_ok ? *(const uint4*)(p.q + (size_t)row * p.q_stride + (size_t)h * d + (e * LPK + sub) * 8) : make_uint4(0, 0, 0, 0);
    if (req < 0) return;                                        // a padded row of a captured batch
    const int kv_len = pos + 1;
    const int first_key = (p.window > 0 && kv_len > p.window) ? kv_len - p.window : 0;
    const int kvh = h / (p.n_heads / p.n_kv_heads);
    const int* bt = p.block_tables + (size_t)req * p.bt_stride;

    float q[E][8];
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const h16x2* qq = (const h16x2*)&q_raw[e];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = h16x2_to_float2(qq[i]);
            q[e][2 * i] = f.x * p.scale; q[e][2 * i + 1] = f.y * p.scale;
        }
    }
    float m = -INFINITY, l = 0.f, acc[E][8];
#pragma unroll
    for (int e = 0; e < E; ++e)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[e][i] = 0.f;

    const int n_pages = (kv_len + PAGE - 1) / PAGE;
    const int page_lo = max(split * p.pages_per_split, first_key / PAGE);
    const int page_hi = min(n_pages, (split + 1) * p.pages_per_split);
    const size_t head_block = (size_t)PAGE * d;

    // With the append fused in, the cache holds the keys before this token's own; its own key and
    // value come from k_new / v_new.
    const bool own_here = p.k_new != nullptr && (pos / PAGE) / p.pages_per_split == split;    // one answer for the CTA
    const int cached_len = p.k_new != nullptr ? pos : kv_len;
    // The warp's pages (page_lo + warp, + WARPS, ...) are taken in chunks of CG key groups, i.e. CH = CG * E
    // warp-wide loads of keys and as many of values: half a page of the widest heads, a whole page
    // up to head size 64, one key group where a lane owns several pieces.  The loads of the next
    // chunk are issued before the current one is used, so that the warp always has loads in flight
    // (the same number of bytes whatever the head size); each chunk does its own step of the online softmax.
    constexpr int CG = E > 1 ? 1 : (GROUPS >= 8 ? GROUPS / 2 : GROUPS);   // key groups per chunk
    constexpr int CH = CG * E;                                // loads per chunk
    constexpr int CPP = GROUPS / CG;                          // chunks per page
    const int my_pages = page_hi > page_lo + warp ? (page_hi - page_lo - warp + WARPS - 1) / WARPS : 0;
    const int n_chunks = my_pages * CPP;
    auto issue = [&](int t, uint4 (&kb)[CH], uint4 (&vb)[CH]) {
        const int pg = page_lo + warp + (t / CPP) * WARPS;
        const int page = bt[pg];
        const h16* kbase = p.cache + (((size_t)page * 2 + 0) * p.n_kv_heads + kvh) * head_block;
        const h16* vbase = p.cache + (((size_t)page * 2 + 1) * p.n_kv_heads + kvh) * head_block;
        const int g0 = (t % CPP) * CG;
#pragma unroll
        for (int g = 0; g < CG; ++g)
#pragma unroll
            for (int e = 0; e < E; ++e) {
                const int key = (g0 + g) * KPL + kgrp;
                kb[g * E + e] = dim_ok ? __ldg((const uint4*)(kbase + (size_t)key * d + (e * LPK + sub) * 8)) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
        for (int g = 0; g < CG; ++g)
#pragma unroll
            for (int e = 0; e < E; ++e) {
                const int key = (g0 + g) * KPL + kgrp;
                vb[g * E + e] = dim_ok ? __ldg((const uint4*)(vbase + (size_t)key * d + (e * LPK + sub) * 8)) : make_uint4(0, 0, 0, 0);
            }
    };
    auto consume = [&](int t, uint4 (&kb)[CH], uint4 (&vb)[CH]) {
        const int pg = page_lo + warp + (t / CPP) * WARPS;
        const int g0 = (t % CPP) * CG;
        float s[CG];
        float chunk_max = -INFINITY;
#pragma unroll
        for (int g = 0; g < CG; ++g) {
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < E; ++e) {                        // one chain of multiply-adds per piece, not one for all
                const h16x2* kk = (const h16x2*)&kb[g * E + e];
                float de = 0.f;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 f = h16x2_to_float2(kk[u]);
                    de = fmaf(q[e][2 * u], f.x, de);
                    de = fmaf(q[e][2 * u + 1], f.y, de);
                }
                dot += de;
            }
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            const int j = pg * PAGE + (g0 + g) * KPL + kgrp;
            s[g] = (j >= first_key && j < cached_len) ? dot : -INFINITY;
            chunk_max = fmaxf(chunk_max, s[g]);
        }
#pragma unroll
        for (int o = 16; o >= LPK; o >>= 1) chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, o));
        if (chunk_max == -INFINITY) return;                      // every key of the chunk masked (warp-uniform)
        const float m_new = fmaxf(m, chunk_max);
        const float corr = (m == -INFINITY) ? 0.f : __expf(m - m_new);
        l *= corr;
#pragma unroll
        for (int e = 0; e < E; ++e)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[e][i] *= corr;
        m = m_new;
#pragma unroll
        for (int g = 0; g < CG; ++g) {
            const bool live = s[g] != -INFINITY;
            const float pj = live ? __expf(s[g] - m) : 0.f;
            l += pj;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                if (!live) vb[g * E + e] = make_uint4(0, 0, 0, 0);   // rows never written may hold anything, NaN included
                const h16x2* vv = (const h16x2*)&vb[g * E + e];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 f = h16x2_to_float2(vv[u]);
                    acc[e][2 * u] = fmaf(pj, f.x, acc[e][2 * u]);
                    acc[e][2 * u + 1] = fmaf(pj, f.y, acc[e][2 * u + 1]);
                }
            }
        }
    };
    {
        uint4 k0[CH], v0[CH], k1[CH], v1[CH];
        if (n_chunks > 0) issue(0, k0, v0);
        for (int t = 0; t < n_chunks; t += 2) {
            if (t + 1 < n_chunks) issue(t + 1, k1, v1);
            consume(t, k0, v0);
            if (t + 2 < n_chunks) issue(t + 2, k0, v0);
            if (t + 1 < n_chunks) consume(t + 1, k1, v1);
        }
    }
    if (own_here) {
        // The token's own key and value go into their page for later steps (CTAs of heads that share a
        // key/value head write the same bytes).  This comes after the pages have been streamed, so that
        // its loads do not stand between the block's start and its first page.
        const int page = bt[pos / PAGE];
        const int pieces = d / 8;
        for (int i = threadIdx.x; i < 2 * pieces; i += WARPS * 32) {
            const int which = i / pieces, piece = i - which * pieces;
            const h16* src = (which ? p.v_new : p.k_new) + (size_t)row * p.kv_stride + (size_t)kvh * d;
            h16* dst = p.cache_w + (((size_t)page * 2 + which) * p.n_kv_heads + kvh) * head_block + (size_t)(pos % PAGE) * d;
            ((uint4*)dst)[piece] = ((const uint4*)src)[piece];
        }
    }
    if (own_here && warp == 0) {
        // the token's own key and value, as one more key of warp 0 (the lanes of key group 0)
        const h16* ksrc = p.k_new + (size_t)row * p.kv_stride + (size_t)kvh * d;
        const h16* vsrc = p.v_new + (size_t)row * p.kv_stride + (size_t)kvh * d;
        uint4 kown[E], vown[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
            kown[e] = dim_ok ? *(const uint4*)(ksrc + (e * LPK + sub) * 8) : make_uint4(0, 0, 0, 0);
            vown[e] = dim_ok ? *(const uint4*)(vsrc + (e * LPK + sub) * 8) : make_uint4(0, 0, 0, 0);
        }
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const h16x2* kk = (const h16x2*)&kown[e];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float2 f = h16x2_to_float2(kk[t]);
                dot = fmaf(q[e][2 * t], f.x, dot);
                dot = fmaf(q[e][2 * t + 1], f.y, dot);
            }
        }
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float s_own = __shfl_sync(0xffffffffu, dot, 0);
        const float m_new = fmaxf(m, s_own);
        const float corr = (m == -INFINITY) ? 0.f : __expf(m - m_new);
        l *= corr;
#pragma unroll
        for (int e = 0; e < E; ++e)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[e][i] *= corr;
        m = m_new;
        if (kgrp == 0) {
            const float pj = __expf(s_own - m);
            l += pj;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                const h16x2* vv = (const h16x2*)&vown[e];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float2 f = h16x2_to_float2(vv[t]);
                    acc[e][2 * t] = fmaf(pj, f.x, acc[e][2 * t]);
                    acc[e][2 * t + 1] = fmaf(pj, f.y, acc[e][2 * t + 1]);
                }
            }
        }
    }
    // lanes with the same dims but other keys -> one accumulator per dim slice; l counted once per key
#pragma unroll
    for (int o = 16; o >= LPK; o >>= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, o);
#pragma unroll
        for (int e = 0; e < E; ++e)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[e][i] += __shfl_xor_sync(0xffffffffu, acc[e][i], o);
    }
    if (lane < LPK) {
#pragma unroll
        for (int e = 0; e < E; ++e)
#pragma unroll
            for (int i = 0; i < 8; ++i) sm_acc[warp][(e * LPK + lane) * 8 + i] = acc[e][i];
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
    __syncthreads();

    // merge the warps
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm_m[w]);
    float L = 0.f, f[WARPS];
    const int t = threadIdx.x;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        f[w] = (sm_m[w] == -INFINITY) ? 0.f : __expf(sm_m[w] - M);
        L += sm_l[w] * f[w];
    }
    for (int t2 = t; t2 < d; t2 += WARPS * 32) {                  // head_dim may exceed the block size
        float o_val = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) o_val += sm_acc[w][t2] * f[w];
        if (p.n_splits == 1) {
            p.out[(size_t)row * p.out_stride + (size_t)h * d + t2] = float_to_h16(o_val / L);
        } else {
            float* dst = p.scratch + (((size_t)ri * p.n_heads + h) * p.n_splits + split) * (d + 2);
            dst[2 + t2] = o_val;
        }
    }
    if (p.n_splits == 1) return;
    if (t == 0) {
        float* dst = p.scratch + (((size_t)ri * p.n_heads + h) * p.n_splits + split) * (d + 2);
        dst[0] = M; dst[1] = L;
    }
    __threadfence();
    __syncthreads();
    if (t == 0) {
        int* c = p.counters + (size_t)ri * p.n_heads + h;
        const int prev = atomicAdd(c, 1);
        last_flag = (prev == p.n_splits - 1);
        if (last_flag) *c = 0;
    }
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    // Merge in split order.  Loads are issued eight splits at a time before their values are used,
    // so that the merge costs a few round trips to the second-level cache, not one per split.
    const float* base = p.scratch + ((size_t)ri * p.n_heads + h) * p.n_splits * (d + 2);
    const size_t stride = (size_t)(d + 2);
    const int S = p.n_splits;
    float GM = -INFINITY;
    for (int s0 = 0; s0 < S; s0 += 8) {
        float ms[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) ms[i] = s0 + i < S ? __ldcg(base + (s0 + i) * stride) : -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) GM = fmaxf(GM, ms[i]);
    }
    float GL = 0.f;
    for (int s0 = 0; s0 < S; s0 += 8) {
        float ms[8], ls[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            ms[i] = s0 + i < S ? __ldcg(base + (s0 + i) * stride) : -INFINITY;
            ls[i] = s0 + i < S ? __ldcg(base + (s0 + i) * stride + 1) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) GL += (ms[i] == -INFINITY) ? 0.f : ls[i] * __expf(ms[i] - GM);
    }
    for (int t2 = t; t2 < d; t2 += WARPS * 32) {
        float o = 0.f;
        for (int s0 = 0; s0 < S; s0 += 8) {
            float ms[8], vs[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                ms[i] = s0 + i < S ? __ldcg(base + (s0 + i) * stride) : -INFINITY;
                vs[i] = s0 + i < S ? __ldcg(base + (s0 + i) * stride + 2 + t2) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) if (ms[i] != -INFINITY) o += vs[i] * __expf(ms[i] - GM);
        }
        p.out[(size_t)row * p.out_stride + (size_t)h * d + t2] = float_to_h16(o / GL);
    }
}

// Launches the kernel for LPK lanes a key and E pieces a lane with 4, 8 or 16 warps a block (16 only for
// E = 1 and at most 16 lanes a key, where the registers allow it; 8 otherwise).
template <int LPK, int E>
int launch_decode(int warps, dim3 grid, cudaStream_t stream, const DecodeParams& p) {
    if constexpr (E == 1 && LPK <= 16) {
        if (warps == 16) return tnx_launch_in_order(attention_decode_kernel<LPK, E, 16>, grid, dim3(16 * 32), 0, stream, p);
    }
    if (warps >= 8) return tnx_launch_in_order(attention_decode_kernel<LPK, E, 8>, grid, dim3(8 * 32), 0, stream, p);
    return tnx_launch_in_order(attention_decode_kernel<LPK, E, 4>, grid, dim3(4 * 32), 0, stream, p);
}

}  // namespace

// Scratch floats and counters needed for n_rows decode rows with n_splits splits.
TNX_EXPORT long long tnx_attention_decode_scratch_floats(int n_rows, int n_heads, int head_dim, int n_splits) {
    return n_splits > 1 ? (long long)n_rows * n_heads * n_splits * (head_dim + 2) : 0;
}

// k_new / v_new: the keys and values of the rows' own tokens ([rows, kv_heads * head_dim], row pitch
// kv_stride elements), which the kernel then writes into the cache itself; null: already appended.
TNX_EXPORT int tnx_attention_decode_append(const void* q, int q_stride, void* cache, const int* block_tables,
                                           int bt_stride, const int* rows, const int* token_request, const int* positions,
                                           void* out, int out_stride, int n_rows, int n_heads, int n_kv_heads, int head_dim,
                                           int page_size, int window, float scale, int n_splits, int pages_per_split,
                                           float* scratch, int* counters, const void* k_new, const void* v_new,
                                           int kv_stride, int warps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (page_size != PAGE || head_dim % 16 || head_dim < 16 || head_dim > 256 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads || q_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15))
        return TNX_ERR_UNSUPPORTED;
    if ((k_new == nullptr) != (v_new == nullptr)) return TNX_ERR_BAD_ARG;
    if (k_new && (kv_stride % 8 || (((uintptr_t)k_new | (uintptr_t)v_new) & 15))) return TNX_ERR_UNSUPPORTED;
    if (n_splits < 1 || pages_per_split < 1) return TNX_ERR_BAD_ARG;
    if (n_splits > 1 && (!scratch || !counters)) return TNX_ERR_BAD_ARG;
    DecodeParams p;
    p.q = (const h16*)q; p.q_stride = q_stride; p.cache = (const h16*)cache;
    p.block_tables = block_tables; p.bt_stride = bt_stride; p.rows = rows; p.token_request = token_request;
    p.positions = positions; p.out = (h16*)out; p.out_stride = out_stride;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.window = window; p.scale = scale;
    p.n_splits = n_splits; p.pages_per_split = pages_per_split; p.scratch = scratch; p.counters = counters;
    p.k_new = (const h16*)k_new; p.v_new = (const h16*)v_new; p.kv_stride = kv_stride; p.cache_w = (h16*)cache;
    dim3 grid(n_heads, n_rows, n_splits);
    const int chunks = head_dim / 8;
    // Eight (or sixteen) warps a block where that puts every (row, head) on the GPU at once with few
    // or no splits (batch 8 of 32 heads: 256 blocks of eight warps and no merge through scratch memory
    // at all: 49 us against 53 with four warps and two splits); four warps otherwise.  The caller's plan
    // says which.
    if (warps != 4 && warps != 8 && warps != 16) return TNX_ERR_BAD_ARG;
    if (warps == 16 && chunks > 16) return TNX_ERR_UNSUPPORTED;      // sixteen warps of the widest heads would spill
    // Pieces of 8 dims per head: a power of two -> that many lanes a key; 3 times a power of two (head
    // sizes 48, 96, 192) -> a lane owns 3 pieces (96: 6.4 against 5.3 TB/s at batch 64); anything else ->
    // the next power of two with idle lanes.  (5 pieces a lane for head sizes 80 and 160 was measured: 210
    // registers, one block an SM, and no faster than the idle lanes: 4.6 TB/s both.)
    switch (chunks) {
        case 2: return launch_decode<2, 1>(warps, grid, stream, p);
        case 3: case 4: return launch_decode<4, 1>(warps, grid, stream, p);
        case 6: return launch_decode<2, 3>(warps, grid, stream, p);
        case 5: case 7: case 8: return launch_decode<8, 1>(warps, grid, stream, p);
        case 12: return launch_decode<4, 3>(warps, grid, stream, p);
        case 24: return launch_decode<8, 3>(warps, grid, stream, p);
        default: break;
    }
    if (chunks <= 16) return launch_decode<16, 1>(warps, grid, stream, p);
    return launch_decode<32, 1>(warps, grid, stream, p);
}

TNX_EXPORT int tnx_attention_decode(const void* q, int q_stride, const void* cache, const int* block_tables,
                                    int bt_stride, const int* rows, const int* token_request, const int* positions,
                                    void* out, int out_stride, int n_rows, int n_heads, int n_kv_heads, int head_dim,
                                    int page_size, int window, float scale, int n_splits, int pages_per_split,
                                    float* scratch, int* counters, cudaStream_t stream) {
    return tnx_attention_decode_append(q, q_stride, const_cast<void*>(cache), block_tables, bt_stride, rows, token_request,
                                       positions, out, out_stride, n_rows, n_heads, n_kv_heads, head_dim, page_size, window,
                                       scale, n_splits, pages_per_split, scratch, counters, nullptr, nullptr, 0, 4, stream);
}

// ---------------------------------------------------------------------------------------------------
// Entry point that allocates nothing (declared in attention_decode_noalloc.h).
//
// Same kernel as tnx_attention_decode; the split partials and the per-(row, head) counters live in
// file-scope device arrays of fixed size instead of buffers that the caller allocates.  Every GPU
// that loads this library holds these arrays (about 4.1 MB) until the process exits.
// ---------------------------------------------------------------------------------------------------
#include <cstdio>
#include <mutex>

#include "attention_decode_noalloc.h"

namespace {
static __device__ __align__(256) float g_noalloc_partials[TNX_NOALLOC_MAX_FLOATS];
static __device__ __align__(256) int g_noalloc_counters[TNX_NOALLOC_MAX_COUNTERS];

constexpr int MAX_DEVICES = 64;
struct NoAllocDevice { bool ready; float* partials; int* counters; };
NoAllocDevice g_noalloc_dev[MAX_DEVICES];
std::mutex g_noalloc_mu;
thread_local char g_noalloc_msg[512] = "";

// In host code the arrays' names are host-side stand-ins, not device addresses: the addresses
// that a kernel may use are asked for once per device, with that device current.
int noalloc_setup(int dev, float** partials, int** counters) {
    std::lock_guard<std::mutex> g(g_noalloc_mu);
    NoAllocDevice& s = g_noalloc_dev[dev];
    if (!s.ready) {
        void *pp = nullptr, *pc = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&pp, g_noalloc_partials);
        if (e != cudaSuccess) return (int)e;
        e = cudaGetSymbolAddress(&pc, g_noalloc_counters);
        if (e != cudaSuccess) return (int)e;
        s.partials = (float*)pp; s.counters = (int*)pc; s.ready = true;
    }
    *partials = s.partials; *counters = s.counters;
    return 0;
}
}  // namespace

TNX_EXPORT const char* tnx_attention_decode_noalloc_last_error() { return g_noalloc_msg; }

TNX_EXPORT int tnx_attention_decode_noalloc(const void* q, int q_stride, const void* cache, const int* block_tables,
                                            int bt_stride, const int* rows, const int* token_request,
                                            const int* positions, void* out, int out_stride, int n_rows, int n_heads,
                                            int n_kv_heads, int head_dim, int page_size, int window, float scale,
                                            int n_splits, int pages_per_split, cudaStream_t stream) {
    g_noalloc_msg[0] = 0;
    if (n_rows <= 0) return 0;
    // Every refusal leaves its reason, and nothing is queued on the stream before the arguments are
    // known to be good (the checks are the kernel's own, made here first).
    if (n_splits < 1 || pages_per_split < 1) {
        snprintf(g_noalloc_msg, sizeof g_noalloc_msg, "n_splits %d and pages_per_split %d must be positive", n_splits, pages_per_split);
        return TNX_ERR_BAD_ARG;
    }
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) {
        snprintf(g_noalloc_msg, sizeof g_noalloc_msg, "n_heads %d must be a positive multiple of n_kv_heads %d", n_heads, n_kv_heads);
        return TNX_ERR_BAD_ARG;
    }
    if (page_size != PAGE || head_dim % 16 || head_dim < 16 || head_dim > 256) {
        snprintf(g_noalloc_msg, sizeof g_noalloc_msg, "sizes refused: page_size must be 16 (got %d) and head_dim a multiple of "
                 "16 from 16 to 256 (got %d)", page_size, head_dim);
        return TNX_ERR_UNSUPPORTED;
    }
    if (q_stride % 8 || (((uintptr_t)q | (uintptr_t)cache) & 15)) {
        snprintf(g_noalloc_msg, sizeof g_noalloc_msg, "q and cache must be 16-byte aligned and q's row pitch a multiple of 8 elements");
        return TNX_ERR_UNSUPPORTED;
    }
    const long long floats = tnx_attention_decode_scratch_floats(n_rows, n_heads, head_dim, n_splits);
    const long long counters = (long long)n_rows * n_heads;
    if (floats > TNX_NOALLOC_MAX_FLOATS || (n_splits > 1 && counters > TNX_NOALLOC_MAX_COUNTERS)) {
        snprintf(g_noalloc_msg, sizeof g_noalloc_msg,
                 "n_rows %d x n_heads %d x n_splits %d x (head_dim %d + 2) = %lld floats and %lld counters exceed the "
                 "built-in scratch of %d floats and %d counters; use fewer splits or tnx_attention_decode with "
                 "scratch of your own", n_rows, n_heads, n_splits, head_dim, floats, counters,
                 TNX_NOALLOC_MAX_FLOATS, TNX_NOALLOC_MAX_COUNTERS);
        return TNX_ERR_UNSUPPORTED;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        snprintf(g_noalloc_msg, sizeof g_noalloc_msg, "cudaGetDevice failed with CUDA error %d", (int)e);
        return (int)e;
    }
    if (dev < 0 || dev >= MAX_DEVICES) {
        snprintf(g_noalloc_msg, sizeof g_noalloc_msg, "device index %d is beyond the %d this library tracks", dev, MAX_DEVICES);
        return TNX_ERR_UNSUPPORTED;
    }
    float* partials = nullptr;
    int* ctrs = nullptr;
    const int rc = noalloc_setup(dev, &partials, &ctrs);
    if (rc != 0) {
        snprintf(g_noalloc_msg, sizeof g_noalloc_msg, "cudaGetSymbolAddress failed with CUDA error %d", rc);
        return rc;
    }
    if (n_splits > 1) {
        // The arrays keep what the last call left; the counters must start at zero.
        e = cudaMemsetAsync(ctrs, 0, (size_t)counters * sizeof(int), stream);
        if (e != cudaSuccess) {
            snprintf(g_noalloc_msg, sizeof g_noalloc_msg, "clearing the counters failed with CUDA error %d", (int)e);
            return (int)e;
        }
    }
    const int r = tnx_attention_decode(q, q_stride, cache, block_tables, bt_stride, rows, token_request, positions, out,
                                       out_stride, n_rows, n_heads, n_kv_heads, head_dim, page_size, window, scale,
                                       n_splits, pages_per_split, partials, ctrs, stream);
    if (r != 0)
        snprintf(g_noalloc_msg, sizeof g_noalloc_msg, "the kernel's launch was refused with code %d", r);
    return r;
}
