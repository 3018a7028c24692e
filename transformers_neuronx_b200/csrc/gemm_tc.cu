// 16-bit (bfloat16, or float16 in the f16 build) matrix product on the 5th-generation tensor cores (tcgen05), operands brought into
// shared memory by TMA, 32-bit accumulators in tensor memory.
//
//   C[m, n] = epilogue( sum_k A[m, k] * W[n, k] )        A: [M, K] h16, W: [N, K] h16, row-major
//   epilogue: + bias[n] (32-bit); activation (by code, common.cuh); + residual[m, n] (32-bit); stored in the 16-bit type or as float.
//
// One CTA computes one 128 x BN tile of D = P Q^T over a range of K.  Two forms:
//   normal (many tokens): P = A (128 tokens), Q = W (BN = 128 features)
//   swapped (few tokens): P = W (128 features), Q = A (BN = 16/32/64/128 tokens): the weight matrix,
//     which is what a decode step has to stream from HBM, fills the 128-row operand and nothing
//     is wasted on padding tokens.  Few output tiles -> K is split over several CTAs.  With 2, 4
//     or 8 splits the CTAs of a tile form a thread-block cluster: each writes its 32-bit partial
//     tile to its own shared memory and then adds one band of rows over all CTAs' tiles (split
//     order, a fixed order) through distributed shared memory and applies the epilogue.  With
//     other split counts (a caller's choice) the partial tiles go to scratch memory and the CTA
//     that finishes last adds them, in the same order.
// Many tokens have two further kernels below: persistent CTAs with 128 x 256 tiles, and CTA pairs
// (tcgen05 cta_group::2) with 256 x 256 tiles, whose last, partly filled round of tiles can be
// shared out over all pairs by K blocks.
//
// Warp roles: warp 0 issues TMA loads, warp 1 allocates tensor memory and issues the MMAs (one
// elected lane), warps 2-5 read the accumulators (tcgen05.ld, one 32-lane quadrant each) and write
// the result.  Shared-memory stages are handed over with mbarriers; every wait is bounded and
// reports through an error word instead of hanging.
//
// TMA: every CTA loads its own tiles (no multicast); the innermost coordinate is a multiple of 64
// elements, so every copy starts on a 128-byte boundary.  K must be a multiple of 8 (row pitch a
// multiple of 16 bytes); K, M and N tails are zero-filled by TMA and masked at the store.
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int BLOCK_K = 64;          // 64 h16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int TILE_P = 128;          // rows of the 128-row operand = TMEM lanes
constexpr int NUM_THREADS = 192;
constexpr int MAX_CLUSTER = 8;               // the portable cluster size

// Instruction descriptor: D = f32, A = B = the build's 16-bit type, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
    return (1u << 4) | IDESC_H16_AB | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_P >> 4) << 24);
}

struct Params {
    int rows_p, rows_q;          // extents of the P (lane) and Q (column) axes
    int K;
    int kb_per_split;            // K blocks per split
    int splits;
    int ldc;
    int act;
    int c_is_h16;
    const float* bias;           // indexed by feature
    const float* residual;       // [M, ldc] 32-bit, may alias C
    void* C;
    float* partials;             // [splits][rows_p_padded][rows_q_padded] when splits > 1
    int* counters;               // one per output tile, zero between calls
    int* err;
    int cluster_reduce;          // few tokens, split K: the CTAs of a tile form a cluster and add their partial tiles
                                 // through distributed shared memory instead of scratch memory
    int sk_tiles;                // paired kernel: the last sk_tiles output tiles are shared out by K blocks
    int sk_pairs;                // ... over the first sk_pairs pairs
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
    return v;
}

template <int BN, bool SWAP>
__device__ __forceinline__ void store_tile_row(const Params& p, int lane_row, int col0, const float (&v)[32], int ncols,
                                               const float* bias_s = nullptr) {
    // lane_row: index on the P axis; col0..col0+ncols: indices on the Q axis.
    if (lane_row >= p.rows_p) return;
    if (SWAP) {
        // P axis = feature n, Q axis = token m: lanes of a warp write consecutive n.
        const int n = lane_row;
        const float b = p.bias ? p.bias[n] : 0.f;
        // The residual may be the output itself: read all of it before the first store, so that
        // the loads are in flight together instead of each waiting behind the store before it.
        float res[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int m = col0 + j;
            res[j] = (p.residual && j < ncols && m < p.rows_q) ? __ldcg(p.residual + (size_t)m * p.ldc + n) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int m = col0 + j;
            if (j < ncols && m < p.rows_q) {
                float x = v[j] + b;
                x = apply_activation(x, p.act);
                x += res[j];
                const size_t o = (size_t)m * p.ldc + n;
                if (p.c_is_h16) ((h16*)p.C)[o] = float_to_h16(x);
                else ((float*)p.C)[o] = x;
            }
        }
    } else {
        // P axis = token m, Q axis = feature n: a thread writes a run of its own row.  `bias_s`
        // (shared memory, the tile's bias from column col0 on) is read by all lanes at one address.
        const int m = lane_row;
        const size_t rowo = (size_t)m * p.ldc;
        const bool full = (col0 + 32 <= p.rows_q) && ncols == 32 && (p.ldc % 8 == 0);
        float x[32];
        if (full) {
            if (p.residual) {
                const float4* rp = (const float4*)(p.residual + rowo + col0);
                float4 rr[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) rr[q] = __ldcg(rp + q);          // all loads before the first store
#pragma unroll
                for (int q = 0; q < 8; ++q) { x[4 * q] = rr[q].x; x[4 * q + 1] = rr[q].y; x[4 * q + 2] = rr[q].z; x[4 * q + 3] = rr[q].w; }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) x[j] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                float t = v[j];
                if (p.bias) t += bias_s ? bias_s[j] : __ldg(p.bias + col0 + j);
                t = apply_activation(t, p.act);
                x[j] += t;
            }
            if (p.c_is_h16) {
                uint4* dst = (uint4*)((h16*)p.C + rowo + col0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    h16x2 h0 = floats_to_h16x2(x[8 * q + 0], x[8 * q + 1]);
                    h16x2 h1 = floats_to_h16x2(x[8 * q + 2], x[8 * q + 3]);
                    h16x2 h2 = floats_to_h16x2(x[8 * q + 4], x[8 * q + 5]);
                    h16x2 h3 = floats_to_h16x2(x[8 * q + 6], x[8 * q + 7]);
                    uint4 u;
                    u.x = *(uint32_t*)&h0; u.y = *(uint32_t*)&h1; u.z = *(uint32_t*)&h2; u.w = *(uint32_t*)&h3;
                    dst[q] = u;
                }
            } else {
                float4* dst = (float4*)((float*)p.C + rowo + col0);
#pragma unroll
                for (int q = 0; q < 8; ++q) dst[q] = make_float4(x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int n = col0 + j;
                float t = v[j];
                if (j < ncols && n < p.rows_q) {
                    if (p.bias) t += __ldg(p.bias + n);
                    t = apply_activation(t, p.act);
                    if (p.residual) t += p.residual[rowo + n];
                }
                x[j] = t;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int n = col0 + j;
                if (j < ncols && n < p.rows_q) {
                    if (p.c_is_h16) ((h16*)p.C)[rowo + n] = float_to_h16(x[j]);
                    else ((float*)p.C)[rowo + n] = x[j];
                }
            }
        }
    }
}

// The sum over a cluster's partial tiles for this CTA's band of rows, fetched from the S CTAs' shared memory
// (16-byte loads, in split order; bias, activation, residual; 16- or 8-byte stores).  A thread keeps four
// neighbouring features and walks over the band's tokens, two at a time with all their loads asked for before
// the first sum (a round trip to another SM's shared memory takes about a microsecond); what depends on the
// features only is computed once.
template <int BN, bool SWAP, int S>
__device__ __forceinline__ void cluster_reduce_items(const Params& p, uint32_t part_addr, int tile_p, int tile_q) {
    constexpr int NR = TILE_P / S;                                   // rows of this CTA's band
    constexpr int GROUPS = SWAP ? NR / 4 : BN / 4;                   // groups of four features
    constexpr int T_STEP = NUM_THREADS / GROUPS, U = 2;
    static_assert(NUM_THREADS % GROUPS == 0, "threads per feature group");
    const int my_rank = (int)cluster_ctarank();
    const int row_lo = NR * my_rank;
    const int g = threadIdx.x % GROUPS, t0 = threadIdx.x / GROUPS;
    const int n = SWAP ? tile_p * TILE_P + row_lo + 4 * g : tile_q * BN + 4 * g;          // first feature
    const int n_lim = SWAP ? p.rows_p : p.rows_q;
    if (n >= n_lim) return;
    const bool whole = n + 3 < n_lim;
    float b[4] = {0.f, 0.f, 0.f, 0.f};
    if (p.bias) {
#pragma unroll
        for (int e = 0; e < 4; ++e) if (n + e < n_lim) b[e] = __ldg(p.bias + n + e);
    }
    // token t of the band: its index m and the byte offset of this thread's four values in a partial tile
    const int m0 = SWAP ? tile_q * BN : tile_p * TILE_P + row_lo;
    const int tokens = min(SWAP ? BN : NR, (SWAP ? p.rows_q : p.rows_p) - m0);
    const uint32_t base = part_addr + (uint32_t)((SWAP ? row_lo + 4 * g : row_lo * (BN + 4) + 4 * g) * 4);
    constexpr uint32_t T_BYTES = (SWAP ? TILE_P : BN + 4) * 4;
    uint32_t src[S];
#pragma unroll
    for (int s = 0; s < S; ++s) src[s] = s == my_rank ? base : map_to_cta(base, (uint32_t)s);
    for (int t = t0; t < tokens; t += T_STEP * U) {
        float4 f[U][S], res[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int tt = t + u * T_STEP;
            res[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (tt < tokens && p.residual) {
                const float* rp = p.residual + (size_t)(m0 + tt) * p.ldc + n;
                if (whole) res[u] = __ldcg((const float4*)rp);
                else { res[u].x = rp[0]; if (n + 1 < n_lim) res[u].y = rp[1]; if (n + 2 < n_lim) res[u].z = rp[2]; }
            }
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const uint32_t a = src[s] + (uint32_t)tt * T_BYTES;
                if (tt >= tokens) {
                    f[u][s] = make_float4(0.f, 0.f, 0.f, 0.f);
                } else if (s == my_rank) {                    // this CTA's own partial tile: a plain shared-memory load
                    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(f[u][s].x), "=f"(f[u][s].y), "=f"(f[u][s].z), "=f"(f[u][s].w) : "r"(a) : "memory");
                } else {
                    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(f[u][s].x), "=f"(f[u][s].y), "=f"(f[u][s].z), "=f"(f[u][s].w) : "r"(a) : "memory");
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int tt = t + u * T_STEP;
            if (tt >= tokens) continue;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < S; ++s) { v[0] += f[u][s].x; v[1] += f[u][s].y; v[2] += f[u][s].z; v[3] += f[u][s].w; }      // split order
            const float rr[4] = {res[u].x, res[u].y, res[u].z, res[u].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = apply_activation(v[e] + b[e], p.act) + rr[e];
            const size_t o = (size_t)(m0 + tt) * p.ldc + n;
            if (whole) {
                if (p.c_is_h16) {
                    h16x2 h0 = floats_to_h16x2(v[0], v[1]), h1 = floats_to_h16x2(v[2], v[3]);
                    uint2 w; w.x = *(uint32_t*)&h0; w.y = *(uint32_t*)&h1;
                    *(uint2*)((h16*)p.C + o) = w;
                } else {
                    *(float4*)((float*)p.C + o) = make_float4(v[0], v[1], v[2], v[3]);
                }
            } else {
                for (int e = 0; e < 4 && n + e < n_lim; ++e) {
                    if (p.c_is_h16) ((h16*)p.C)[o + e] = float_to_h16(v[e]);
                    else ((float*)p.C)[o + e] = v[e];
                }
            }
        }
    }
}

// The same sum when the partial tiles' bands have been sent to their owners (swapped form): this CTA's own band
// lies in its staging area, the S - 1 others' in the receive area, all [col][row of the band]; plain shared loads.
// What a thread of the sum over received bands needs from memory and can ask for long before the sum: the bias of
// its four features (before the wait for the preceding kernel: no kernel writes it) and, where its tokens are at most
// two, their residual values (right after that wait).  They then stand in registers through the main loop instead
// of costing a round trip to the second-level cache in the product's tail.
struct EarlyOperands {
    float bias[4];
    float4 res[2];
    bool have;                   // the residual values are in res (else the sum reads them itself)
};

template <int BN, int S>
__device__ __forceinline__ void cluster_sum_received(const Params& p, const float* staged, const float* recv, int r, int tile_p, int tile_q,
                                                     const EarlyOperands& early) {
    // A thread keeps its four features and walks over the tokens: everything that depends on the features
    // only (bias, bounds, the addresses' fixed parts) is computed once.
    constexpr int NR = TILE_P / S, GROUPS = NR / 4, COL_STEP = NUM_THREADS / GROUPS;
    static_assert(NUM_THREADS % GROUPS == 0, "threads per band row group");
    const int rg = threadIdx.x % GROUPS, col0 = threadIdx.x / GROUPS;
    const int n = tile_p * TILE_P + r * NR + 4 * rg;                       // first feature
    if (n >= p.rows_p) return;
    const bool whole = n + 3 < p.rows_p;
    const float b[4] = {early.bias[0], early.bias[1], early.bias[2], early.bias[3]};
    const float* src[S];
#pragma unroll
    for (int s = 0; s < S; ++s) src[s] = (s == r ? staged + (size_t)r * BN * NR : recv + (size_t)(s < r ? s : s - 1) * BN * NR) + 4 * rg;
    const int m0 = tile_q * BN;
    const int cols = min(BN, p.rows_q - m0);                               // tokens that exist
    constexpr int U = 2;
    for (int col = col0; col < cols; col += COL_STEP * U) {
        float4 res[U];
        float v[U][4];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = col + u * COL_STEP;
            res[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (early.have) {
                res[u] = early.res[u];                                     // this thread's only tokens: col0 and col0 + COL_STEP
            } else if (c < cols && p.residual) {
                const float* rp = p.residual + (size_t)(m0 + c) * p.ldc + n;
                if (whole) res[u] = __ldcg((const float4*)rp);
                else { res[u].x = rp[0]; if (n + 1 < p.rows_p) res[u].y = rp[1]; if (n + 2 < p.rows_p) res[u].z = rp[2]; }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = col + u * COL_STEP;
            v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.f;
            if (c < cols) {
#pragma unroll
                for (int s = 0; s < S; ++s) {                              // split order
                    const float4 f = *(const float4*)(src[s] + c * NR);
                    v[u][0] += f.x; v[u][1] += f.y; v[u][2] += f.z; v[u][3] += f.w;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = col + u * COL_STEP;
            if (c >= cols) continue;
            const float rr[4] = {res[u].x, res[u].y, res[u].z, res[u].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) v[u][e] = apply_activation(v[u][e] + b[e], p.act) + rr[e];
            const size_t o = (size_t)(m0 + c) * p.ldc + n;
            if (whole) {
                if (p.c_is_h16) {
                    h16x2 h0 = floats_to_h16x2(v[u][0], v[u][1]), h1 = floats_to_h16x2(v[u][2], v[u][3]);
                    uint2 w; w.x = *(uint32_t*)&h0; w.y = *(uint32_t*)&h1;
                    *(uint2*)((h16*)p.C + o) = w;
                } else {
                    *(float4*)((float*)p.C + o) = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
                }
            } else {
                for (int e = 0; e < 4 && n + e < p.rows_p; ++e) {
                    if (p.c_is_h16) ((h16*)p.C)[o + e] = float_to_h16(v[u][e]);
                    else ((float*)p.C)[o + e] = v[u][e];
                }
            }
        }
    }
}

template <int BN, int STAGES, bool SWAP>
__global__ void __launch_bounds__(NUM_THREADS, SWAP ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, const Params p) {
    constexpr int A_BYTES = TILE_P * BLOCK_K * 2;            // 16 KB
    constexpr int B_BYTES = BN * BLOCK_K * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr int LD_COLS = BN < 32 ? 16 : 32;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], tmem_full_bar, recv_bar;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int last_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_p = blockIdx.x, tile_q = blockIdx.y, split = blockIdx.z;
    // Split K summed in a cluster, swapped form, 2, 4 or 8 splits: every CTA sends the bands of its partial tile
    // to their owners (one bulk copy from shared memory to shared memory each) and adds up what it receives
    // with plain shared-memory loads.  The staging area (a tile) and the receive area (S - 1 bands of it) must
    // fit the stages; where they do not (128 tokens with 4 or 8 splits), or the addresses do not allow 16-byte
    // accesses, the owners fetch the bands from the other CTAs' shared memory instead.
    constexpr int TILE_BYTES = BN * TILE_P * 4;
    const bool sum_by_push = SWAP && p.cluster_reduce && (p.splits == 2 || p.splits == 4 || p.splits == 8) &&
                             TILE_BYTES * (2 * p.splits - 1) <= STAGES * STAGE_BYTES * p.splits && p.ldc % 4 == 0 &&
                             !(((uintptr_t)p.C | (uintptr_t)p.residual | (uintptr_t)p.bias) & 15);
    const int num_kb_total = (p.K + BLOCK_K - 1) / BLOCK_K;
    const int kb_begin = split * p.kb_per_split;
    const int kb_end = min(num_kb_total, kb_begin + p.kb_per_split);
    const int num_kb = max(0, kb_end - kb_begin);

    // One K block = one stage: the weight tile and the activation tile complete the same barrier.
    // The weights are never written by a kernel, so their loads may start before the preceding
    // kernel has finished (programmatic dependent launch); the activations may not.
    auto load_weights = [&](int i) {
        const int s = i % STAGES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        uint8_t* a_dst = smem + (size_t)s * STAGE_BYTES;
        const int kx = (kb_begin + i) * BLOCK_K;
        if (SWAP) tma_load_2d(a_dst, &map_p, &full_bar[s], kx, tile_p * TILE_P);
        else tma_load_2d(a_dst + A_BYTES, &map_q, &full_bar[s], kx, tile_q * BN);
    };
    auto load_activations = [&](int i) {
        const int s = i % STAGES;
        uint8_t* a_dst = smem + (size_t)s * STAGE_BYTES;
        const int kx = (kb_begin + i) * BLOCK_K;
        if (SWAP) tma_load_2d(a_dst + A_BYTES, &map_q, &full_bar[s], kx, tile_q * BN);
        else tma_load_2d(a_dst, &map_p, &full_bar[s], kx, tile_p * TILE_P);
    };
    pdl_launch_dependents();
    int issued = 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&tmem_full_bar, 1);
        mbar_init(&recv_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_p) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_q) : "memory");
        for (; issued < num_kb && issued < STAGES; ++issued) load_weights(issued);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, TMEM_COLS);
        tmem_relinquish();
    }
    // (the indices are those of cluster_sum_received)
    EarlyOperands early;
    early.have = false;
    early.bias[0] = early.bias[1] = early.bias[2] = early.bias[3] = 0.f;
    early.res[0] = early.res[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int e_groups = TILE_P / 4 / (sum_by_push ? p.splits : 1);
    const int e_n = tile_p * TILE_P + (sum_by_push ? (int)cluster_ctarank() * (TILE_P / p.splits) : 0) + 4 * ((int)threadIdx.x % e_groups);
    if (sum_by_push && p.bias) {
#pragma unroll
        for (int e = 0; e < 4; ++e) if (e_n + e < p.rows_p) early.bias[e] = __ldg(p.bias + e_n + e);
    }
    pdl_wait();                       // from here on the preceding kernel's results may be read, and ours written
    if (sum_by_push) {
        const int col_step = NUM_THREADS / e_groups, col0 = (int)threadIdx.x / e_groups;
        const int cols = min(BN, p.rows_q - tile_q * BN);
        early.have = cols <= 2 * col_step;
        if (early.have && p.residual && e_n < p.rows_p) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int c = col0 + u * col_step;
                if (c < cols) {
                    const float* rp = p.residual + (size_t)(tile_q * BN + c) * p.ldc + e_n;
                    if (e_n + 3 < p.rows_p) early.res[u] = __ldcg((const float4*)rp);
                    else { early.res[u].x = rp[0]; if (e_n + 1 < p.rows_p) early.res[u].y = rp[1]; if (e_n + 2 < p.rows_p) early.res[u].z = rp[2]; }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_smem;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < issued; ++i) load_activations(i);
            for (int i = issued; i < num_kb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                ok = mbar_wait(&empty_bar[s], ph ^ 1, p.err, 1);
                if (!ok) break;
                load_weights(i);
                load_activations(i);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            for (int i = 0; i < num_kb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                ok = mbar_wait(&full_bar[s], ph, p.err, 2);
                if (!ok) break;
                const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_BYTES;
                const uint64_t adesc = smem_desc_sw128(a_addr);
                const uint64_t bdesc = smem_desc_sw128(b_addr);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    // advancing 16 elements along K = 32 bytes = 2 units of the address field
                    umma_h16(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                              (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);          // the stage is free once these MMAs have read it
            }
            umma_commit(&tmem_full_bar);             // accumulators complete
        }
    } else {
        // Epilogue warps 2..5: TMEM lane quadrant = warp % 4.
        const int quad = warp & 3;
        const int row_in_tile = quad * 32 + lane;
        ok = __all_sync(0xffffffffu, mbar_wait(&tmem_full_bar, 0, p.err, 3));     // one answer for the warp
        tc_fence_after();
        const int lane_row = tile_p * TILE_P + row_in_tile;
        if (ok) {
            if (p.splits == 1) {
#pragma unroll 1
                for (int c = 0; c < BN; c += LD_COLS) {
                    uint32_t r[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c;
                    if (LD_COLS == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
                    tmem_ld_wait();
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = (j < LD_COLS && num_kb > 0) ? __uint_as_float(r[j]) : 0.f;
                    store_tile_row<BN, SWAP>(p, lane_row, tile_q * BN + c, v, LD_COLS);
                }
            } else if (p.cluster_reduce && !sum_by_push) {
                // 32-bit partial tile -> this CTA's shared memory, [col 0..BN)[row 0..127], over the
                // first stages (every load into them has been consumed by now)
                // (swapped: [col][row], the lanes of a warp write consecutive floats; otherwise [row][col]
                // with rows of BN + 4 floats, written 16 bytes at a time: eight lanes then cover all banks)
                float* part = (float*)smem + (SWAP ? row_in_tile : row_in_tile * (BN + 4));
#pragma unroll 1
                for (int c = 0; c < BN; c += LD_COLS) {
                    uint32_t r[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c;
                    if (LD_COLS == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
                    tmem_ld_wait();
                    if (SWAP) {
#pragma unroll
                        for (int j = 0; j < LD_COLS; ++j) part[(c + j) * TILE_P] = num_kb > 0 ? __uint_as_float(r[j]) : 0.f;
                    } else {
#pragma unroll
                        for (int j = 0; j < LD_COLS; j += 4)
                            *(float4*)(part + c + j) = num_kb > 0 ? make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]))
                                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
            } else if (!p.cluster_reduce) {
                // 32-bit partial tile -> scratch: [split][tile][col 0..BN)[row 0..127]: the 32 lanes
                // of a warp write 32 consecutive floats
                const size_t tiles = (size_t)gridDim.x * gridDim.y;
                const size_t tile_id = (size_t)tile_p * gridDim.y + tile_q;
                float* dst = p.partials + ((size_t)split * tiles + tile_id) * TILE_P * BN + row_in_tile;
#pragma unroll 1
                for (int c = 0; c < BN; c += LD_COLS) {
                    uint32_t r[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c;
                    if (LD_COLS == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < LD_COLS; ++j)
                        __stcg(dst + (size_t)(c + j) * TILE_P, num_kb > 0 ? __uint_as_float(r[j]) : 0.f);
                }
            }
        }
    }

    // ---- split-K within a cluster: every CTA adds a band of rows over all partial tiles ----------
    if (p.splits > 1 && p.cluster_reduce && sum_by_push) {
        const int S = p.splits, r = (int)cluster_ctarank();
        const int nr = TILE_P / S;
        const uint32_t band_bytes = (uint32_t)(BN * nr * 4);
        float* const recv = (float*)(smem + TILE_BYTES);
        if (warp >= 2) {
            // the partial tile -> the staging area, [band][col][row of the band]: a band is one run of bytes
            const int quad = warp & 3, rr = quad * 32 + lane;
            float* part = (float*)smem + (rr / nr) * BN * nr + rr % nr;
#pragma unroll 1
            for (int c = 0; c < BN; c += LD_COLS) {
                uint32_t v[32];
                if (ok) {
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c;
                    if (LD_COLS == 32) tmem_ld32(taddr, v); else tmem_ld16(taddr, v);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < LD_COLS; ++j) part[(c + j) * nr] = (ok && num_kb > 0) ? __uint_as_float(v[j]) : 0.f;    // defined even if a wait ran out
            }
            fence_proxy_async_smem();                     // the staged tile is read by bulk copies
        }
        if (threadIdx.x == 0) mbar_expect_tx(&recv_bar, (uint32_t)(S - 1) * band_bytes);
        tc_fence_before();
        cluster_sync();                                   // every CTA's tile is staged, its stages idle, its barrier armed
        if ((int)threadIdx.x < S && (int)threadIdx.x != r) {
            const int t = (int)threadIdx.x;               // the owner of band t gets it, as contributor r
            const uint32_t src = smem_u32(smem) + (uint32_t)t * band_bytes;
            const uint32_t dst = map_to_cta(smem_u32(recv) + (uint32_t)(r < t ? r : r - 1) * band_bytes, (uint32_t)t);
            const uint32_t bar = map_to_cta(smem_u32(&recv_bar), (uint32_t)t);
            asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(dst), "r"(src), "r"(band_bytes), "r"(bar) : "memory");
        }
        const bool got = mbar_wait(&recv_bar, 0, p.err, 4);
        __syncwarp();
        // What the others sent here has arrived, so they may let go of it: a CTA leaves when all have said so.
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        if (got) {
            if (S == 2) cluster_sum_received<BN, 2>(p, (const float*)smem, recv, r, tile_p, tile_q, early);
            else if (S == 4) cluster_sum_received<BN, 4>(p, (const float*)smem, recv, r, tile_p, tile_q, early);
            else cluster_sum_received<BN, 8>(p, (const float*)smem, recv, r, tile_p, tile_q, early);
        }
        __syncwarp();
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    } else if (p.splits > 1 && p.cluster_reduce) {
        if (warp >= 2 && !ok) {                           // a wait ran out: the partial tile must still be defined
            const int rr = (warp & 3) * 32 + lane;
            float* part = (float*)smem + (SWAP ? rr : rr * (BN + 4));
            for (int c = 0; c < BN; ++c) part[SWAP ? c * TILE_P : c] = 0.f;
        }
        tc_fence_before();
        cluster_sync();                                   // all partial tiles of the cluster are written
        const int S = p.splits, r = (int)cluster_ctarank();
        const int row_lo = TILE_P * r / S, n_rows = TILE_P * (r + 1) / S - row_lo;
        const uint32_t part_addr = smem_u32(smem);
        // Four neighbouring features at a time where the band and the output allow it (16-byte
        // loads from the other SMs' shared memory, 16- or 8-byte stores), else one by one.
        const bool vec = (S == 2 || S == 4 || S == 8) && p.ldc % 4 == 0 && !(((uintptr_t)p.C | (uintptr_t)p.residual | (uintptr_t)p.bias) & 15);
        if (vec) {
            if (S == 2) cluster_reduce_items<BN, SWAP, 2>(p, part_addr, tile_p, tile_q);
            else if (S == 4) cluster_reduce_items<BN, SWAP, 4>(p, part_addr, tile_p, tile_q);
            else cluster_reduce_items<BN, SWAP, 8>(p, part_addr, tile_p, tile_q);
        } else
        for (int item = threadIdx.x; item < n_rows * BN; item += NUM_THREADS) {
            // consecutive threads: consecutive features, which lie side by side in the output
            int row, col;
            if (SWAP) { col = item / n_rows; row = row_lo + item - col * n_rows; }
            else { row = row_lo + item / BN; col = item - (item / BN) * BN; }
            const int n = SWAP ? tile_p * TILE_P + row : tile_q * BN + col;      // feature
            const int m = SWAP ? tile_q * BN + col : tile_p * TILE_P + row;      // token
            const bool live = SWAP ? (n < p.rows_p && m < p.rows_q) : (m < p.rows_p && n < p.rows_q);
            const size_t o = (size_t)m * p.ldc + n;
            const float res = (live && p.residual) ? __ldcg(p.residual + o) : 0.f;      // in flight during the sum
            const uint32_t a = part_addr + (uint32_t)((SWAP ? col * TILE_P + row : row * (BN + 4) + col) * 4);
            // all loads first (they travel to the other SMs together), then the sum in split order
            float f[MAX_CLUSTER];
#pragma unroll
            for (int s = 0; s < MAX_CLUSTER; ++s) f[s] = s < S ? ld_cluster_f32(map_to_cta(a, (uint32_t)s)) : 0.f;
            float v = 0.f;
#pragma unroll
            for (int s = 0; s < MAX_CLUSTER; ++s) if (s < S) v += f[s];
            if (live) {
                if (p.bias) v += __ldg(p.bias + n);
                v = apply_activation(v, p.act);
                v += res;
                if (p.c_is_h16) ((h16*)p.C)[o] = float_to_h16(v);
                else ((float*)p.C)[o] = v;
            }
        }
        cluster_sync();                                   // no CTA leaves while its partial tile may still be read
    }

    // ---- split-K: the CTA that finishes last adds the partial tiles in split order -------------
    if (p.splits > 1 && !p.cluster_reduce) {
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const int tile_id = tile_p * gridDim.y + tile_q;
            const int prev = atomicAdd(&p.counters[tile_id], 1);
            last_flag = (prev == p.splits - 1);
            if (last_flag) p.counters[tile_id] = 0;           // ready for the next call
        }
        __syncthreads();
        if (last_flag && warp >= 2) {
            __threadfence();
            const int quad = warp & 3;
            const int row_in_tile = quad * 32 + lane;
            const int lane_row = tile_p * TILE_P + row_in_tile;
            const size_t tiles = (size_t)gridDim.x * gridDim.y;
            const size_t tile_id = (size_t)tile_p * gridDim.y + tile_q;
#pragma unroll 1
            for (int c = 0; c < BN; c += LD_COLS) {
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.f;
                // Split order: the sum does not depend on timing.  The loads of four splits are issued
                // together, so that the sum costs a few round trips to the second-level cache, not one
                // per split.
                constexpr int GROUP = LD_COLS == 16 ? 4 : 2;
                const float* src0 = p.partials + tile_id * TILE_P * BN + row_in_tile + (size_t)c * TILE_P;
                const size_t split_stride = tiles * TILE_P * BN;
                for (int s0 = 0; s0 < p.splits; s0 += GROUP) {
                    float f[GROUP][LD_COLS];
#pragma unroll
                    for (int g = 0; g < GROUP; ++g) {
                        if (s0 + g < p.splits) {
                            const float* src = src0 + (size_t)(s0 + g) * split_stride;
#pragma unroll
                            for (int j = 0; j < LD_COLS; ++j) f[g][j] = __ldcg(src + (size_t)j * TILE_P);
                        } else {
#pragma unroll
                            for (int j = 0; j < LD_COLS; ++j) f[g][j] = 0.f;
                        }
                    }
#pragma unroll
                    for (int g = 0; g < GROUP; ++g)
#pragma unroll
                        for (int j = 0; j < LD_COLS; ++j) v[j] += f[g][j];
                }
                store_tile_row<BN, SWAP>(p, lane_row, tile_q * BN + c, v, LD_COLS);
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------------------------
    if (!ok) {
        // A wait ran out: give copies in flight time to land before the shared memory is released.
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 1000000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Where an epilogue warp takes its 32 rows x 32 columns of sums from: tensor memory, or (a tile
// whose K range was shared out over several CTAs) the partial tiles in scratch memory, added in the
// order of the contributors so that the sum does not depend on who finished last.
struct AccSource {
    uint32_t tmem_addr;          // this warp's lanes, column 0 of the accumulator
    const float* part0;          // null, or the partial tiles (this thread's row): contributor 0 lies at
    int n_parts;                 // part0 + first_off, contributor s > 0 at part0 + s * stride
    long long first_off, stride;
};
constexpr int PART_LD = 128;     // partial tiles are [column][128 rows]: the lanes of a warp write 128 bytes

template <bool FROM_SCRATCH>
__device__ __forceinline__ void acc_load_begin(const AccSource& a, int c, uint32_t (&r)[32]) {
    if (!FROM_SCRATCH) { tmem_ld32(a.tmem_addr + (uint32_t)c, r); return; }
    // Sixteen columns at a time; the loads of contributor s + 1 are issued before the values of
    // contributor s are added, so that two round trips to the second-level cache are in flight.
    auto part = [&](int s) { return a.part0 + (s == 0 ? a.first_off : a.stride * s) + (size_t)c * PART_LD; };
#pragma unroll
    for (int h = 0; h < 32; h += 16) {
        float f[16], g[16];
        {
            const float* src = part(0) + (size_t)h * PART_LD;
#pragma unroll
            for (int j = 0; j < 16; ++j) { f[j] = __ldcg(src + (size_t)j * PART_LD); r[h + j] = 0u; }
        }
        for (int s = 0; s < a.n_parts; s += 2) {
            if (s + 1 < a.n_parts) {
                const float* src = part(s + 1) + (size_t)h * PART_LD;
#pragma unroll
                for (int j = 0; j < 16; ++j) g[j] = __ldcg(src + (size_t)j * PART_LD);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) r[h + j] = __float_as_uint(__uint_as_float(r[h + j]) + f[j]);
            if (s + 1 < a.n_parts) {
                if (s + 2 < a.n_parts) {
                    const float* src = part(s + 2) + (size_t)h * PART_LD;
#pragma unroll
                    for (int j = 0; j < 16; ++j) f[j] = __ldcg(src + (size_t)j * PART_LD);
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) r[h + j] = __float_as_uint(__uint_as_float(r[h + j]) + g[j]);
            }
        }
    }
}
template <bool FROM_SCRATCH>
__device__ __forceinline__ void acc_load_end(const AccSource& a) {
    if (!FROM_SCRATCH) tmem_ld_wait();
}

// Epilogue of one warp of the many-token kernels: its 32 accumulator rows x WIDTH columns -> C.
// With a residual (32-bit, possibly C itself) the loads of the next 32 columns are issued before
// the current ones are stored, so that a tile costs one memory round trip, not one per chunk.
template <int WIDTH, bool FROM_SCRATCH = false>
__device__ __forceinline__ void drain_accumulator(const Params& p, const AccSource& acc, int row, int col_base,
                                                  const float* bias_tile) {
    // The choice of path must be the same for all lanes of the warp: tcgen05.ld is a warp-wide
    // instruction.  Rows beyond the matrix are handled by predicating the loads and stores.
    const bool pipelined = p.residual && (p.ldc % 8 == 0) && (col_base + WIDTH <= p.rows_q);
    const bool valid = row < p.rows_p;
    if (!pipelined) {
#pragma unroll 1
        for (int c = 0; c < WIDTH; c += 32) {
            uint32_t r[32];
            acc_load_begin<FROM_SCRATCH>(acc, c, r);
            acc_load_end<FROM_SCRATCH>(acc);
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            store_tile_row<WIDTH, false>(p, row, col_base + c, v, 32, p.bias ? bias_tile + c : nullptr);
        }
        return;
    }
    const size_t row_off = valid ? (size_t)row * p.ldc + col_base : 0;
    const float* res_row = p.residual + row_off;
    float* out_row = (float*)p.C + row_off;
    float4 cur[8], nxt[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) cur[q] = valid ? __ldcg((const float4*)res_row + q) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
    for (int c = 0; c < WIDTH; c += 32) {
        uint32_t r[32];
        acc_load_begin<FROM_SCRATCH>(acc, c, r);
        if (c + 32 < WIDTH && valid) {
#pragma unroll
            for (int q = 0; q < 8; ++q) nxt[q] = __ldcg((const float4*)(res_row + c + 32) + q);
        }
        acc_load_end<FROM_SCRATCH>(acc);
        const float* b = p.bias ? bias_tile + c : nullptr;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            float4 o;
            float t0 = __uint_as_float(r[4 * q]), t1 = __uint_as_float(r[4 * q + 1]);
            float t2 = __uint_as_float(r[4 * q + 2]), t3 = __uint_as_float(r[4 * q + 3]);
            if (b) { t0 += b[4 * q]; t1 += b[4 * q + 1]; t2 += b[4 * q + 2]; t3 += b[4 * q + 3]; }
            if (p.act) { t0 = apply_activation(t0, p.act); t1 = apply_activation(t1, p.act); t2 = apply_activation(t2, p.act); t3 = apply_activation(t3, p.act); }
            o.x = cur[q].x + t0; o.y = cur[q].y + t1; o.z = cur[q].z + t2; o.w = cur[q].w + t3;
            if (valid) ((float4*)(out_row + c))[q] = o;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) cur[q] = nxt[q];
    }
}

// ---- many tokens: persistent CTAs, 128 x 256 tiles, two accumulators in tensor memory ---------------
//
// One CTA per SM walks over output tiles (tile = first + i * CTAs; consecutive tiles share the weight
// tile and differ in the token tile, so CTAs running at the same time reuse weights and activations
// in L2).  The shared-memory ring of K blocks runs on across tiles.  Tensor memory holds two
// 128 x 256 accumulators: while the epilogue warps drain one, the MMA warp fills the other.
constexpr int PBN = 256;
constexpr int PSTAGES = 4;

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                          const Params p, int tiles_m, int tiles_n) {
    constexpr int A_BYTES = TILE_P * BLOCK_K * 2;             // 16 KB
    constexpr int B_BYTES = PBN * BLOCK_K * 2;                // 32 KB
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[PSTAGES], empty_bar[PSTAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_smem;
    __shared__ float bias_tile[2][PBN];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (p.K + BLOCK_K - 1) / BLOCK_K;
    const int n_tiles = tiles_m * tiles_n;
    const int first = blockIdx.x, stride = gridDim.x;
    const int my_tiles = first < n_tiles ? (n_tiles - first + stride - 1) / stride : 0;
    const long long total = (long long)my_tiles * num_kb;     // K blocks this CTA loads, over all its tiles

    auto tile_of = [&](long long it, int& tm, int& tn, int& kb) {
        const int t = first + (int)(it / num_kb) * stride;
        kb = (int)(it % num_kb);
        tm = t % tiles_m; tn = t / tiles_m;
    };
    auto load_weights = [&](long long it) {
        int tm, tn, kb; tile_of(it, tm, tn, kb);
        const int s = (int)(it % PSTAGES);
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(smem + (size_t)s * STAGE_BYTES + A_BYTES, &map_q, &full_bar[s], kb * BLOCK_K, tn * PBN);
    };
    auto load_activations = [&](long long it) {
        int tm, tn, kb; tile_of(it, tm, tn, kb);
        const int s = (int)(it % PSTAGES);
        tma_load_2d(smem + (size_t)s * STAGE_BYTES, &map_p, &full_bar[s], kb * BLOCK_K, tm * TILE_P);
    };

    pdl_launch_dependents();
    long long issued = 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < PSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_p) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_q) : "memory");
        for (; issued < total && issued < PSTAGES; ++issued) load_weights(issued);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, 512);
        tmem_relinquish();
    }
    pdl_wait();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_smem;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            for (long long it = 0; it < issued; ++it) load_activations(it);
            for (long long it = issued; it < total && ok; ++it) {
                const int s = (int)(it % PSTAGES);
                const uint32_t ph = (uint32_t)((it / PSTAGES) & 1);
                ok = mbar_wait(&empty_bar[s], ph ^ 1, p.err, 11);
                if (!ok) break;
                load_weights(it);
                load_activations(it);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(PBN);
            long long it = 0;
            for (int t = 0; t < my_tiles && ok; ++t) {
                const int acc = t & 1;
                const uint32_t acc_ph = (uint32_t)((t >> 1) & 1);
                ok = mbar_wait(&acc_empty[acc], acc_ph ^ 1, p.err, 12);     // the epilogue has drained this accumulator
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * PBN);
                for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
                    const int s = (int)(it % PSTAGES);
                    const uint32_t ph = (uint32_t)((it / PSTAGES) & 1);
                    ok = mbar_wait(&full_bar[s], ph, p.err, 13);
                    if (!ok) break;
                    const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint64_t adesc = smem_desc_sw128(a_addr);
                    const uint64_t bdesc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                        umma_h16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty_bar[s]);
                }
                umma_commit(&acc_full[acc]);
            }
        }
    } else {
        const int quad = warp & 3;
        const int row_in_tile = quad * 32 + lane;
        for (int t = 0; t < my_tiles && ok; ++t) {
            const int acc = t & 1;
            const uint32_t acc_ph = (uint32_t)((t >> 1) & 1);
            const int tile = first + t * stride;
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            if (p.bias) {                                  // this tile's bias -> shared memory (epilogue threads only)
                const int et = threadIdx.x - 64;
                for (int j = et; j < PBN; j += 128) bias_tile[acc][j] = (tn * PBN + j < p.rows_q) ? p.bias[tn * PBN + j] : 0.f;
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[acc], acc_ph, p.err, 14));
            if (!ok) break;
            tc_fence_after();
            const AccSource src{tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * PBN), nullptr, 0, 0, 0};
            drain_accumulator<PBN>(p, src, tm * TILE_P + row_in_tile, tn * PBN, bias_tile[acc]);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[acc])) : "memory");
            }
        }
    }
    if (!ok) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 1000000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Epilogue of one warp with a 32-bit residual, through TMA: the residual's 32 x 32 boxes are
// fetched into shared memory two boxes ahead (the first two while the MMAs of the tile still run),
// the accumulator is added in place and the box is written back by a TMA store.  Global memory is
// then read and written in whole 128-byte rows instead of one 16-byte piece per thread and row, and
// no thread waits for a load.  Rows and columns beyond the matrix are zero-filled by the load and
// clipped by the store.  `n` counts the boxes this warp has handled since the kernel began: box n
// uses buffer n % 3 and the phase (n / 3) & 1 of that buffer's barrier.
constexpr int EPI_BUFS = 3;
constexpr int EPI_BOX_BYTES = 32 * 32 * 4;                    // 4 KB: 32 rows x 128 bytes, 128-byte swizzle

struct EpilogueTma {
    const CUtensorMap* map_res;
    const CUtensorMap* map_out;
    uint8_t* bufs;                // this warp's EPI_BUFS boxes, 1024-byte aligned
    uint64_t* bars;               // this warp's EPI_BUFS barriers
    uint32_t n;
};

// Lane 0 only.  Fetch box `c` of the tile (columns col_base + 32 c .., rows row0 ..) as box number `n`.
__device__ __forceinline__ void epilogue_tma_fetch(const EpilogueTma& e, uint32_t n, int row0, int col) {
    const uint32_t b = n % EPI_BUFS;
    mbar_expect_tx(&e.bars[b], EPI_BOX_BYTES);
    tma_load_2d(e.bufs + (size_t)b * EPI_BOX_BYTES, e.map_res, &e.bars[b], col, row0);
}

// Lane 0, before the accumulator is ready: start the first two boxes of the tile.
__device__ __forceinline__ void epilogue_tma_begin(const EpilogueTma& e, int row0, int col_base) {
    tma_store_wait_read<1>();                                 // the buffers of boxes n and n+1 are no longer being stored from
    epilogue_tma_fetch(e, e.n, row0, col_base);
    epilogue_tma_fetch(e, e.n + 1, row0, col_base + 32);
}

template <int WIDTH, bool FROM_SCRATCH = false>
__device__ __forceinline__ bool drain_accumulator_tma(const Params& p, EpilogueTma& e, const AccSource& acc, int row0,
                                                      int col_base, const float* bias_tile, int lane) {
#pragma unroll 1
    for (int c = 0; c < WIDTH; c += 32) {
        const uint32_t b = e.n % EPI_BUFS;
        uint32_t r[32];
        acc_load_begin<FROM_SCRATCH>(acc, c, r);
        const bool got = __all_sync(0xffffffffu, mbar_wait(&e.bars[b], (e.n / EPI_BUFS) & 1, p.err, 31));
        acc_load_end<FROM_SCRATCH>(acc);
        if (!got) return false;                               // the same answer in every lane of the warp
        // lane = row of the box; its 128 bytes are eight 16-byte pieces, piece j stored at j ^ (row % 8)
        uint8_t* rowp = e.bufs + (size_t)b * EPI_BOX_BYTES + lane * 128;
        const float* bias = p.bias ? bias_tile + c : nullptr;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            float4* cell = (float4*)(rowp + ((q ^ (lane & 7)) << 4));
            float4 x = *cell;
            float t0 = __uint_as_float(r[4 * q]), t1 = __uint_as_float(r[4 * q + 1]);
            float t2 = __uint_as_float(r[4 * q + 2]), t3 = __uint_as_float(r[4 * q + 3]);
            if (bias) { t0 += bias[4 * q]; t1 += bias[4 * q + 1]; t2 += bias[4 * q + 2]; t3 += bias[4 * q + 3]; }
            if (p.act) { t0 = apply_activation(t0, p.act); t1 = apply_activation(t1, p.act); t2 = apply_activation(t2, p.act); t3 = apply_activation(t3, p.act); }
            x.x += t0; x.y += t1; x.z += t2; x.w += t3;
            *cell = x;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(e.map_out, e.bufs + (size_t)b * EPI_BOX_BYTES, col_base + c, row0);
            tma_store_commit();
            if (c + 64 < WIDTH) {
                tma_store_wait_read<1>();                     // the box before this one has left its buffer
                epilogue_tma_fetch(e, e.n + 2, row0, col_base + c + 64);
            }
        }
        __syncwarp();
        ++e.n;
    }
    return true;
}

// ---- many tokens, CTA pairs: 256 x 256 tiles with tcgen05 cta_group::2 -------------------------------
//
// Two CTAs on neighbouring SMs form a cluster and share one MMA: CTA r of the pair holds rows
// r*128.. of the A tile and rows r*128.. of the (256-row) B tile in its own shared memory, and the
// 128 x 256 accumulator of its rows in its own tensor memory.  One thread of CTA 0 issues the MMAs
// for both.  A stage is 32 KB per CTA instead of 48 KB for the same MMA work, so six stages fit
// and each SM takes in a third fewer bytes per FLOP.  Each CTA loads its own tiles with TMA (no
// multicast); loads of both CTAs complete the full-barrier of CTA 0; the MMA thread's commits
// release the stage in both CTAs.  Five stages leave room for the boxes of the TMA epilogue.
constexpr int CSTAGES = 5;
constexpr int PAIR_EPI_BYTES = 4 * EPI_BUFS * EPI_BOX_BYTES;     // 48 KB: three boxes for each epilogue warp

// TMA load into this CTA's shared memory whose bytes are counted on a barrier given by its
// shared::cluster address (CTA 0's barrier).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_h16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__host__ __device__ constexpr uint32_t instr_desc_pair(int n) {      // M = 256 over the pair
    return (1u << 4) | IDESC_H16_AB | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                    const __grid_constant__ CUtensorMap map_res, const __grid_constant__ CUtensorMap map_out,
                    const Params p, int tiles_m, int tiles_n, int tma_epilogue) {
    constexpr int A_BYTES = TILE_P * BLOCK_K * 2;             // 16 KB: this CTA's 128 rows of A
    constexpr int B_BYTES = 128 * BLOCK_K * 2;                // 16 KB: this CTA's 128 rows of the 256-row B tile
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* epi_smem = smem + (size_t)CSTAGES * STAGE_BYTES;  // 1024-byte aligned: the stages are 32 KB
    __shared__ uint64_t full_bar[CSTAGES], empty_bar[CSTAGES], acc_full[2], acc_empty[2], epi_bar[4][EPI_BUFS];
    __shared__ uint32_t tmem_base_smem;
    __shared__ float bias_tile[2][256];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int num_kb = (p.K + BLOCK_K - 1) / BLOCK_K;
    const int n_tiles = tiles_m * tiles_n;                    // 256 x 256 tiles
    // Work of pair g of G.  Tiles [0, dp_tiles) are computed whole, tile g + t * G by pair g.  The
    // last sk_tiles tiles (fewer than G: they would leave pairs idle in a last wave) are laid end to
    // end as sk_tiles * num_kb K blocks and cut into GS equal runs for the first GS pairs (GS is
    // chosen so that a tile has few contributors); a run covers parts of at most two tiles (its
    // "segments"), which come first in the pair's list of items.
    const int G = gridDim.x >> 1, g = blockIdx.x >> 1, GS = p.sk_pairs;
    const int dp_tiles = n_tiles - p.sk_tiles;
    const int my_dp = g < dp_tiles ? (dp_tiles - g + G - 1) / G : 0;
    const long long U = (long long)p.sk_tiles * num_kb;
    const long long u0 = g < GS ? U * g / GS : 0, u1 = g < GS ? U * (g + 1) / GS : 0;
    const int seg_tile0 = (int)(u0 / num_kb);                 // first shared tile this pair touches
    const int n_seg = u1 > u0 ? (int)((u1 - 1) / num_kb) - seg_tile0 + 1 : 0;
    const int n_items = n_seg + my_dp;
    const long long total = (u1 - u0) + (long long)my_dp * num_kb;

    // item i -> tile, K blocks [kb0, kb1)
    auto item_of = [&](int i, int& tile, int& kb0, int& kb1) {
        if (i < n_seg) {
            const int rel = seg_tile0 + i;
            const long long lo = (long long)rel * num_kb, hi = lo + num_kb;
            kb0 = (int)((u0 > lo ? u0 : lo) - lo);
            kb1 = (int)((u1 < hi ? u1 : hi) - lo);
            tile = dp_tiles + rel;
        } else {
            tile = g + (i - n_seg) * G; kb0 = 0; kb1 = num_kb;
        }
    };
    // A walk over the K blocks this pair loads, item after item, without a division per step: the
    // loading thread has a few hundred cycles for each.
    struct Cursor { int item, kb, kb1, x_row, w_row, stage; };
    auto cursor_set = [&](Cursor& c) {
        if (c.item >= n_items) return;
        int tile; item_of(c.item, tile, c.kb, c.kb1);
        c.x_row = (tile % tiles_m) * 256 + (int)rank * 128;
        c.w_row = (tile / tiles_m) * 256 + (int)rank * 128;
    };
    auto cursor_next = [&](Cursor& c) {
        c.stage = c.stage + 1 == CSTAGES ? 0 : c.stage + 1;
        if (++c.kb == c.kb1) { ++c.item; cursor_set(c); }
    };
    // shared::cluster addresses of CTA 0's full barriers (the ones the MMA thread waits on)
    auto full0 = [&](int s) { return map_to_cta(smem_u32(&full_bar[s]), 0); };
    auto load_weights = [&](const Cursor& c) {
        if (leader) mbar_expect_tx(&full_bar[c.stage], 2 * STAGE_BYTES);     // both CTAs' bytes land on this barrier
        tma_load_2d_pair(smem + (size_t)c.stage * STAGE_BYTES + A_BYTES, &map_q, full0(c.stage), c.kb * BLOCK_K, c.w_row);
    };
    auto load_activations = [&](const Cursor& c) {
        tma_load_2d_pair(smem + (size_t)c.stage * STAGE_BYTES, &map_p, full0(c.stage), c.kb * BLOCK_K, c.x_row);
    };

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < CSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }   // 4 warps x 2 CTAs
        for (int w = 0; w < 4; ++w)
            for (int b = 0; b < EPI_BUFS; ++b) mbar_init(&epi_bar[w][b], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_p) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_q) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_smem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                           // both CTAs' barriers exist before anything remote
    tc_fence_after();
    int issued = 0;
    Cursor cw{0, 0, 0, 0, 0, 0};
    if (threadIdx.x == 0) {
        cursor_set(cw);
        for (; issued < total && issued < CSTAGES; ++issued) { load_weights(cw); cursor_next(cw); }   // weights: before the dependency wait
    }
    pdl_wait();
    const uint32_t tmem_base = tmem_base_smem;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            Cursor ca{0, 0, 0, 0, 0, 0};
            cursor_set(ca);
            for (int it = 0; it < issued; ++it) { load_activations(ca); cursor_next(ca); }
            uint32_t ph = 0;                                  // parity of the stages' second use
            for (long long it = issued; it < total && ok; ++it) {
                ok = mbar_wait(&empty_bar[cw.stage], ph, p.err, 21);
                if (!ok) break;
                load_weights(cw);
                load_activations(cw);
                cursor_next(cw);
                if (cw.stage == 0) ph ^= 1;
            }
        }
    } else if (warp == 1) {
        if (leader && lane == 0) {
            constexpr uint32_t idesc = instr_desc_pair(256);
            int mma_stage = 0;
            uint32_t mma_phase = 0;
            for (int t = 0; t < n_items && ok; ++t) {
                const int acc = t & 1;
                const uint32_t acc_ph = (uint32_t)((t >> 1) & 1);
                int tile, kb0, kb1; item_of(t, tile, kb0, kb1);
                ok = mbar_wait(&acc_empty[acc], acc_ph ^ 1, p.err, 22);      // both CTAs drained this accumulator
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * 256);
                for (int kb = kb0; kb < kb1 && ok; ++kb) {
                    const int s = mma_stage;
                    ok = mbar_wait(&full_bar[s], mma_phase, p.err, 23);
                    if (!ok) break;
                    if (++mma_stage == CSTAGES) { mma_stage = 0; mma_phase ^= 1; }
                    const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint64_t adesc = smem_desc_sw128(a_addr);
                    const uint64_t bdesc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                        umma_h16_pair(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(map_to_cta(smem_u32(&empty_bar[s]), 0));    // the stage is free in both CTAs
                    umma_commit_pair(map_to_cta(smem_u32(&empty_bar[s]), 1));
                }
                umma_commit_pair(map_to_cta(smem_u32(&acc_full[acc]), 0));
                umma_commit_pair(map_to_cta(smem_u32(&acc_full[acc]), 1));
            }
        }
    } else {
        const int quad = warp & 3;
        EpilogueTma epi{&map_res, &map_out, epi_smem + (size_t)quad * EPI_BUFS * EPI_BOX_BYTES, epi_bar[quad], 0u};
        constexpr long long HALF_TILE = 256LL * PART_LD;      // floats of one CTA's half of a partial tile
        for (int t = 0; t < n_items && ok; ++t) {
            const int acc = t & 1;
            const uint32_t acc_ph = (uint32_t)((t >> 1) & 1);
            int tile, kb0, kb1; item_of(t, tile, kb0, kb1);
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            const bool whole = kb0 == 0 && kb1 == num_kb;
            if (p.bias) {                                  // this tile's bias -> shared memory (epilogue threads only)
                const int et = threadIdx.x - 64;
                for (int j = et; j < 256; j += 128) bias_tile[acc][j] = (tn * 256 + j < p.rows_q) ? p.bias[tn * 256 + j] : 0.f;
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            const int row0 = tm * 256 + (int)rank * 128 + quad * 32;
            if (whole && tma_epilogue && lane == 0) epilogue_tma_begin(epi, row0, tn * 256);
            ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[acc], acc_ph, p.err, 24));
            if (!ok) break;
            tc_fence_after();
            AccSource src{tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * 256), nullptr, 0, 0, 0};
            if (whole) {
                if (tma_epilogue) ok = drain_accumulator_tma<256>(p, epi, src, row0, tn * 256, bias_tile[acc], lane);
                else drain_accumulator<256>(p, src, row0 + lane, tn * 256, bias_tile[acc]);
                tc_fence_before();
                __syncwarp();
                if (!ok) break;
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
                continue;
            }
            // A segment: this warp's 32 rows of the partial sums -> scratch memory, as item t of pair g.
            float* mine = p.partials + ((long long)(g * 2 + t) * 2 + rank) * HALF_TILE + quad * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < 256; c += 32) {
                uint32_t r[32];
                tmem_ld32(src.tmem_addr + (uint32_t)c, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) __stcg(mine + (size_t)(c + j) * PART_LD, __uint_as_float(r[j]));
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
            // Who else works on this tile: the pairs whose runs hold its first and its last K block.
            const int rel = tile - dp_tiles;
            const long long x0 = (long long)rel * num_kb, x1 = x0 + num_kb - 1;
            const int g_first = (int)(((x0 + 1) * GS - 1) / U), g_last = (int)(((x1 + 1) * GS - 1) / U);
            __threadfence();
            __syncwarp();
            int last = 0;
            if (lane == 0) {
                int* counter = p.counters + (rel * 2 + (int)rank) * 4 + quad;
                last = atomicAdd(counter, 1) == g_last - g_first;
                if (last) *counter = 0;                      // ready for the next call
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (!last) continue;
            // The warp that arrives last adds the partial tiles, first contributor first, and finishes the tile.
            __threadfence();
            const int first_seg = rel - (int)((U * g_first / GS) / num_kb);
            src.part0 = p.partials + ((long long)(g_first * 2) * 2 + rank) * HALF_TILE + quad * 32 + lane;
            src.n_parts = g_last - g_first + 1;
            src.first_off = (long long)first_seg * 2 * HALF_TILE;
            src.stride = 4 * HALF_TILE;
            if (tma_epilogue) {
                if (lane == 0) epilogue_tma_begin(epi, row0, tn * 256);
                ok = drain_accumulator_tma<256, true>(p, epi, src, row0, tn * 256, bias_tile[acc], lane);
            } else {
                drain_accumulator<256, true>(p, src, row0 + lane, tn * 256, bias_tile[acc]);
            }
        }
        if (tma_epilogue && lane == 0) tma_store_wait_read<0>();      // shared memory is read out before the CTA ends
    }
    if (!ok) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 1000000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                           // neither CTA leaves while the other may still reach into it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---- host side ----------------------------------------------------------------------------------
template <int BN, int STAGES, bool SWAP>
int launch(const CUtensorMap& mp, const CUtensorMap& mq, const Params& p, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = (size_t)STAGES * (TILE_P * BLOCK_K * 2 + BN * BLOCK_K * 2) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (p.cluster_reduce)
        return tnx_launch_cluster(1, dim3(1, 1, grid.z), gemm_tc_kernel<BN, STAGES, SWAP>, grid, dim3(NUM_THREADS), smem, stream, mp, mq, p);
    return tnx_launch_ex(1, gemm_tc_kernel<BN, STAGES, SWAP>, grid, dim3(NUM_THREADS), smem, stream, mp, mq, p);
}

}  // namespace

// Many tokens: which kernel, and how many of the paired kernel's tiles are shared out by K blocks.

// Up to this many tokens the swapped form runs (the tokens are the N extent of one MMA tile).
// (Measured at 65..128 tokens against 128 x 128 and 128 x 256 tiles of the many-token kernels: equal
// or faster on every layer product of the 6.7B and 13B sizes, [4096 x 16384] 32 against 50 us.)
static constexpr int FEW_TOKENS_MAX = 128;
static int few_tokens_max() { return FEW_TOKENS_MAX; }
TNX_EXPORT int tnx_gemm_tc_few_tokens() { return few_tokens_max(); }

struct ManyTokensPlan { int kind; int pairs; int sk_tiles; int sk_pairs; int splits; };   // kind 0: 128 x 128 tiles, 1: CTA pairs, 2: persistent, 3: 128 x 256 tiles with K split in clusters
// A plan imposed from outside (-1: the estimates below choose).  0: 128 x 128 tiles; 1: CTA pairs, whole
// tiles; 2: persistent 128 x 256 tiles; 4: CTA pairs with the last wave shared out by K blocks; 31, 32,
// 34, 38: 128 x 256 tiles with K split 1, 2, 4, 8 ways in clusters.  It exists so that a test can time
// every kernel that could run a product and hold the estimates' choice against the best of them.
static int g_forced_plan = -1;
TNX_EXPORT void tnx_gemm_tc_force_plan(int plan) { g_forced_plan = plan; }

static ManyTokensPlan plan_many_tokens(int M, int N, int K, int sms) {
    ManyTokensPlan r{2, 0, 0, 0, 1};
    const int kb = (K + BLOCK_K - 1) / BLOCK_K;
    const int tiles_m = (M + TILE_P - 1) / TILE_P;
    if (g_forced_plan >= 0) {
        const int G = sms / 2, n_tiles = ((M + 255) / 256) * ((N + 255) / 256), rest = n_tiles % G;
        const int sk_pairs = rest * 4 < G ? rest * 4 : G;
        const int tiles_p = tiles_m * ((N + 255) / 256);
        r.kind = -1;                                                // refused unless the sizes allow the plan
        if (g_forced_plan == 0 || g_forced_plan == 2) r.kind = g_forced_plan;
        else if (g_forced_plan == 1) { r.kind = 1; r.pairs = n_tiles < G ? n_tiles : G; }
        else if (g_forced_plan == 4 && rest > 0 && (long long)rest * kb >= 4LL * sk_pairs) {
            r.kind = 1; r.pairs = G; r.sk_tiles = rest; r.sk_pairs = sk_pairs;
        } else if (g_forced_plan > 30 && g_forced_plan <= 30 + MAX_CLUSTER) {
            const int sp = g_forced_plan - 30;
            if ((sp & (sp - 1)) == 0 && tiles_p * sp <= sms && (sp == 1 || sp * 4 <= kb)) { r.kind = 3; r.splits = sp; }
        }
        return r;
    }
    // Estimated times in microseconds, from measurements at 256..2,048 tokens: a K block of a
    // 256 x 256 pair tile takes 0.45 us, of a 128 x 128 single tile 0.38 us; start and drain 8 / 6 us.
    const float t_single = (float)((tiles_m * ((N + 127) / 128) + sms - 1) / sms) * kb * 0.38f + 6.f;
    const int G = sms / 2;
    const int n_tiles = ((M + 255) / 256) * ((N + 255) / 256);          // 256 x 256 tiles of the paired kernel
    const int full = n_tiles / G, rest = n_tiles % G;
    const float t_tile = kb * 0.45f;
    float t_pair = (float)(full + (rest > 0)) * t_tile + 8.f;
    // The tiles of a partly filled last wave (all tiles, when there are fewer than pairs) can be
    // shared out by K blocks over GS pairs, at most four to a tile: that wave then takes rest / GS
    // of a tile's time, but GS + rest partial tiles are written and read again (0.1 us each at the
    // rate the second-level cache gives beside the main loop's loads) and the warp that adds them
    // up needs 2.8 us per contributor, which hides behind a following whole tile if there is one.
    // A margin of 1.3 on these costs; every pair must get at least four K blocks.
    int sk_pairs = rest * 4 < G ? rest * 4 : G;
    float t_share = 1e30f;
    // Measured at 129..2,048 tokens over the layer products of the 6.7B, 13B and 30B sizes and a
    // vocabulary-sized N: sharing out pays where every shared tile is cut into exactly four runs (a pair
    // then holds part of one tile only: 5-32 % faster behind a whole wave, and without one when K is long).
    // With runs that straddle two tiles it pays while the last wave holds at most 0.55 tiles per pair and
    // K is 256 blocks or more (10-35 %; up to 0.75 tiles per pair behind a whole wave), or 100 blocks or
    // more behind a whole wave, 80 behind two (3-16 %); with a fuller last wave or a shorter K it lost
    // 5-40 % against whole tiles in one more wave.
    const bool four_runs = rest * 4 <= G;
    const bool sparse_rest = rest * 100 <= G * 55;
    const bool long_k = kb >= 256 && (full > 0 ? rest * 100 <= G * 75 : sparse_rest);
    const bool behind_waves = sparse_rest && ((full >= 1 && kb >= 100) || (full >= 2 && kb >= 80));
    if (rest > 0 && (long long)rest * kb >= 4LL * sk_pairs && (four_runs || long_k || behind_waves)) {
        const float reduce = ((float)sk_pairs / rest + 1.f) * 2.8f;
        const float exposed = full > 0 ? (reduce > t_tile ? reduce - t_tile : 0.f) : reduce;
        t_share = ((float)full + (float)rest / sk_pairs) * t_tile + 8.f + 1.3f * ((sk_pairs + rest) * 0.1f + exposed);
    }
    if (M < 256) {
        // 129..255 tokens: the weights are streamed once and the tensor cores idle.  Few 128 x 256
        // tiles would leave SMs idle: 128 x 128 tiles, one per CTA, fill the GPU better then;
        // otherwise the single-CTA persistent kernel with 128 x 256 tiles (a K block 0.45 us).  The
        // paired kernel (half of whose 256 token rows may be empty) wins where K is long and the
        // tiles are few, by sharing them out.
        const int tiles_p = tiles_m * ((N + 255) / 256);
        // Few tiles and a long K (the output projections of a layer): 128 x 256 tiles with K split 4 or
        // 8 ways over the CTAs of a cluster, which add up through shared memory like the few-token
        // form does (measured at 129..255 tokens: 22 against 28 us for [4096 x 4096], 44-50 against 60 us
        // for [4096 x 16384]; with more tiles and a split of 2 the kernels below are faster).
        {
            int sp = MAX_CLUSTER;
            while (sp > 1 && (tiles_p * sp > sms || sp * 4 > kb)) sp >>= 1;
            if (sp >= 4) { r.kind = 3; r.splits = sp; return r; }
        }
        const bool single = tiles_p * 4 < sms * 3;
        // In as many waves the persistent kernel is 5-8 % slower than the pairs (measured), so it must win outright.
        const float t_here = single ? t_single : (float)((tiles_p + sms - 1) / sms) * kb * 0.45f * 1.05f + 8.f;
        if (t_here <= t_pair && t_here <= t_share) { r.kind = single ? 0 : 2; return r; }
    } else {
        // 256 tokens and more: where the 128 x 256 tiles fit the GPU in one wave they can split K 1, 2, 4 or
        // 8 ways in clusters as above.  A K block of such a tile takes 0.45 us; start and drain 8 us, the sum
        // over a cluster 2 + splits us (measured at 256..768 tokens: [4096 x 16384] 43 / 69 / 71 us at
        // 256 / 384 / 512 tokens against 63 / 87 / 89 us; [12288 x 4096] 40 against 50 us at 384).  It has to
        // win by a tenth: where the estimates tie, the paired kernel was the faster one.
        const int tiles_p = tiles_m * ((N + 255) / 256);
        int best_sp = 0;
        float t_split = 1e30f;
        for (int sp = 1; sp <= MAX_CLUSTER && tiles_p * sp <= sms && (sp == 1 || sp * 4 <= kb); sp <<= 1) {
            const float t = (float)((kb + sp - 1) / sp) * 0.45f + 8.f + (sp > 1 ? 2.f + (float)sp : 0.f);
            if (t < t_split) { t_split = t; best_sp = sp; }
        }
        // The persistent kernel's 128 x 256 tiles waste less of a last token tile than the pairs' 256 rows
        // (320 tokens: three tiles of 128 against two of 256): where that saves a wave it is 15-25 % faster
        // (measured at 320, 384 and 640 tokens), in as many waves 3-7 % slower.
        const float t_persistent = (float)((tiles_p + sms - 1) / sms) * kb * 0.45f * 1.05f + 8.f;
        const float t_other = fminf(fminf(t_single, t_persistent), fminf(t_pair, t_share));
        if (best_sp > 0 && t_split * 1.1f < t_other) { r.kind = 3; r.splits = best_sp; return r; }
        if (t_single <= t_pair && t_single <= t_share && t_single <= t_persistent) { r.kind = 0; return r; }
        if (t_persistent < t_pair && t_persistent < t_share) { r.kind = 2; return r; }
    }
    r.kind = 1;
    if (t_share < t_pair) { r.pairs = G; r.sk_tiles = rest; r.sk_pairs = sk_pairs; }
    else r.pairs = n_tiles < G ? n_tiles : G;
    return r;
}

// Bytes of 32-bit scratch and number of tile counters that tnx_gemm_tc needs for these sizes (0
// when K is not split).  The caller owns both; the counters must be zero before the first call and
// are left zero by every call.
TNX_EXPORT int tnx_gemm_tc_plan(int M, int N, int K, int n_sms, int* splits, long long* scratch_bytes, int* n_counters) {
    *splits = 1; *scratch_bytes = 0; *n_counters = 0;
    if (M > few_tokens_max()) {
        // paired kernel: two partial 256 x 256 tiles per pair, and a counter per shared tile, CTA and epilogue warp
        const ManyTokensPlan mt = plan_many_tokens(M, N, K, n_sms);
        if (mt.sk_tiles > 0) {
            *scratch_bytes = (long long)mt.pairs * 2 * 256 * 256 * 4;
            *n_counters = mt.sk_tiles * 8;
        }
        return 0;
    }
    // Few tokens: the weight matrix has (N / 128) tiles; K is split 2, 4 or 8 ways, as far as the
    // CTAs still fit on the GPU at once (two to an SM) and every split keeps at least four K blocks.
    // The CTAs of a tile form a cluster and add their partial tiles through shared memory, so no
    // scratch memory is needed.  (Measured on the layer sizes of the 6.7B and 13B models at 8 and
    // 64 tokens: a second round of CTAs, or a cluster of 3, costs more than a coarser split.)
    const int tiles = (N + TILE_P - 1) / TILE_P;
    const int kb = (K + BLOCK_K - 1) / BLOCK_K;
    // Clusters of 4 and 8 do not fill the last places (the CTAs of a cluster lie in one GPC): measured at 8 tokens,
    // 72 and 74 tiles split 4 ways (288 and 296 CTAs for 296 places) took 38 and 21 us where a split of 2 takes 31
    // and 16, while 56 tiles split 4 ways (224) and 32 tiles split 8 ways (256) are the fastest of their kind and
    // 148 tiles split 2 ways (296) still beat no split.  So clusters of 4 and 8 may take nine places in ten.
    int s = MAX_CLUSTER;
    for (; s > 1; s >>= 1) {
        if (s * 4 > kb) continue;
        if (s == 2 ? tiles * s <= 2 * n_sms : tiles * s * 10 <= 2 * n_sms * 9) break;
    }
    *splits = s;
    return 0;
}

TNX_EXPORT int tnx_gemm_tc(const void* A, const void* W, const float* bias, const float* residual, void* C,
                           int M, int N, int K, int lda, int ldw, int ldc, int act, int c_h16,
                           int splits, float* scratch, int* counters, int* err_word, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || lda % 8 || ldw % 8 || lda < K || ldw < K || ldc < N) return TNX_ERR_UNSUPPORTED;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return TNX_ERR_UNSUPPORTED;
    if (residual && c_h16) return TNX_ERR_BAD_ARG;
    if (act < 0 || act >= TNX_ACT_COUNT) return TNX_ERR_BAD_ARG;
    if (!err_word) return TNX_ERR_BAD_ARG;
    Params p{};
    p.K = K; p.ldc = ldc; p.act = act; p.c_is_h16 = c_h16; p.bias = bias; p.residual = residual; p.C = C;
    p.err = err_word; p.partials = scratch; p.counters = counters;
    const int kb = (K + BLOCK_K - 1) / BLOCK_K;
    CUtensorMap mp, mq;
    if (M > few_tokens_max()) {
        p.rows_p = M; p.rows_q = N; p.splits = 1; p.kb_per_split = kb;
        if (!make_map(&mp, A, M, K, lda, TILE_P)) return TNX_ERR_UNSUPPORTED;
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        static int cached_sms[64] = {0};
        if (dev >= 0 && dev < 64) {
            if (!cached_sms[dev]) cudaDeviceGetAttribute(&cached_sms[dev], cudaDevAttrMultiProcessorCount, dev);
            sms = cached_sms[dev];
        }
        const int tiles_m = (M + TILE_P - 1) / TILE_P, tiles_n = (N + PBN - 1) / PBN;
        ManyTokensPlan mt = plan_many_tokens(M, N, K, sms);
        if (mt.kind < 0) return TNX_ERR_UNSUPPORTED;
        if (mt.kind == 0) {
            if (!make_map(&mq, W, N, K, ldw, 128)) return TNX_ERR_UNSUPPORTED;
            dim3 grid((M + TILE_P - 1) / TILE_P, (N + 127) / 128, 1);
            return launch<128, 6, false>(mp, mq, p, grid, stream);
        }
        if (mt.kind == 3) {
            if (!make_map(&mq, W, N, K, ldw, 256)) return TNX_ERR_UNSUPPORTED;
            p.splits = mt.splits; p.kb_per_split = (kb + mt.splits - 1) / mt.splits; p.cluster_reduce = mt.splits > 1;
            dim3 grid((M + TILE_P - 1) / TILE_P, (N + 255) / 256, mt.splits);
            return launch<256, 4, false>(mp, mq, p, grid, stream);
        }
        if (mt.kind == 1) {
            const int ptiles_m = (M + 255) / 256, ptiles_n = (N + 255) / 256;
            if (mt.sk_tiles > 0 && (!scratch || !counters)) {          // no scratch given: whole tiles only
                mt.sk_tiles = 0; mt.sk_pairs = 0;
                if (mt.pairs > ptiles_m * ptiles_n) mt.pairs = ptiles_m * ptiles_n;
            }
            p.sk_tiles = mt.sk_tiles; p.sk_pairs = mt.sk_pairs;
            if (!make_map(&mq, W, N, K, ldw, 128)) return TNX_ERR_UNSUPPORTED;
            constexpr size_t psmem = (size_t)CSTAGES * (TILE_P * BLOCK_K * 2 + 128 * BLOCK_K * 2) + PAIR_EPI_BYTES + 1024;
            // A 32-bit residual goes through TMA boxes when the row pitch and the addresses allow it.
            CUtensorMap mres = mp, mout = mp;
            int tma_epilogue = 0;
            if (residual && !c_h16 && ldc % 4 == 0 && !(((uintptr_t)residual | (uintptr_t)C) & 15))
                tma_epilogue = make_map_f32(&mres, residual, M, N, ldc, 32) && make_map_f32(&mout, C, M, N, ldc, 32);
            static bool pconfigured = false;
            if (!pconfigured) {
                cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)psmem);
                if (e != cudaSuccess) return (int)e;
                pconfigured = true;
            }
            return tnx_launch_ex(1, gemm_tc_pair_kernel, dim3(2 * mt.pairs), dim3(NUM_THREADS), psmem, stream, mp, mq, mres, mout, p,
                                 ptiles_m, ptiles_n, tma_epilogue);
        }
        if (!make_map(&mq, W, N, K, ldw, PBN)) return TNX_ERR_UNSUPPORTED;
        constexpr size_t smem = (size_t)PSTAGES * (TILE_P * BLOCK_K * 2 + PBN * BLOCK_K * 2) + 1024;
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
        const int ctas = tiles_m * tiles_n < sms ? tiles_m * tiles_n : sms;
        return tnx_launch_ex(1, gemm_tc_persistent_kernel, dim3(ctas), dim3(NUM_THREADS), smem, stream, mp, mq, p,
                             tiles_m, tiles_n);
    }
    if (splits < 1) splits = 1;
    // Split K: with scratch memory and counters the CTA that finishes last adds the partial tiles;
    // without them the CTAs of a tile form a cluster (at most 8) and add up through shared memory.
    if (splits > 1 && (!scratch || !counters)) {
        if (splits > MAX_CLUSTER) return TNX_ERR_BAD_ARG;
        p.cluster_reduce = 1;
    }
    p.rows_p = N; p.rows_q = M; p.splits = splits; p.kb_per_split = (kb + splits - 1) / splits;
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    if (!make_map(&mp, W, N, K, ldw, TILE_P) || !make_map(&mq, A, M, K, lda, bn)) return TNX_ERR_UNSUPPORTED;
    dim3 grid((N + TILE_P - 1) / TILE_P, 1, splits);
    // stage counts that let two CTAs share an SM's shared memory
    if (bn == 16) return launch<16, 6, true>(mp, mq, p, grid, stream);
    if (bn == 32) return launch<32, 5, true>(mp, mq, p, grid, stream);
    if (bn == 64) return launch<64, 4, true>(mp, mq, p, grid, stream);
    return launch<128, 3, true>(mp, mq, p, grid, stream);
}

// ---- a wait that runs out, for the tests of the error path --------------------------------------------
// One warp waits, with a limit of `limit_ns`, on an mbarrier at which nothing ever arrives.  The wait
// gives up by itself, the kernel records `code` in the error word and returns: this is what every
// bounded wait of the kernels above does when a copy or a product never completes.
namespace {
__global__ void wait_runs_out_kernel(int* err, int code, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait_limit(&bar, 0, err, code, limit_ns);
}
}  // namespace

TNX_EXPORT int tnx_selftest_wait_runs_out(int* err, int code, long long limit_ns, cudaStream_t stream) {
    if (!err || limit_ns <= 0 || limit_ns > 100000000ll) return TNX_ERR_BAD_ARG;      // 0.1 s at most
    return tnx_launch_in_order(wait_runs_out_kernel, dim3(1), dim3(32), 0, stream, err, code, (unsigned long long)limit_ns);
}

