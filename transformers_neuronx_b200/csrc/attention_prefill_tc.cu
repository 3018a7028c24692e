// Causal attention of prompt portions over the paged 16-bit cache on the 5th-generation tensor
// cores (tcgen05), for head sizes 64, 80, 96, 112 and 128 (described for 128).  Same work items and the
// same result as attention_prefill.cu; this kernel is the fast one.
//
// Work item = (request, tile of 128 of its query rows, head); keys in tiles of 64 (four pages).
//   S = Q K^T   : tcgen05.mma M=128 (queries) N=64 (keys) K=128 (head), Q and K from shared memory
//                 (TMA, 128-byte swizzle, K-major), S in tensor memory (two buffers)
//   softmax     : four warps, one thread per query row: the row of S is read from tensor memory,
//                 masked, exponentiated with the running maximum (32-bit), the row of P written
//                 back to tensor memory as bfloat16, over the scores it came from
//   O += P V    : tcgen05.mma M=128 N=128 (head) K=64 (keys), P read from tensor memory (no trip
//                 through shared memory and its proxy fence); V is the [key][head] tile as it lies
//                 in the cache's pages, i.e. the "MN-major" form of the B operand; O stays in tensor
//                 memory over all key tiles and is rescaled there when the running maximum grows
// Warp 0 issues the TMA loads (two stages of K, three of V, eight lanes a copy each; the page
// numbers of the work item are read into shared memory first), one lane of warp 1 the MMAs of
// O += P V and one lane of warp 6 those of S = Q K^T (the scores of tile j+1 are issued as soon as
// their K tile is there and their buffer free, so that the tensor core works while the softmax
// warps do), warps 2-5 are the softmax warps.  Two CTAs fit on an SM.
// Every wait is bounded and reports through the error word.
//
// The cache's memory must hold finite numbers everywhere (it is allocated zeroed): rows of a page
// that no token has written yet are loaded with their page and multiplied by probabilities that
// are exactly zero.
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int BQ = 128, BKV = 64, PAGE = 16;
constexpr int ATOM_Q = BQ * 128;             // bytes of one 64-column slice of the Q tile (16 KB)
constexpr int ATOM_KV = BKV * 128;           // bytes of one 64-column slice of a K or V tile (8 KB)
constexpr int MAX_PAGES_SMEM = 128;          // page numbers kept in shared memory (2,048 keys); beyond: read from global
// Head size D (64..128 in steps of 16), KS stages of K tiles and VS of V tiles.  A head size between 64
// and 128 uses the layout of 128: its second 64-column slice is partly filled (the TMA box of a K or V
// tile reaches beyond the tensor's last column there and is filled with zeros; that of Q reaches into
// the next head's columns), and the MMAs stop at the head's own columns.  Everything lives in dynamic
// shared memory, the tiles first: with no static shared memory the dynamic part starts at the
// CTA's shared window, which is 1024-byte aligned as the swizzled tiles need (checked at run time).
// D = 128: Q 32 KB + (2 + 3) x 16 KB, so that two CTAs fit on an SM to the byte; D = 64: Q 16 KB +
// (3 + 4) x 8 KB, stages enough to cover the time a tile takes to arrive.
template <int D, int KS, int VS>
struct Layout {
    static constexpr int SLICES = (D + 63) / 64;                 // 64-column slices of a row (the last may be partly used)
    static constexpr int Q_BYTES = SLICES * ATOM_Q, KV_BYTES = SLICES * ATOM_KV;
    static constexpr int TILE_BYTES = Q_BYTES + (KS + VS) * KV_BYTES;
    static constexpr int SMEM_BYTES = TILE_BYTES + 256 + MAX_PAGES_SMEM * 4;
};
constexpr uint32_t TMEM_COLS = 256;          // S0 [0,64) S1 [64,128) O [128,128 + D)
constexpr int THREADS = 224;
constexpr int QK_WARP = 6;
constexpr float RESCALE_STEP = 8.f;          // log2 units: see the softmax warps

struct TcPrefillParams {
    const int* block_tables; int bt_stride;
    const int* tile_req; const int* tile_q0;
    const int* q_start; const int* q_len; const int* ctx_len;
    h16* out; int out_stride;
    int n_heads, n_kv_heads;
    int window;
    float scale_log2;
    int* err;
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// D (+)= A B with A read from tensor memory (lane = row, a column = two consecutive h16 of K).
__device__ __forceinline__ void umma_h16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// B operand given as [K rows][N contiguous] (MN-major), rows 128 bytes, 128-byte swizzle: groups of
// 8 rows (K) are 1024 bytes apart, the next 64 columns (N) `lbo_bytes` further.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t saddr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D = f32, A = B = h16, M = 128, N = n; b_mn: B is MN-major.
__host__ __device__ constexpr uint32_t idesc_attn(int n, int b_mn) {
    return (1u << 4) | IDESC_H16_AB | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

template <int D, int K_STAGES, int V_STAGES>
__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const TcPrefillParams p) {
    using L = Layout<D, K_STAGES, V_STAGES>;
    constexpr int SLICES = L::SLICES, Q_BYTES = L::Q_BYTES, KV_BYTES = L::KV_BYTES, TILE_BYTES = L::TILE_BYTES;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + Q_BYTES;                   // [K_STAGES] K tiles
    uint8_t* sV = sK + K_STAGES * KV_BYTES;       // [V_STAGES] V tiles
    uint64_t* bars = (uint64_t*)(smem + TILE_BYTES);
    uint64_t& q_full = bars[0];
    uint64_t* k_full = bars + 1;                  // [K_STAGES]
    uint64_t* k_empty = k_full + K_STAGES;
    uint64_t* v_full = k_empty + K_STAGES;        // [V_STAGES]
    uint64_t* v_empty = v_full + V_STAGES;
    uint64_t* s_full = v_empty + V_STAGES;        // [2]
    uint64_t* s_empty = s_full + 2;
    uint64_t& p_full = s_empty[2];
    uint64_t& o_full = s_empty[3];
    uint32_t& tmem_base_smem = *(uint32_t*)(s_empty + 4);
    int* pages_s = (int*)(smem + TILE_BYTES + 256);
    if (smem_u32(smem) & 1023u) {                 // cannot happen with no static shared memory; never compute on a wrong layout
        if (threadIdx.x == 0) atomicExch(p.err, 30);
        return;
    }

    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = gridDim.y - 1 - blockIdx.y, h = blockIdx.x;      // heaviest tiles first, of all heads
    const int req = p.tile_req[item], q0 = p.tile_q0[item];
    if (req < 0) return;                                              // a padded work item of a captured step
    const int qs = p.q_start[req], ql = p.q_len[req], ctx = p.ctx_len[req];
    const int rows = min(BQ, ql - q0);
    const int kvh = h / (p.n_heads / p.n_kv_heads);
    const int* bt = p.block_tables + (size_t)req * p.bt_stride;
    const int pos0 = ctx + q0, pos_last = pos0 + rows - 1;
    const int kv_total = ctx + ql;
    int key_begin = 0;
    if (p.window > 0) key_begin = max(0, pos0 - p.window + 1) / BKV * BKV;
    const int n_tiles = (pos_last - key_begin) / BKV + 1;

    // K and V stages start as zeros: pages that do not exist are not loaded, and what a stage holds
    // then must be finite (it is multiplied by probabilities that are zero).
    for (int i = threadIdx.x; i < (K_STAGES + V_STAGES) * KV_BYTES / 16; i += THREADS) ((uint4*)sK)[i] = make_uint4(0, 0, 0, 0);
    const int first_page = key_begin / PAGE;
    const int n_pages = (min(kv_total, key_begin + n_tiles * BKV) - key_begin + PAGE - 1) / PAGE;   // pages that exist
    for (int i = threadIdx.x; i < n_pages && i < MAX_PAGES_SMEM; i += THREADS) pages_s[i] = bt[first_page + i];
    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < K_STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < V_STAGES; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 4); }
        mbar_init(&p_full, 4); mbar_init(&o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_kv) : "memory");
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, TMEM_COLS);
        tmem_relinquish();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the zeros, before TMA writes beside them
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_smem;
    bool ok = true;

    if (warp == 0) {
        // ---- TMA producer ---------------------------------------------------------------------------
        // A tile is up to eight copies of 2 KB (four pages x the 64-column slices of the head).  One thread issuing
        // sixteen of them per key tile was the slowest part of the kernel, so eight lanes issue one
        // copy each; lane 0 waits for the stage and announces the bytes.
        if (lane == 0) {
            mbar_expect_tx(&q_full, Q_BYTES);
#pragma unroll
            for (int sl = 0; sl < SLICES; ++sl) tma_load_2d(sQ + sl * ATOM_Q, &map_q, &q_full, h * D + sl * 64, qs + q0);
        }
        const int g = (lane >> 1) & 3, a = lane & 1;          // this lane's page of the tile and half of the head
        // the page this lane copies for key tile j (-1 where the context ends before), and how many pages exist
        auto tile_page = [&](int j, int& n_valid) {
            const int first = j * 4;
            n_valid = min(4, max(0, n_pages - first));
            const int i = first + g;
            return i < n_pages ? (i < MAX_PAGES_SMEM ? pages_s[i] : bt[first_page + i]) : -1;
        };
        auto load_tile = [&](int j, int which, uint8_t* stage, uint64_t* full, uint64_t* empty, uint32_t parity, int code) {
            int n_valid;
            const int page = tile_page(j, n_valid);
            // Only pages that are copied are announced: behind a sliding window the first tile may
            // begin with blocks that were given back already (-1 in the block table); their part of
            // the stage keeps finite numbers, and the window masks those keys.
            n_valid = __popc(__ballot_sync(0xffffffffu, lane < 8 && a == 0 && page >= 0));
            int good = 1;
            if (lane == 0) {
                good = mbar_wait(empty, parity, p.err, code) ? 1 : 0;
                if (good) mbar_expect_tx(full, (uint32_t)(n_valid * SLICES * PAGE * 128));
            }
            good = __shfl_sync(0xffffffffu, good, 0);
            if (good && lane < 8 && a < SLICES && page >= 0) {
                const int row = ((page * 2 + which) * p.n_kv_heads + kvh) * PAGE;
                tma_load_2d(stage + a * ATOM_KV + g * PAGE * 128, &map_kv, full, a * 64, row);
            }
            return good != 0;
        };
        auto load_k = [&](int j) {
            const int ks = j % K_STAGES;                     // last used by tile j - K_STAGES
            return load_tile(j, 0, sK + ks * KV_BYTES, &k_full[ks], &k_empty[ks], (uint32_t)(((j / K_STAGES) & 1) ^ 1), 31);
        };
        auto load_v = [&](int j) {
            const int vs = j % V_STAGES;
            return load_tile(j, 1, sV + vs * KV_BYTES, &v_full[vs], &v_empty[vs], (uint32_t)(((j / V_STAGES) & 1) ^ 1), 40);
        };
        // Keys run K_STAGES tiles ahead of the values: the scores of a tile are wanted a whole
        // softmax earlier than its values, and a K stage is free as soon as its scores are done.
        for (int j = 0; j < K_STAGES && j < n_tiles && ok; ++j) ok = load_k(j);
        for (int j = 0; j < n_tiles && ok; ++j) {
            ok = load_v(j);
            if (ok && j + K_STAGES < n_tiles) ok = load_k(j + K_STAGES);
        }
    } else if (warp == 1) {
        // ---- MMA issuer of O += P V ---------------------------------------------------------------------
        // (The scores have an issuing thread of their own, warp 6: one thread issuing the twelve MMAs
        // and four commits of a key tile was the slowest part of the kernel.)
        if (lane == 0) {
            constexpr uint32_t idesc_pv = idesc_attn(D, 1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                ok = mbar_wait(&p_full, (uint32_t)(j & 1), p.err, 36);
                if (ok) ok = mbar_wait(&v_full[j % V_STAGES], (uint32_t)((j / V_STAGES) & 1), p.err, 41);
                if (!ok) break;
                tc_fence_after();
                const uint32_t p_tmem = tmem_base + (uint32_t)((j & 1) * BKV);         // P lies over the scores it came from
                const uint32_t v_addr = smem_u32(sV + (j % V_STAGES) * KV_BYTES);
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    // 16 keys further: 8 columns of P (two h16 each), 16 rows of V
                    const uint64_t bdesc = smem_desc_sw128_mn(v_addr + k * 16 * 128, ATOM_KV);
                    umma_h16_a_tmem(tmem_base + 128, p_tmem + (uint32_t)(k * 8), bdesc, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&o_full);
                umma_commit(&v_empty[j % V_STAGES]);          // the V tile is free, and so is P's place in the score buffer
            }
        }
    } else if (warp == QK_WARP) {
        // ---- MMA issuer of S = Q K^T ----------------------------------------------------------------------
        // Tile n goes to score buffer n & 1, which must be free twice over: the softmax warps have
        // read the scores of tile n - 2 (s_empty), and P V of tile n - 2, whose P lay in the same
        // columns, has finished (v_empty of that tile's V stage; its next completion is P V of tile
        // n + 1, which cannot come before these scores).
        if (lane == 0) {
            constexpr uint32_t idesc_qk = idesc_attn(BKV, 0);
            const uint32_t q_addr = smem_u32(sQ);
            ok = mbar_wait(&q_full, 0, p.err, 32);
            for (int n = 0; n < n_tiles && ok; ++n) {
                ok = mbar_wait(&k_full[n % K_STAGES], (uint32_t)((n / K_STAGES) & 1), p.err, 33);
                if (ok) ok = mbar_wait(&s_empty[n & 1], (uint32_t)(((n >> 1) & 1) ^ 1), p.err, 35);
                if (ok && n >= 2) ok = mbar_wait(&v_empty[(n - 2) % V_STAGES], (uint32_t)(((n - 2) / V_STAGES) & 1), p.err, 34);
                if (!ok) break;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sK + (n % K_STAGES) * KV_BYTES);
                const uint32_t d_tmem = tmem_base + (uint32_t)((n & 1) * BKV);
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint64_t adesc = smem_desc_sw128(q_addr + (k >> 2) * ATOM_Q + (k & 3) * 32);
                    const uint64_t bdesc = smem_desc_sw128(k_addr + (k >> 2) * ATOM_KV + (k & 3) * 32);
                    umma_h16(d_tmem, adesc, bdesc, idesc_qk, k > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[n & 1]);
                umma_commit(&k_empty[n % K_STAGES]);          // the K tile is free once these MMAs have read it
            }
        }
    } else {
        // ---- softmax warps: thread = query row ----------------------------------------------------------
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        const int qpos = pos0 + r;
        float m_run = -INFINITY, l_run = 0.f;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int b = j & 1;
            const int k0 = key_begin + j * BKV;
            ok = mbar_wait(&s_full[b], (uint32_t)((j >> 1) & 1), p.err, 37);
            if (!ok) break;
            tc_fence_after();
            uint32_t raw0[32], raw1[32];
            tmem_ld32(lane_base + (uint32_t)(b * BKV), raw0);
            tmem_ld32(lane_base + (uint32_t)(b * BKV + 32), raw1);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[b]);             // the scores are in registers
            float s[64];
#pragma unroll
            for (int i = 0; i < 32; ++i) { s[i] = __uint_as_float(raw0[i]); s[32 + i] = __uint_as_float(raw1[i]); }
            bool need_mask = k0 + BKV - 1 > qpos;
            if (p.window > 0) need_mask = need_mask || (k0 <= qpos - p.window);
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int key = k0 + i;
                    bool keep = key <= qpos;
                    if (p.window > 0) keep = keep && key > qpos - p.window;
                    if (!keep) s[i] = -INFINITY;
                }
            }
            // the row's maximum and sum as four chains each: no instruction waits for the one before it
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], s[i]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // The reference the exponentials are taken against moves up only when the maximum has
            // grown by more than 2^RESCALE_STEP: until then P holds values up to 2^RESCALE_STEP
            // instead of 1, which 32-bit sums and bfloat16 products carry as well, and O (which a
            // move of the reference has to rescale in tensor memory) is left alone.
            const float mx_scaled = (mx == -INFINITY) ? -INFINITY : mx * p.scale_log2;
            const bool grow = mx_scaled > m_run + RESCALE_STEP;            // m_run: the reference, in log2 units
            const float m_new = grow ? mx_scaled : m_run;
            const float m_scaled = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = (!grow || m_run == -INFINITY) ? (grow ? 0.f : 1.f) : ex2_approx(m_run - m_new);
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t packed[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float p0 = ex2_approx(fmaf(s[2 * i], p.scale_log2, -m_scaled));
                const float p1 = ex2_approx(fmaf(s[2 * i + 1], p.scale_log2, -m_scaled));
                sum4[i & 3] += p0 + p1;
                h16x2 h2 = floats_to_h16x2(p0, p1);
                packed[i] = *(uint32_t*)&h2;
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            l_run = l_run * corr + sum;
            m_run = m_new;
            if (j > 0) {
                // P V of the tile before has finished: its O is complete and the P buffer is free
                ok = mbar_wait(&o_full, (uint32_t)((j - 1) & 1), p.err, 38);
                if (!ok) break;
                tc_fence_after();
                if (!__all_sync(0xffffffffu, corr == 1.f)) {     // the maximum of some row grew: rescale O
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + 128u + (uint32_t)c, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tmem_st32(lane_base + 128u + (uint32_t)c, o);
                    }
                    tmem_st_wait();
                }
            }
            // this row of P -> tensor memory, over the first half of the scores it came from (which
            // are in registers): 64 bfloat16 in 32 columns.  The MMA warp issues P V of this tile
            // before the scores of tile j + 2 (which go to this buffer), and the tensor core works
            // in the order of issue.
            tmem_st32(lane_base + (uint32_t)(b * BKV), packed);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full);
        }
        if (ok) ok = mbar_wait(&o_full, (uint32_t)((n_tiles - 1) & 1), p.err, 39);
        if (ok) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            h16* orow = p.out + (size_t)(qs + q0 + r) * p.out_stride + (size_t)h * D;
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                uint32_t o[32];
                tmem_ld32(lane_base + 128u + (uint32_t)c, o);
                tmem_ld_wait();
                if (r < rows) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (c + 8 * q >= D) break;                // the last 32 columns of a head size like 80 are partly beyond it
                        uint4 u;
                        h16x2 h0 = floats_to_h16x2(__uint_as_float(o[8 * q]) * inv, __uint_as_float(o[8 * q + 1]) * inv);
                        h16x2 h1 = floats_to_h16x2(__uint_as_float(o[8 * q + 2]) * inv, __uint_as_float(o[8 * q + 3]) * inv);
                        h16x2 h2 = floats_to_h16x2(__uint_as_float(o[8 * q + 4]) * inv, __uint_as_float(o[8 * q + 5]) * inv);
                        h16x2 h3 = floats_to_h16x2(__uint_as_float(o[8 * q + 6]) * inv, __uint_as_float(o[8 * q + 7]) * inv);
                        u.x = *(uint32_t*)&h0; u.y = *(uint32_t*)&h1; u.z = *(uint32_t*)&h2; u.w = *(uint32_t*)&h3;
                        *(uint4*)(orow + c + 8 * q) = u;
                    }
                }
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
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int D, int KS, int VS>
int launch_tc(const CUtensorMap& mq, const CUtensorMap& mkv, const TcPrefillParams& p, int n_heads, int n_items, cudaStream_t stream) {
    constexpr int smem = Layout<D, KS, VS>::SMEM_BYTES;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<D, KS, VS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return tnx_launch_in_order(attention_prefill_tc_kernel<D, KS, VS>, dim3(n_heads, n_items), dim3(THREADS), smem, stream, mq, mkv, p);   // heads vary fastest
}

}  // namespace

// Same arguments as tnx_attention_prefill plus the error word; head_dim must be 64, 80, 96, 112 or 128 and
// n_rows_q is the number of rows of the q / out buffers (for the TMA descriptor).
TNX_EXPORT int tnx_attention_prefill_tc(const void* q, int q_stride, int n_rows_q, const void* cache, long long cache_rows,
                                        const int* block_tables, int bt_stride, const int* tile_req, const int* tile_q0,
                                        const int* q_start, const int* q_len, const int* ctx_len, void* out,
                                        int out_stride, int n_items, int n_heads, int n_kv_heads, int head_dim,
                                        int page_size, int window, float scale, int* err_word, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (head_dim < 64 || head_dim > 128 || head_dim % 16 || page_size != PAGE || n_kv_heads <= 0 || n_heads % n_kv_heads || q_stride % 8 ||
        out_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15) || ((uintptr_t)out & 15) ||
        cache_rows > 0x7fffffffLL || !err_word)
        return TNX_ERR_UNSUPPORTED;
    CUtensorMap mq, mkv;
    if (!make_map(&mq, q, n_rows_q, n_heads * head_dim, q_stride, BQ)) return TNX_ERR_UNSUPPORTED;
    if (!make_map(&mkv, cache, (int)cache_rows, head_dim, head_dim, PAGE)) return TNX_ERR_UNSUPPORTED;
    TcPrefillParams p;
    p.block_tables = block_tables; p.bt_stride = bt_stride; p.tile_req = tile_req; p.tile_q0 = tile_q0;
    p.q_start = q_start; p.q_len = q_len; p.ctx_len = ctx_len; p.out = (h16*)out; p.out_stride = out_stride;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
    p.err = err_word;
    switch (head_dim) {
        case 128: return launch_tc<128, 2, 3>(mq, mkv, p, n_heads, n_items, stream);
        case 112: return launch_tc<112, 2, 3>(mq, mkv, p, n_heads, n_items, stream);
        case 96: return launch_tc<96, 2, 3>(mq, mkv, p, n_heads, n_items, stream);
        case 80: return launch_tc<80, 2, 3>(mq, mkv, p, n_heads, n_items, stream);
        default: return launch_tc<64, 3, 4>(mq, mkv, p, n_heads, n_items, stream);
    }
}
