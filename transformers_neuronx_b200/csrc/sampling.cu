// Next-token choice from 32-bit logits, one cluster of thread blocks per row (1, 2, 4 or 8 blocks, as
// many as keep all rows on the GPU at once: a row of 50,272 logits is walked up to fifteen times, and
// with few rows one block per row would leave most of the GPU idle).  A block owns a contiguous
// slice of the row; histograms and sums are added up across the cluster through distributed shared
// memory, and since all of them are integers the result does not depend on the cluster's size.
//
//   temperature <= 0 : argmax, the lowest index winning a tie.
//   temperature  > 0 : s_i = logit_i / temperature (the suppressed id, if any, at -inf);
//                      top-k: keep the k largest s_i; top-p: of those, keep the most likely tokens
//                      until their probability reaches top_p (a token is kept when the mass
//                      before it is < top_p); then draw from softmax over the kept tokens by
//                      inverse CDF in index order with one Philox uniform per (seed, counter).
//
// A row's parameters come either from one array per parameter (null: the default) or packed, 16
// 32-bit words a row (ROW_WORDS below), which is how the engine sends them: in the same buffer
// and the same copy as the step's other index arrays.  Up to four ids per row can be suppressed
// (a request's end-of-sequence ids), and the fixed draw is a per-row flag.
//
// Everything that decides the outcome is integer arithmetic: the thresholds are found by radix
// selection on order-preserving integer keys, and probability masses are summed as 2^-40
// fixed-point integers, so a draw depends on (logits, parameters, seed, counter) alone and not
// on the order in which threads run.  Tokens tied with the k-th largest are all kept.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;
constexpr int GROUPS = 8;                    // copies of the mass histogram: four warps share one
// The 64-bit mass histogram of the top-p passes is kept in GROUPS copies that are added up after
// a pass: nearly all tokens of a row fall into a few bins of the keys' top byte, and 1,024 threads
// adding into the same few shared-memory words was most of this kernel's time (0.7 ms a call).

__device__ __forceinline__ uint32_t ordered_key(float v) {
    uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
        const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += W0; k1 += W1;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// exp(s - mx) as a 2^-40 fixed-point integer.  The product with 2^40 is exact in 32-bit (a change of
// the exponent), so this is the value a 64-bit computation would truncate to as well.
// A score that is NaN, or -inf where every score is, has no mass (the conversion of a NaN is not zero).
__device__ __forceinline__ unsigned long long mass_of(float s, float mx) {
    const float e = expf(s - mx);
    return e == e ? __float2ull_rz(e * 1099511627776.0f) : 0ull;
}

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

// TOP_P false: the caller passes no top_p array; the kernel then does without the copies of the
// mass histogram (shared memory that would otherwise be taken from the first-level cache).
// Packed parameters of a row: word 0 temperature (float), 1 top_k, 2 top_p (float), 3 min_keep,
// 4-5 seed (low, high), 6-7 counter (low, high), 8 flags (bit 0: the fixed draw), 9-12 suppressed
// ids (-1: none), 13-15 zero.
constexpr int ROW_WORDS = 16;

struct SampleArgs {
    const float* temperature; const int* top_k; const float* top_p; const int* min_keep;
    const unsigned long long* seeds; const unsigned long long* counters;
    int deterministic, suppress_id;
    const int* packed;               // [rows][ROW_WORDS], or null: the arrays above
    const int* err_word;             // when given, out[rows] receives its value (the kernels' error word
    int n_rows;                      //   travels to the host with the sampled ids)
};

__device__ __forceinline__ uint32_t cluster_map(const void* smem_ptr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(smem_ptr)), "r"(rank));
    return r;
}
__device__ __forceinline__ unsigned long long cluster_ld_u64(uint32_t addr) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Grid (rows, blocks a row), clusters of (1, blocks a row): the rows on the axis that has no limit worth the name.
template <bool TOP_P>
__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, const SampleArgs a, int* __restrict__ out) {
    __shared__ unsigned long long warp_hist64[TOP_P ? GROUPS * 256 : THREADS];
    unsigned long long* sums = warp_hist64;                      // [THREADS], used after the histogram passes
    static_assert(GROUPS * 256 >= THREADS, "the partial sums of the last phase reuse the histogram copies");
    __shared__ float fscratch[32];
    __shared__ ArgMax ascratch[32];
    __shared__ unsigned int chist[256];
    __shared__ unsigned long long mhist[256];
    // What a block hands to the others of its cluster: two buffers used in turn, so that a block may fill
    // the next one while a slower block still reads the last (one cluster barrier per exchange).
    __shared__ unsigned long long xbuf[2][256];
    __shared__ unsigned int sh_prefix, sh_remaining;
    __shared__ unsigned long long sh_above, sh_total;
    pdl_launch_dependents();
    pdl_wait();

    const int r = blockIdx.x, tid = threadIdx.x;
    const int CS = gridDim.y, rank = blockIdx.y;
    const int slice = (V + CS - 1) / CS;
    const int v_lo = min(V, rank * slice), v_hi = min(V, v_lo + slice);          // this block's tokens
    int xp = 0;                                                  // exchanges so far (the same in every block)
    const float* row = logits + (size_t)r * ld;
    if (a.err_word && r == 0 && rank == 0 && tid == 0) out[a.n_rows] = *a.err_word;
    // After xbuf[xp & 1][0 .. n) has been written by every block: the values of all blocks, combined by `op`,
    // in every thread that asks (index i < n).
    auto exchange_ready = [&]() { __syncthreads(); if (CS > 1) cluster_sync_all(); };
    auto gather_sum = [&](int i) -> unsigned long long {
        unsigned long long t = 0;
        for (int rk = 0; rk < CS; ++rk) t += cluster_ld_u64(cluster_map(&xbuf[xp & 1][i], (uint32_t)rk));
        return t;
    };
    // No block may leave while another may still read its shared memory.
    auto leave = [&]() { if (CS > 1) cluster_sync_all(); };
    float T, P;
    int k, n_min, deterministic, sup0, sup1 = -1, sup2 = -1, sup3 = -1;
    unsigned long long seed, ctr;
    if (a.packed) {
        const int* w = a.packed + (size_t)r * ROW_WORDS;
        T = __int_as_float(w[0]); k = w[1]; P = __int_as_float(w[2]); n_min = w[3];
        seed = (unsigned long long)(unsigned)w[4] | ((unsigned long long)(unsigned)w[5] << 32);
        ctr = (unsigned long long)(unsigned)w[6] | ((unsigned long long)(unsigned)w[7] << 32);
        deterministic = w[8] & 1;
        sup0 = w[9]; sup1 = w[10]; sup2 = w[11]; sup3 = w[12];
    } else {
        T = a.temperature ? a.temperature[r] : 0.f;
        k = a.top_k ? a.top_k[r] : 0;
        P = a.top_p ? a.top_p[r] : 1.f;
        n_min = a.min_keep ? a.min_keep[r] : 1;
        seed = a.seeds ? a.seeds[r] : 0ull;
        ctr = a.counters ? a.counters[r] : 0ull;
        deterministic = a.deterministic;
        sup0 = a.suppress_id;
    }
#define SUPPRESSED(i) ((i) == sup0 || (i) == sup1 || (i) == sup2 || (i) == sup3)

    if (!(T > 0.f)) {
        ArgMax best{-INFINITY, 0x7fffffff};
        for (int i = v_lo + tid; i < v_hi; i += THREADS) best = better(best, ArgMax{SUPPRESSED(i) ? -INFINITY : row[i], i});
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        if ((tid & 31) == 0) ascratch[tid >> 5] = best;
        __syncthreads();
        if (tid < 32) {
            best = ascratch[tid];
            for (int o = 16; o > 0; o >>= 1) {
                ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
                best = better(best, other);
            }
            if (tid == 0) xbuf[0][0] = ((unsigned long long)__float_as_uint(best.v) << 32) | (unsigned)best.i;
        }
        exchange_ready();
        if (rank == 0 && tid == 0) {
            for (int rk = 1; rk < CS; ++rk) {
                const unsigned long long o = cluster_ld_u64(cluster_map(&xbuf[0][0], (uint32_t)rk));
                best = better(best, ArgMax{__uint_as_float((unsigned)(o >> 32)), (int)(unsigned)o});
            }
            out[r] = best.i == 0x7fffffff ? 0 : best.i;
        }
        leave();
        return;
    }

#define SCORE(i) (SUPPRESSED(i) ? -INFINITY : row[(i)] / T)
    float mx = -INFINITY;
    for (int i = v_lo + tid; i < v_hi; i += THREADS) mx = fmaxf(mx, SCORE(i));
    mx = block_max(mx, fscratch);
    if (CS > 1) {
        if (tid == 0) xbuf[xp & 1][0] = __float_as_uint(mx);
        exchange_ready();
        for (int rk = 0; rk < CS; ++rk)
            mx = fmaxf(mx, __uint_as_float((unsigned)cluster_ld_u64(cluster_map(&xbuf[xp & 1][0], (uint32_t)rk))));
        ++xp;
    }

    // The key of the k-th largest score, by radix selection on the keys' four bytes (1 <= k < V).
    auto kth_largest_key = [&](int k) -> uint32_t {
        __syncthreads();
        if (tid == 0) { sh_prefix = 0; sh_remaining = (unsigned)k; }
        uint32_t mask = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) chist[tid] = 0;
            __syncthreads();
            const uint32_t prefix = sh_prefix;
            for (int i = v_lo + tid; i < v_hi; i += THREADS) {
                const uint32_t key = ordered_key(SCORE(i));
                if ((key & mask) == prefix) atomicAdd(&chist[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (CS > 1) {                                          // the counts of the whole row
                if (tid < 256) xbuf[xp & 1][tid] = chist[tid];
                exchange_ready();
                if (tid < 256) chist[tid] = (unsigned)gather_sum(tid);
                ++xp;
                __syncthreads();
            }
            if (tid < 32) {
                // The highest digit b with count(digits >= b) >= remaining (0 if none): lane l looks at
                // digits 8 l .. 8 l + 7, the counts of the lanes above it come from a suffix sum.
                const unsigned remaining = sh_remaining;
                unsigned v[8], tot = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) { v[j] = chist[tid * 8 + j]; tot += v[j]; }
                unsigned incl = tot;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned nb = __shfl_down_sync(0xffffffffu, incl, o);
                    if (tid + o < 32) incl += nb;
                }
                unsigned cum = incl - tot;                 // tokens with digits in the lanes above
                int b_found = -1;
                unsigned cum_found = 0;
#pragma unroll
                for (int j = 7; j >= 0; --j) {
                    const int b = tid * 8 + j;
                    if (b_found < 0 && (cum + v[j] >= remaining || b == 0)) { b_found = b; cum_found = cum; }
                    cum += v[j];
                }
                const unsigned who = __ballot_sync(0xffffffffu, b_found >= 0);     // lane 0 always answers
                const int src = 31 - __clz(who);
                const int b = __shfl_sync(0xffffffffu, b_found, src);
                const unsigned cum_b = __shfl_sync(0xffffffffu, cum_found, src);
                if (tid == 0) {
                    sh_remaining = remaining - cum_b;
                    sh_prefix = prefix | ((uint32_t)b << shift);
                }
            }
            mask |= 255u << shift;
            __syncthreads();
        }
        return sh_prefix;
    };

    // Of the tokens with keys >= floor_key, taken from the most likely down: the lowest key that is
    // still kept when a token is kept as long as the mass of all keys above its own is < limit.
    auto lowest_key_within_mass = [&](unsigned long long limit, uint32_t floor_key) -> uint32_t {
        __syncthreads();
        if (tid == 0) { sh_prefix = 0; sh_above = 0; }
        uint32_t mask = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int j = tid; j < GROUPS * 256; j += THREADS) warp_hist64[j] = 0;
            __syncthreads();
            const uint32_t prefix = sh_prefix;
            unsigned long long* mine64 = warp_hist64 + (tid >> 5) % GROUPS * 256;
            for (int i = v_lo + tid; i < v_hi; i += THREADS) {
                const float s = SCORE(i);
                const uint32_t key = ordered_key(s);
                if (key >= floor_key && (key & mask) == prefix) atomicAdd(&mine64[(key >> shift) & 255u], mass_of(s, mx));
            }
            __syncthreads();
            if (tid < 256) {
                unsigned long long c = 0;
                for (int w = 0; w < GROUPS; ++w) c += warp_hist64[w * 256 + tid];
                mhist[tid] = c;
                if (CS > 1) xbuf[xp & 1][tid] = c;
            }
            if (CS > 1) {                                          // the masses of the whole row
                exchange_ready();
                if (tid < 256) mhist[tid] = gather_sum(tid);
                ++xp;
            }
            __syncthreads();
            if (tid < 32) {
                // The lowest digit whose tokens may still be kept: the lowest b with
                // (mass above the prefix) + mass(digits > b) < limit, or 255 if there is none.
                unsigned long long v[8], tot = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) { v[j] = mhist[tid * 8 + j]; tot += v[j]; }
                unsigned long long incl = tot;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned long long nb = __shfl_down_sync(0xffffffffu, incl, o);
                    if (tid + o < 32) incl += nb;
                }
                unsigned long long above = sh_above + (incl - tot);      // mass above this lane's highest digit
                int b_found = -1;
                unsigned long long above_found = 0;
#pragma unroll
                for (int j = 7; j >= 0; --j) {
                    const int b = tid * 8 + j;
                    if (above < limit || b == 255) { b_found = b; above_found = above; }     // keeps the lowest
                    above += v[j];
                }
                const unsigned who = __ballot_sync(0xffffffffu, b_found >= 0);     // lane 31 always answers
                const int src = __ffs(who) - 1;
                const int chosen = __shfl_sync(0xffffffffu, b_found, src);
                const unsigned long long chosen_above = __shfl_sync(0xffffffffu, above_found, src);
                if (tid == 0) {
                    sh_above = chosen_above;
                    sh_prefix = prefix | ((uint32_t)chosen << shift);
                }
            }
            mask |= 255u << shift;
            __syncthreads();
        }
        return sh_prefix;
    };

    // The mass of all tokens with keys >= floor_key.
    auto mass_from = [&](uint32_t floor_key) -> unsigned long long {
        unsigned long long local = 0;
        for (int i = v_lo + tid; i < v_hi; i += THREADS) {
            const float s = SCORE(i);
            if (ordered_key(s) >= floor_key) local += mass_of(s, mx);
        }
        __syncthreads();
        if (tid == 0) sh_total = 0;
        __syncthreads();
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if ((tid & 31) == 0) atomicAdd(&sh_total, local);
        __syncthreads();
        if (CS == 1) return sh_total;
        if (tid == 0) xbuf[xp & 1][0] = sh_total;
        exchange_ready();
        const unsigned long long all = gather_sum(0);
        ++xp;
        return all;
    };

    // ---- top-k: the key of the k-th largest score (0 keeps everything) ----------------------
    uint32_t thr = 0;
    if (k > 0 && k < V) thr = kth_largest_key(k);

    // ---- top-p over the tokens that top-k kept, but never fewer than min_keep of them ----------
    if (TOP_P && P < 1.f) {
        unsigned long long limit = (unsigned long long)((double)P * (double)mass_from(thr));
        if (limit < 1) limit = 1;                      // the most likely token is always kept
        uint32_t thr_p = lowest_key_within_mass(limit, thr);
        if (n_min > 1) {
            const uint32_t thr_n = n_min < V ? kth_largest_key(n_min) : 0u;
            if (thr_n < thr_p) thr_p = thr_n;
        }
        if (thr_p > thr) thr = thr_p;
    }

    // ---- the reference's fixed draw (its uniform replaced by 0.5): the kept tokens from the most
    // likely down, the first at which the summed probability reaches one half; the lowest index of a tie
    if (TOP_P && deterministic) {
        const unsigned long long total = mass_from(thr);
        if (total == 0) { if (rank == 0 && tid == 0) out[r] = 0; leave(); return; }
        const uint32_t key = lowest_key_within_mass((total + 1) / 2, thr);
        int first = 0x7fffffff;
        for (int i = v_lo + tid; i < v_hi; i += THREADS)
            if (ordered_key(SCORE(i)) == key) { first = i; break; }
        for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
        __syncthreads();
        if ((tid & 31) == 0) ascratch[tid >> 5].i = first;
        __syncthreads();
        if (tid < 32) {
            first = ascratch[tid].i;
            for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
            if (tid == 0) xbuf[xp & 1][0] = (unsigned)first;
        }
        exchange_ready();
        if (rank == 0 && tid == 0) {
            for (int rk = 1; rk < CS; ++rk) first = min(first, (int)(unsigned)cluster_ld_u64(cluster_map(&xbuf[xp & 1][0], (uint32_t)rk)));
            out[r] = first == 0x7fffffff ? 0 : first;
        }
        leave();
        return;
    }

    // ---- inverse CDF in index order over the kept tokens --------------------------------------
    // A thread owns a contiguous run of its block's slice, so that thread and block order is index order.
    const int chunk = (v_hi - v_lo + THREADS - 1) / THREADS;
    const int lo = min(v_hi, v_lo + tid * chunk), hi = min(v_hi, lo + chunk);
    unsigned long long local = 0;
    for (int i = lo; i < hi; ++i) {
        const float s = SCORE(i);
        if (ordered_key(s) >= thr) local += mass_of(s, mx);
    }
    __syncthreads();                                  // the histogram copies are done with: `sums` lies over them
    sums[tid] = local;
    __syncthreads();
    if (tid < 32) {                                   // exclusive scan of 1024 partial sums
        unsigned long long run = 0;
        const int base = tid * 32;
        for (int j = 0; j < 32; ++j) { unsigned long long v = sums[base + j]; sums[base + j] = run; run += v; }
        unsigned long long incl = run;
        for (int o = 1; o < 32; o <<= 1) {
            unsigned long long nb = __shfl_up_sync(0xffffffffu, incl, o);
            if (tid >= o) incl += nb;
        }
        const unsigned long long excl = incl - run;
        for (int j = 0; j < 32; ++j) sums[base + j] += excl;
        if (tid == 31) { sh_total = incl; xbuf[xp & 1][0] = incl; }
    }
    exchange_ready();
    unsigned long long before = 0, total = 0;         // the mass of the blocks before this one, and of the row
    if (CS > 1) {
        for (int rk = 0; rk < CS; ++rk) {
            const unsigned long long t = cluster_ld_u64(cluster_map(&xbuf[xp & 1][0], (uint32_t)rk));
            if (rk < rank) before += t;
            total += t;
        }
    } else {
        total = sh_total;
    }
    uint32_t rnd[4];
    philox4x32_10((uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), rnd);
    // target = floor(total * u), u = rnd / 2^32 in [0, 1)
    const unsigned long long target = __umul64hi(total, (unsigned long long)rnd[0] << 32);
    const unsigned long long mine = before + sums[tid];
    if (local > 0 && target >= mine && target < mine + local) {       // exactly one thread of the cluster, if total > 0
        unsigned long long run = mine;
        int pick = lo;
        for (int i = lo; i < hi; ++i) {
            const float s = SCORE(i);
            if (ordered_key(s) >= thr) {
                run += mass_of(s, mx);
                pick = i;
                if (run > target) break;
            }
        }
        out[r] = pick;
    }
    if (total == 0 && rank == 0 && tid == 0) out[r] = 0;               // every score was -inf or NaN
    leave();
#undef SCORE
#undef SUPPRESSED
}
// Blocks a row: 8, 4 or 2 while all rows' blocks fit the GPU at once and a block keeps at least 2,048
// tokens of the row (measured at 8 rows of 50,272 logits: one block a row took 12 us for the argmax and
// 209 us with temperature and top-p).
int g_forced_blocks = 0;                   // a test's own number of blocks a row (0: the rule below)
int blocks_per_row(int n_rows, int V) {
    if (g_forced_blocks > 0) return g_forced_blocks;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 1;
    }
    // (Clusters of 8 and 4 find room on half of the SMs only: 16 rows took 107 us with 8 blocks each, 82 with 4.)
    for (int c = 8; c > 1; c >>= 1)
        if ((long long)n_rows * c * (c > 2 ? 2 : 1) <= sms && V >= c * 2048) return c;
    return 1;
}

int launch_sample(bool with_top_p, int n_rows, int V, cudaStream_t stream, const float* logits, int ld, const SampleArgs& a, int* out) {
    const int c = blocks_per_row(n_rows, V);
    if (with_top_p)
        return tnx_launch_cluster(0, dim3(1, c), sample_kernel<true>, dim3(n_rows, c), dim3(THREADS), 0, stream, logits, ld, V, a, out);
    return tnx_launch_cluster(0, dim3(1, c), sample_kernel<false>, dim3(n_rows, c), dim3(THREADS), 0, stream, logits, ld, V, a, out);
}

}  // namespace

// min_keep (per row, may be null: 1): top-p never keeps fewer tokens than this.  deterministic: the
// draw's uniform number is replaced by one half and the tokens are taken from the most likely down.
TNX_EXPORT int tnx_sample(const float* logits, int ld, int n_rows, int V, const float* temperature,
                          const int* top_k, const float* top_p, const int* min_keep, int deterministic,
                          const unsigned long long* seeds, const unsigned long long* counters, int suppress_id,
                          int* out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0 || ld < V) return TNX_ERR_BAD_ARG;
    SampleArgs a = {temperature, top_k, top_p, min_keep, seeds, counters, deterministic, suppress_id, nullptr, nullptr, n_rows};
    return launch_sample(top_p || deterministic, n_rows, V, stream, logits, ld, a, out);
}

// The same with every row's parameters packed (ROW_WORDS 32-bit words a row, see above).  with_top_p: 0
// when no row uses top-p or the fixed draw (the lighter kernel variant).  err_word (may be null): a
// device word copied to out[n_rows], so `out` then holds n_rows + 1 entries.
TNX_EXPORT int tnx_sample_packed(const float* logits, int ld, int n_rows, int V, const int* packed, int with_top_p,
                                 const int* err_word, int* out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0 || ld < V || !packed) return TNX_ERR_BAD_ARG;
    SampleArgs a = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, -1, packed, err_word, n_rows};
    return launch_sample(with_top_p != 0, n_rows, V, stream, logits, ld, a, out);
}

TNX_EXPORT int tnx_sample_row_words() { return ROW_WORDS; }

// For tests: 1, 2, 4 or 8 blocks a row whatever the sizes (0: the library's own rule again).  The drawn
// tokens must not depend on it.
TNX_EXPORT int tnx_sample_force_blocks_per_row(int blocks) {
    if (blocks != 0 && blocks != 1 && blocks != 2 && blocks != 4 && blocks != 8) return TNX_ERR_BAD_ARG;
    g_forced_blocks = blocks;
    return 0;
}
