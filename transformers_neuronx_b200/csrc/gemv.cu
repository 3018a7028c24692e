// Matrix product for one to four tokens (the decode step of one to four requests):
//
//   C[m, n] = epilogue( sum_k A[m, k] * W[n, k] )        A: [M, K] h16, W: [N, K] h16, row-major
//   epilogue: + bias[n] (32-bit); activation (by code, common.cuh); + residual[m, n] (32-bit); stored in the 16-bit type or as float.
//
// With so few tokens the product is a stream of the weight matrix through the multiply-add units:
// there is nothing for the tensor cores to win, and plain 16-byte loads keep more bytes in flight
// per SM than the TMA path of the tensor-core kernel does.  A block of 128 or 256 threads holds the
// tokens' activations in shared memory and walks over groups of R weight rows; thread t takes the
// 16-byte pieces t, t + threads, ... of each row, with the loads of the next step (or of the next group
// of rows) issued before the current pieces are used.  Blocks share the rows out evenly.  Sums are 32-bit; the order of the additions
// depends only on K, never on M or on the other tokens, so a token's result is the same alone and
// beside others.  The weights are read before the kernel ahead has finished (they are never
// written by a kernel); the activations after.
//
// The activations can also be given as rows of the 32-bit residual stream with a LayerNorm to apply
// (tnx_gemv_ln): every block then normalizes the rows itself as it fills its shared memory (three
// walks over a row that lies in the second-level cache: mean, variance of the formula, the affine),
// and the LayerNorm kernel, its launch and the trip of its output through memory are not needed.
// With one token that is 2 us a product, a twentieth of the step.
#include "common.cuh"

namespace {

struct LnArgs { const float* x; int ldx; const float* gamma; const float* beta; float eps; };


__device__ __forceinline__ uint4 load_stream(const uint4* p) { return __ldcs(p); }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
#ifdef TNX_F16
    const h16x2* h = (const h16x2*)&v;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = h16x2_to_float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
#else
    // a bfloat16 is the upper half of the float with the same value
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
#endif
}

template <int M, int R, int THREADS>
__global__ void __launch_bounds__(THREADS)
gemv_kernel(const h16* __restrict__ A, int lda, const h16* __restrict__ W, int ldw,
            const float* __restrict__ bias, const float* residual, void* C, int ldc,
            int act, int c_is_h16, int N, int K, const LnArgs ln) {
    extern __shared__ uint4 xs[];                         // [M][K / 8] pieces of the activations
    __shared__ float red[THREADS / 32][R * M];
    __shared__ float lnred[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K8 = K >> 3;
    // This block's rows: an equal share of the N rows (to within one row), taken R at a time; the
    // last group of a block may be shorter.
    const int row_begin = (int)((long long)N * blockIdx.x / gridDim.x);
    const int row_end = (int)((long long)N * (blockIdx.x + 1) / gridDim.x);

    auto fetch = [&](uint4 (&dst)[R], int row0, int p) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (row0 + r < row_end) dst[r] = load_stream((const uint4*)(W + (size_t)(row0 + r) * ldw) + p);
            else dst[r] = make_uint4(0u, 0u, 0u, 0u);
        }
    };

    pdl_launch_dependents();
    uint4 cur[R];
    if (row_begin < row_end && tid < K8) fetch(cur, row_begin, tid);
    pdl_wait();                                           // from here on the activations may be read, and C written
    if (ln.x == nullptr) {
        for (int i = tid; i < M * K8; i += THREADS) {
            const int m = i / K8, p = i - m * K8;
            xs[i] = *((const uint4*)(A + (size_t)m * lda) + p);
        }
    } else {
        // y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * gamma + beta, all in 32-bit (layernorm.cu).
        // The row is read from memory once and kept in shared memory (behind the activations' pieces)
        // for the two further walks.
        float4* rowf = (float4*)(xs + M * K8);
        // The scale and the shift of this thread's first EARLY pieces are asked for together with the row, so that
        // they are not one more round trip to the second-level cache behind the statistics.
        constexpr int EARLY = 4;
        float4 ga[EARLY][2], be[EARLY][2];
#pragma unroll
        for (int i = 0; i < EARLY; ++i) {
            const int p = tid + i * THREADS;
            const bool in = p < K8;
            ga[i][0] = (ln.gamma && in) ? __ldg((const float4*)ln.gamma + 2 * p) : make_float4(1.f, 1.f, 1.f, 1.f);
            ga[i][1] = (ln.gamma && in) ? __ldg((const float4*)ln.gamma + 2 * p + 1) : make_float4(1.f, 1.f, 1.f, 1.f);
            be[i][0] = (ln.beta && in) ? __ldg((const float4*)ln.beta + 2 * p) : make_float4(0.f, 0.f, 0.f, 0.f);
            be[i][1] = (ln.beta && in) ? __ldg((const float4*)ln.beta + 2 * p + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll 1
        for (int m = 0; m < M; ++m) {
            const float4* src = (const float4*)(ln.x + (size_t)m * ln.ldx);
            if (m > 0) __syncthreads();                   // the row before is done with
            float sum = 0.f;
            for (int p = tid; p < K8; p += THREADS) {
                const float4 a = src[2 * p], b = src[2 * p + 1];
                rowf[2 * p] = a; rowf[2 * p + 1] = b;
                sum += ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
            }
            const float mean = block_sum(sum, lnred) / (float)K;
            float q = 0.f;
            for (int p = tid; p < K8; p += THREADS) {     // a thread walks the pieces it wrote itself
                const float4 a = rowf[2 * p], b = rowf[2 * p + 1];
                const float d0 = a.x - mean, d1 = a.y - mean, d2 = a.z - mean, d3 = a.w - mean;
                const float d4 = b.x - mean, d5 = b.y - mean, d6 = b.z - mean, d7 = b.w - mean;
                q += ((d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3)) + ((d4 * d4 + d5 * d5) + (d6 * d6 + d7 * d7));
            }
            const float rstd = 1.0f / sqrtf(block_sum(q, lnred) / (float)K + ln.eps);
            auto finish_piece = [&](int p, const float4& g0, const float4& g1, const float4& b0, const float4& b1) {
                const float4 a = rowf[2 * p], b = rowf[2 * p + 1];
                float y[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = (y[e] - mean) * rstd;
                y[0] = y[0] * g0.x + b0.x; y[1] = y[1] * g0.y + b0.y; y[2] = y[2] * g0.z + b0.z; y[3] = y[3] * g0.w + b0.w;
                y[4] = y[4] * g1.x + b1.x; y[5] = y[5] * g1.y + b1.y; y[6] = y[6] * g1.z + b1.z; y[7] = y[7] * g1.w + b1.w;
                h16x2 h0 = floats_to_h16x2(y[0], y[1]), h1 = floats_to_h16x2(y[2], y[3]);
                h16x2 h2 = floats_to_h16x2(y[4], y[5]), h3 = floats_to_h16x2(y[6], y[7]);
                uint4 u;
                u.x = *(uint32_t*)&h0; u.y = *(uint32_t*)&h1; u.z = *(uint32_t*)&h2; u.w = *(uint32_t*)&h3;
                xs[m * K8 + p] = u;
            };
#pragma unroll
            for (int i = 0; i < EARLY; ++i) {
                const int p = tid + i * THREADS;
                if (p < K8) finish_piece(p, ga[i][0], ga[i][1], be[i][0], be[i][1]);
            }
            for (int p = tid + EARLY * THREADS; p < K8; p += THREADS) {       // rows longer than the early pieces cover
                const float4 one = make_float4(1.f, 1.f, 1.f, 1.f), zero = make_float4(0.f, 0.f, 0.f, 0.f);
                finish_piece(p, ln.gamma ? ((const float4*)ln.gamma)[2 * p] : one, ln.gamma ? ((const float4*)ln.gamma)[2 * p + 1] : one,
                             ln.beta ? ((const float4*)ln.beta)[2 * p] : zero, ln.beta ? ((const float4*)ln.beta)[2 * p + 1] : zero);
            }
        }
    }
    __syncthreads();

    for (int row0 = row_begin; row0 < row_end; row0 += R) {
        float acc[R][M];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
        // What the threads that finish the rows need from memory is asked for before the walk over K, not after it
        // (where the whole block would wait for the round trip).
        float early_bias = 0.f, early_res = 0.f;
        if (tid < R * M) {
            const int r = tid / M, m = tid - r * M;
            const int n = row0 + r;
            if (n < row_end) {
                if (bias) early_bias = __ldg(bias + n);
                if (residual) early_res = residual[(size_t)m * ldc + n];
            }
        }
        for (int p = tid; p < K8; p += THREADS) {
            uint4 nxt[R];
            const int pn = p + THREADS;
            if (pn < K8) fetch(nxt, row0, pn);
            else if (row0 + R < row_end) fetch(nxt, row0 + R, tid);
            float xf[M][8];
#pragma unroll
            for (int m = 0; m < M; ++m) unpack8(xs[m * K8 + p], xf[m]);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float wf[8];
                unpack8(cur[r], wf);
#pragma unroll
                for (int m = 0; m < M; ++m)
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[r][m] = fmaf(wf[e], xf[m][e], acc[r][m]);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) cur[r] = nxt[r];
        }
        // the block's sum: lanes, then warps, in a fixed order
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float v = warp_sum(acc[r][m]);
                if (lane == 0) red[warp][r * M + m] = v;
            }
        __syncthreads();
        if (tid < R * M) {
            const int r = tid / M, m = tid - r * M;
            const int n = row0 + r;
            if (n < row_end) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < THREADS / 32; ++w) v += red[w][tid];
                v += early_bias;
                v = apply_activation(v, act);
                const size_t o = (size_t)m * ldc + n;
                v += early_res;
                if (c_is_h16) ((h16*)C)[o] = float_to_h16(v);
                else ((float*)C)[o] = v;
            }
        }
        __syncthreads();
    }
}

template <int M, int R, int THREADS>
int launch(const h16* A, int lda, const h16* W, int ldw, const float* bias, const float* residual, void* C, int ldc,
           int act, int c_h16, int N, int K, int sms, const LnArgs& ln, cudaStream_t stream) {
    const size_t smem = (size_t)M * K * 2 + (ln.x ? (size_t)K * 4 : 0);          // with a LayerNorm: one 32-bit row beside the activations
    static size_t configured = 48 * 1024 - 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<M, R, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    // blocks per SM for the shared-memory sizes asked about last (a model's products alternate between a few)
    static size_t asked_smem[4] = {~(size_t)0, ~(size_t)0, ~(size_t)0, ~(size_t)0};
    static int asked_per_sm[4] = {0, 0, 0, 0};
    static int asked_next = 0;
    int per_sm = -1;
    for (int i = 0; i < 4; ++i)
        if (asked_smem[i] == smem) per_sm = asked_per_sm[i];
    if (per_sm < 0) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemv_kernel<M, R, THREADS>, THREADS, smem);
        if (e != cudaSuccess) return (int)e;
        asked_smem[asked_next] = smem; asked_per_sm[asked_next] = n; asked_next = (asked_next + 1) & 3;
        per_sm = n;
    }
    if (per_sm < 1) return TNX_ERR_UNSUPPORTED;
    int blocks = sms * per_sm;
    if (blocks > (N + R - 1) / R) blocks = (N + R - 1) / R;
    return tnx_launch_ex(1, gemv_kernel<M, R, THREADS>, dim3(blocks), dim3(THREADS), smem, stream, A, lda, W, ldw, bias, residual, C, ldc,
                         act, c_h16, N, K, ln);
}

}  // namespace

// Whether tnx_gemv takes these sizes: one to four tokens, K a multiple of 8, the activations of
// all tokens within the shared memory of a block (and of several blocks per SM for 3 or 4 tokens).
// It is the faster kernel for one token; with two it is level with the tensor-core kernel and with
// three and four the multiply-adds, not the memory, set its pace (measured).
TNX_EXPORT int tnx_gemv_supported(int M, int N, int K) {
    if (M < 1 || M > 4 || N < 1 || K < 8 || K % 8) return 0;
    const long long smem = (long long)M * K * 2;
    return smem <= (M <= 2 ? 112 * 1024 : 64 * 1024);
}

static int gemv_any(const void* A, const void* W, const float* bias, const float* residual, void* C,
                    int M, int N, int K, int lda, int ldw, int ldc, int act, int c_h16, const LnArgs& ln, cudaStream_t stream) {
    if (!tnx_gemv_supported(M, N, K)) return TNX_ERR_UNSUPPORTED;
    if (ldw % 8 || ldw < K || ldc < N || ((uintptr_t)W & 15)) return TNX_ERR_UNSUPPORTED;
    if (ln.x) {
        if (ln.ldx % 4 || ln.ldx < K || ((uintptr_t)ln.x & 15)) return TNX_ERR_UNSUPPORTED;
        if ((ln.gamma && ((uintptr_t)ln.gamma & 15)) || (ln.beta && ((uintptr_t)ln.beta & 15))) return TNX_ERR_UNSUPPORTED;
        if ((long long)M * K * 2 + (long long)K * 4 > 112 * 1024) return TNX_ERR_UNSUPPORTED;
    } else if (lda % 8 || lda < K || ((uintptr_t)A & 15)) {
        return TNX_ERR_UNSUPPORTED;
    }
    if (residual && c_h16) return TNX_ERR_BAD_ARG;
    if (act < 0 || act >= TNX_ACT_COUNT) return TNX_ERR_BAD_ARG;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    static int cached_sms[64] = {0};
    if (dev >= 0 && dev < 64) {
        if (!cached_sms[dev]) cudaDeviceGetAttribute(&cached_sms[dev], cudaDevAttrMultiProcessorCount, dev);
        sms = cached_sms[dev];
    }
    const h16* a = (const h16*)A;
    const h16* w = (const h16*)W;
    // Rows of up to 4,096 elements: blocks of 128 threads (four steps of a row instead of two between
    // the block-wide sums); longer rows: 256 threads.  The choice depends on K alone, so that the
    // order of the additions does not depend on the number of tokens.
#define GEMV_LAUNCH(M_, R_)                                                                                              \
    (K <= 4096 ? launch<M_, R_, 128>(a, lda, w, ldw, bias, residual, C, ldc, act, c_h16, N, K, sms, ln, stream)       \
               : launch<M_, R_, 256>(a, lda, w, ldw, bias, residual, C, ldc, act, c_h16, N, K, sms, ln, stream))
    switch (M) {
        case 1: return GEMV_LAUNCH(1, 8);
        case 2: return GEMV_LAUNCH(2, 8);
        case 3: return GEMV_LAUNCH(3, 4);
        default: return GEMV_LAUNCH(4, 4);
    }
#undef GEMV_LAUNCH
}

TNX_EXPORT int tnx_gemv(const void* A, const void* W, const float* bias, const float* residual, void* C,
                        int M, int N, int K, int lda, int ldw, int ldc, int act, int c_h16, cudaStream_t stream) {
    return gemv_any(A, W, bias, residual, C, M, N, K, lda, ldw, ldc, act, c_h16, LnArgs{nullptr, 0, nullptr, nullptr, 0.f}, stream);
}

// The same product with A = LayerNorm(x): x [M, K] 32-bit rows (pitch ldx elements), gamma and beta
// [K] 32-bit or null.
TNX_EXPORT int tnx_gemv_ln(const float* x, int ldx, const float* gamma, const float* beta, float eps, const void* W,
                           const float* bias, const float* residual, void* C, int M, int N, int K, int ldw, int ldc,
                           int act, int c_h16, cudaStream_t stream) {
    if (!x) return TNX_ERR_BAD_ARG;
    return gemv_any(nullptr, W, bias, residual, C, M, N, K, 0, ldw, ldc, act, c_h16, LnArgs{x, ldx, gamma, beta, eps}, stream);
}
