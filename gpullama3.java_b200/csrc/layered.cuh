// layered.cuh -- device kernels of "layered" plans: models described by a LIST of layers (each with its own mixer sizes and
// feed-forward) instead of one repeated block, with BF16 weights and a 32-bit residual stream.  First user: Pibidra.
//
// Mechanisms, each with its constants as kernel arguments so other designs can pick them up:
//   * k_norm_rows       sandwich norm: x += N(y; w_post), optional pass prologue (x += x0, x += step), out = N(x; w_pre),
//                       N(v; w) = v / sqrt(mean(v^2) + eps) * (w_off + w); also the embedding gather (x = scale * E[token], optionally
//                       normalised); with post_plain the sublayer output is added as x += y * w_post (a layer scale behind a pre-norm);
//   * k_matvec_bf16     decode projection: BF16 weight rows streamed with 128-bit loads, FP32 activation and accumulator,
//                       bias or gated-activation epilogue (gelu_tanh(g) * u);
//   * k_gemm_f32 / k_gemm_bf16   prefill projections for any M, N, K: true FP32 on the CUDA cores, or BF16 operands on the
//                       tensor cores (mma.sync m16n8k16, FP32 accumulation), same epilogues;
//   * k_qk_prep         whole-projection RMS norm of q and of k (one statistic over ALL heads), K / V rows into the window ring;
//   * k_window_attention  sliding-window attention over a ring cache with a soft logit cap, a learned bucketed distance bias
//                       and a softmax whose denominator carries an extra exp(0) (a value-less sink), sigmoid output gate.
// The projection kernels take optional operand VIEWS (MvView / GemmView): a row stride for A, per-head batches, grouped rows for a
// mixture of experts, an input scale and a sigmoid-gate epilogue; the attention kernels take row strides for the key and value
// caches, so one cached row can serve as key and value (latent attention, latent.cuh).
// Everything the residual, the norms and the softmax touch is FP32; explicit fmaf keeps fused multiply-adds although the
// translation unit is compiled with -fmad=false for the bit-exact GGUF kernels.
#pragma once
#include "common.cuh"
#include <cuda_bf16.h>

namespace ly {

typedef __nv_bfloat16 bf16;

enum { EPI_STORE = 0, EPI_GATED = 1, EPI_ACT = 2 }; // C = A W^T (+ bias)  |  H = act(A Wg^T) * (A Wu^T), W = [Wg; Wu] stacked by rows  |  H = act(A W^T (+ bias))
enum { ACT_GELU_TANH = 0, ACT_SILU = 1, ACT_RELU = 2, ACT_GELU_ERF = 3 };

__device__ __forceinline__ float bf_lo(unsigned v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(unsigned v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ float act_apply(int act, float z) {
    if (act == ACT_SILU) return z / (1.0f + expf(-z));
    if (act == ACT_RELU) return fmaxf(z, 0.0f);
    if (act == ACT_GELU_ERF) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f)); // the exact GELU: z * Phi(z)
    // tanh form of GELU: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
    const float u = 0.7978845608028654f * fmaf(0.044715f * z * z, z, z);
    return 0.5f * z * (1.0f + tanhf(u));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Every thread of the block gets the total; red holds 32 floats.  blockDim.x is a multiple of 32.
__device__ __forceinline__ float block_sum(float v, float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads(); // red may still be read from a previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.0f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    return t;
}

// ---------------------------------------------------------------------------------------------------------------------
// Sandwich norm over rows.  One CTA per row; the row lives in shared memory between the passes.
// ---------------------------------------------------------------------------------------------------------------------
struct NormArgs {
    float *x;            // [n][E] residual stream
    float *x0;           // [n][E] embedding output kept for the loop passes (nullable)
    const float *y;      // [n][E] sublayer output: x += N(y; w_post) (nullable)
    const float *w_post; // [E]
    const bf16 *emb;     // embedding table [vocab][E]: x = emb_scale * emb[token] (nullable)
    const int *tokens;   // [n] (nullable: the step's own token)
    const StepState *st;
    float emb_scale;
    int add_x0;          // pass prologue: x += x0
    const float *step;   // pass prologue: x += step (nullable)
    const float *w_pre;  // [E]: out = N(x; w_pre) (nullable)
    float *out32;        // [n][E] (one of out32 / out16, or none)
    bf16 *out16;
    const int *gather;   // output row r is computed from x row gather[r] (only with y == emb == nullptr)
    float *trace;        // [n][E]: copy of x after the post-norm part (nullable)
    float eps;
    int E;
    float w_off;         // added to every norm weight: 1 for weights stored as a deviation from one, 0 for weights used as stored
    int post_plain;      // 1: x += y * w_post (no statistic of y: a layer scale)
    const float *w_emb;  // [E] (nullable): the gathered embedding row is normalised, x = N(scale * emb[token]; w_emb)
};
#define LY_NORM_THREADS 256

__global__ void __launch_bounds__(LY_NORM_THREADS) k_norm_rows(NormArgs a) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[32];
    const int r = blockIdx.x, tid = threadIdx.x, E = a.E;
    const size_t src = (size_t)(a.gather ? a.gather[r] : r) * E, dst = (size_t)r * E;
    if (a.emb) {
        const int token = a.tokens ? a.tokens[r] : a.st->token;
        const bf16 *e = a.emb + (size_t)token * E;
        for (int i = tid; i < E; i += LY_NORM_THREADS) {
            const float v = __bfloat162float(e[i]) * a.emb_scale;
            row[i] = v;
            if (a.x0) a.x0[src + i] = v;
        }
        if (a.w_emb) {
            __syncthreads();
            float ss = 0.0f;
            for (int i = tid; i < E; i += LY_NORM_THREADS) ss = fmaf(row[i], row[i], ss);
            ss = block_sum(ss, red);
            const float inv = 1.0f / sqrtf(ss / (float)E + a.eps);
            for (int i = tid; i < E; i += LY_NORM_THREADS) {
                const float v = row[i] * inv * (a.w_off + a.w_emb[i]);
                row[i] = v;
                if (a.x0) a.x0[src + i] = v;
            }
        }
    } else {
        for (int i = tid; i < E; i += LY_NORM_THREADS) row[i] = a.x[src + i];
    }
    if (a.y && a.post_plain) {
        for (int i = tid; i < E; i += LY_NORM_THREADS) row[i] = fmaf(a.y[src + i], a.w_post[i], row[i]);
    } else if (a.y) {
        float ss = 0.0f;
        for (int i = tid; i < E; i += LY_NORM_THREADS) { const float v = a.y[src + i]; ss = fmaf(v, v, ss); }
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)E + a.eps);
        for (int i = tid; i < E; i += LY_NORM_THREADS) row[i] += a.y[src + i] * inv * (a.w_off + a.w_post[i]);
    }
    if (a.trace)
        for (int i = tid; i < E; i += LY_NORM_THREADS) a.trace[src + i] = row[i];
    if (a.add_x0)
        for (int i = tid; i < E; i += LY_NORM_THREADS) row[i] += a.x0[src + i];
    if (a.step)
        for (int i = tid; i < E; i += LY_NORM_THREADS) row[i] += a.step[i];
    if (!a.gather && (a.emb || a.y || a.add_x0 || a.step))
        for (int i = tid; i < E; i += LY_NORM_THREADS) a.x[src + i] = row[i];
    if (a.w_pre) {
        float ss = 0.0f;
        for (int i = tid; i < E; i += LY_NORM_THREADS) ss = fmaf(row[i], row[i], ss);
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)E + a.eps);
        for (int i = tid; i < E; i += LY_NORM_THREADS) {
            const float v = row[i] * inv * (a.w_off + a.w_pre[i]);
            if (a.out32) a.out32[dst + i] = v;
            if (a.out16) a.out16[dst + i] = __float2bfloat16_rn(v);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Decode projection y = W x (+ bias) or h = act(Wg x) * (Wu x): one warp per output row, the activation staged once per
// CTA in shared memory, weights streamed with 128-bit non-allocating loads.  W is [N][K] BF16 (EPI_GATED: [2N][K], gate rows
// first).  K % 8 == 0 takes the vector path, anything else the scalar one.
// ---------------------------------------------------------------------------------------------------------------------
#define LY_MV_THREADS 256

__device__ __forceinline__ float dot_row_bf16(const bf16 *__restrict__ w, const float *xs, int K, int lane, bool vec) {
    float acc = 0.0f;
    if (vec) {
        for (int k = lane * 8; k < K; k += 256) {
            const int4 q = ldg128_stream(w + k);
            const float4 x0 = *reinterpret_cast<const float4 *>(xs + k), x1 = *reinterpret_cast<const float4 *>(xs + k + 4);
            acc = fmaf(bf_lo((unsigned)q.x), x0.x, acc); acc = fmaf(bf_hi((unsigned)q.x), x0.y, acc);
            acc = fmaf(bf_lo((unsigned)q.y), x0.z, acc); acc = fmaf(bf_hi((unsigned)q.y), x0.w, acc);
            acc = fmaf(bf_lo((unsigned)q.z), x1.x, acc); acc = fmaf(bf_hi((unsigned)q.z), x1.y, acc);
            acc = fmaf(bf_lo((unsigned)q.w), x1.z, acc); acc = fmaf(bf_hi((unsigned)q.w), x1.w, acc);
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(__bfloat162float(w[k]), xs[k], acc);
    }
    return warp_sum(acc);
}

// Optional second grid dimension of a decode projection: blockIdx.y = b selects a per-head operand (offsets b * w_bs / x_bs /
// y_bs into W, x, y) and, with `group`, the weight matrix of expert group[b] (offset group[b] * w_gs).  in_scale[b] multiplies
// the INPUT of a gated projection (act(s g) * (s u)); mul multiplies a stored result by sigmoid(mul[b * y_bs + n]).
struct MvView {
    long long w_bs, x_bs, y_bs;
    const int *group;
    long long w_gs;
    const float *in_scale;
    const float *mul;
    int n_groups; // > 0: a CTA whose group[b] >= n_groups has nothing to do (an expert without weights: the identity)
};

template <int EPI>
__global__ void __launch_bounds__(LY_MV_THREADS) k_matvec_bf16(const bf16 *__restrict__ W, const float *__restrict__ bias, const float *__restrict__ x,
                                                              float *__restrict__ y, int N, int K, int act, MvView v_) {
    extern __shared__ __align__(16) float xs[];
    const int b = blockIdx.y;
    if (v_.group && v_.n_groups > 0 && v_.group[b] >= v_.n_groups) return;
    W += (size_t)b * v_.w_bs + (v_.group ? (size_t)v_.group[b] * v_.w_gs : (size_t)0);
    x += (size_t)b * v_.x_bs;
    y += (size_t)b * v_.y_bs;
    const float sc = v_.in_scale ? v_.in_scale[b] : 1.0f;
    for (int i = threadIdx.x; i < K; i += LY_MV_THREADS) xs[i] = x[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool vec = (K & 7) == 0 && (((size_t)W) & 15) == 0;
    for (int n = blockIdx.x * (LY_MV_THREADS / 32) + warp; n < N; n += gridDim.x * (LY_MV_THREADS / 32)) {
        float v = dot_row_bf16(W + (size_t)n * K, xs, K, lane, vec);
        if (EPI == EPI_GATED) {
            const float u = dot_row_bf16(W + (size_t)(N + n) * K, xs, K, lane, vec);
            v = act_apply(act, v * sc) * (u * sc);
        } else if (EPI == EPI_ACT) {
            if (bias) v += bias[n];
            v = act_apply(act, v);
        } else {
            if (bias) v += bias[n];
            if (v_.mul) v *= 1.0f / (1.0f + expf(-v_.mul[(size_t)b * v_.y_bs + n]));
        }
        if (lane == 0) y[n] = v;
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Views of a prefill projection's operands, shared by the FP32 and the tensor-core kernel.  All optional (zero = plain GEMM):
//   * lda: row stride of A when A is a column block of a wider buffer;
//   * blockIdx.z batches (per-head products): column offset z * a_bs into an A row, element offset z * w_bs into W, column
//     offset z * c_bs into a C row;
//   * grouped rows (mixture of experts): blockIdx.y is a TILE of at most 64 entries of `perm`, a list of slots sorted by
//     group; tile t belongs to group tile_group[t] (-1: nothing to do) whose weight matrix starts at tile_group[t] * w_gs,
//     and covers perm[tile_row0[t] .. + tile_rows[t]).  A slot s reads A row s / a_div and writes C row s.  in_scale[s]
//     multiplies the INPUT of a gated projection: act(sc g) * (sc u);
//   * mul: a stored result is multiplied by sigmoid(mul[row][z * c_bs + n]) (an output gate).
// ---------------------------------------------------------------------------------------------------------------------
struct GemmView {
    int lda;
    long long a_bs, w_bs, c_bs;
    const int *tile_group, *tile_row0, *tile_rows, *perm;
    int a_div;
    long long w_gs;
    const float *in_scale;
    const float *mul;
    int ldmul;
};

// Fills the A / C row numbers of this CTA's 64 rows (-1: outside); returns false when the tile has no work.
__device__ __forceinline__ bool gemm_rows(const GemmView &g, int M, int *s_arow, int *s_crow, int tid, int nthreads) {
    if (g.tile_group) {
        const int t = blockIdx.y;
        if (g.tile_group[t] < 0) return false;
        const int r0 = g.tile_row0[t], nr = g.tile_rows[t];
        for (int r = tid; r < 64; r += nthreads) {
            const int slot = r < nr ? g.perm[r0 + r] : -1;
            s_crow[r] = slot;
            s_arow[r] = slot < 0 ? -1 : slot / g.a_div;
        }
    } else {
        const int m0 = blockIdx.y * 64;
        for (int r = tid; r < 64; r += nthreads) s_arow[r] = s_crow[r] = m0 + r < M ? m0 + r : -1;
    }
    return true;
}

template <typename T> __device__ __forceinline__ void store_out(T *p, float v);
template <> __device__ __forceinline__ void store_out<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16 *p, float v) { *p = __float2bfloat16_rn(v); }

template <int EPI>
__device__ __forceinline__ float gemm_epilogue(const GemmView &g, float a0, float a1, const float *bias, int crow, int n, long long c_off, int act) {
    if (EPI == EPI_GATED) {
        const float sc = g.in_scale ? g.in_scale[crow] : 1.0f;
        return act_apply(act, a0 * sc) * (a1 * sc);
    }
    if (EPI == EPI_ACT) return act_apply(act, a0 + (bias ? bias[n] : 0.0f));
    float v = a0 + (bias ? bias[n] : 0.0f);
    if (g.mul) v *= 1.0f / (1.0f + expf(-g.mul[(size_t)crow * g.ldmul + c_off + n]));
    return v;
}

// ---------------------------------------------------------------------------------------------------------------------
// Prefill projection in true FP32 (no tensor cores): C[M][N] = A[M][K] W[N][K]^T.  64 x 64 x 16 tiles, 4 x 4 per thread.
// OUT_T = float or bf16 (the gated epilogue feeds the next GEMM).
// ---------------------------------------------------------------------------------------------------------------------
template <int EPI, typename OUT_T>
__global__ void __launch_bounds__(256) k_gemm_f32(const float *__restrict__ A, const bf16 *__restrict__ W, const float *__restrict__ bias,
                                                   OUT_T *__restrict__ C, int M, int N, int K, int ldc, int act, GemmView g) {
    constexpr int BM = 64, BN = 64, BK = 16, NB = EPI == EPI_GATED ? 2 : 1;
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[NB][BK][BN + 4];
    __shared__ int s_arow[64], s_crow[64];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * BN;
    if (!gemm_rows(g, M, s_arow, s_crow, tid, 256)) return;
    const int lda = g.lda ? g.lda : K;
    const long long c_off = (long long)blockIdx.z * g.c_bs;
    A += (size_t)blockIdx.z * g.a_bs;
    W += (size_t)blockIdx.z * g.w_bs + (g.tile_group ? (size_t)g.tile_group[blockIdx.y] * g.w_gs : (size_t)0);
    __syncthreads();
    float acc[NB][4][4];
#pragma unroll
    for (int b = 0; b < NB; b++)
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[b][i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += 256) {
            const int r = e / BK, c = e % BK;
            const int m = s_arow[r], k = k0 + c;
            As[c][r] = (m >= 0 && k < K) ? A[(size_t)m * lda + k] : 0.0f;
        }
#pragma unroll
        for (int b = 0; b < NB; b++)
            for (int e = tid; e < BN * BK; e += 256) {
                const int r = e / BK, c = e % BK;
                const int n = n0 + r, k = k0 + c;
                Bs[b][c][r] = (n < N && k < K) ? __bfloat162float(W[((size_t)b * N + n) * K + k]) : 0.0f;
            }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float av[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float bv[4];
#pragma unroll
                for (int j = 0; j < 4; j++) bv[j] = Bs[b][kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[b][i][j] = fmaf(av[i], bv[j], acc[b][i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = s_crow[ty * 4 + i];
        if (m < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            store_out<OUT_T>(C + (size_t)m * ldc + c_off + n, gemm_epilogue<EPI>(g, acc[0][i][j], acc[NB - 1][i][j], bias, m, n, c_off, act));
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Prefill projection on the tensor cores for ANY M, N, K: BF16 operands, FP32 accumulation (mma.sync.m16n8k16).  64 x 64 x 32
// tiles, four warps of 32 x 32; operands staged through padded shared memory (row stride 80 bytes: conflict-free fragment
// reads); out-of-range rows and the K tail are zero-filled.  The shapes the tcgen05 GEMM accepts go there instead.
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// 64 x 32 BF16 tile of a row-major matrix (row stride ld) into shared memory (stride 40 elements), zero-filled outside.
// rowmap (shared memory, nullable) names the source row of every tile row (-1: none); without it tile row r is row r0 + r < R.
__device__ __forceinline__ void load_tile_bf16(bf16 (*dst)[40], const bf16 *__restrict__ src, int r0, int R, const int *rowmap, int ld, int k0, int K, bool vec,
                                               int tid, int nthreads) {
    if (vec) { // 4 chunks of 8 elements per row
        for (int e = tid; e < 64 * 4; e += nthreads) {
            const int r = e >> 2, c = (e & 3) * 8;
            const int row = rowmap ? rowmap[r] : (r0 + r < R ? r0 + r : -1);
            int4 v = make_int4(0, 0, 0, 0);
            if (row >= 0 && k0 + c < K) v = *reinterpret_cast<const int4 *>(src + (size_t)row * ld + k0 + c);
            *reinterpret_cast<int4 *>(&dst[r][c]) = v;
        }
    } else {
        for (int e = tid; e < 64 * 32; e += nthreads) {
            const int r = e >> 5, c = e & 31;
            const int row = rowmap ? rowmap[r] : (r0 + r < R ? r0 + r : -1);
            dst[r][c] = (row >= 0 && k0 + c < K) ? src[(size_t)row * ld + k0 + c] : __float2bfloat16_rn(0.0f);
        }
    }
}

template <int EPI, typename OUT_T>
__global__ void __launch_bounds__(128) k_gemm_bf16(const bf16 *__restrict__ A, const bf16 *__restrict__ W, const float *__restrict__ bias,
                                                    OUT_T *__restrict__ C, int M, int N, int K, int ldc, int act, GemmView gv) {
    constexpr int NB = EPI == EPI_GATED ? 2 : 1;
    __shared__ __align__(16) bf16 As[64][40];
    __shared__ __align__(16) bf16 Bs[NB][64][40];
    __shared__ int s_arow[64], s_crow[64];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 64;
    if (!gemm_rows(gv, M, s_arow, s_crow, tid, 128)) return;
    const int lda = gv.lda ? gv.lda : K;
    const long long c_off = (long long)blockIdx.z * gv.c_bs;
    A += (size_t)blockIdx.z * gv.a_bs;
    W += (size_t)blockIdx.z * gv.w_bs + (gv.tile_group ? (size_t)gv.tile_group[blockIdx.y] * gv.w_gs : (size_t)0);
    const bool vecA = (K & 7) == 0 && (lda & 7) == 0 && (((size_t)A) & 15) == 0;
    const bool vecW = (K & 7) == 0 && (((size_t)W) & 15) == 0;
    __syncthreads();
    float acc[NB][2][4][4];
#pragma unroll
    for (int b = 0; b < NB; b++)
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[b][i][j][e] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 32) {
        load_tile_bf16(As, A, 0, 0, s_arow, lda, k0, K, vecA, tid, 128);
#pragma unroll
        for (int b = 0; b < NB; b++) load_tile_bf16(Bs[b], W + (size_t)b * N * K, n0, N, nullptr, K, k0, K, vecW, tid, 128);
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 32; kk += 16) {
            unsigned af[2][4];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const int r = wm + i * 16 + g;
                af[i][0] = *reinterpret_cast<const unsigned *>(&As[r][kk + 2 * t]);
                af[i][1] = *reinterpret_cast<const unsigned *>(&As[r + 8][kk + 2 * t]);
                af[i][2] = *reinterpret_cast<const unsigned *>(&As[r][kk + 2 * t + 8]);
                af[i][3] = *reinterpret_cast<const unsigned *>(&As[r + 8][kk + 2 * t + 8]);
            }
#pragma unroll
            for (int b = 0; b < NB; b++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    unsigned bfr[2];
                    const int n = wn + j * 8 + g;
                    bfr[0] = *reinterpret_cast<const unsigned *>(&Bs[b][n][kk + 2 * t]);
                    bfr[1] = *reinterpret_cast<const unsigned *>(&Bs[b][n][kk + 2 * t + 8]);
#pragma unroll
                    for (int i = 0; i < 2; i++) mma_bf16_16816(acc[b][i][j], af[i], bfr);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int m = s_crow[wm + i * 16 + g + (e >> 1) * 8];
                const int n = n0 + wn + j * 8 + 2 * t + (e & 1);
                if (m < 0 || n >= N) continue;
                store_out<OUT_T>(C + (size_t)m * ldc + c_off + n, gemm_epilogue<EPI>(gv, acc[0][i][j][e], acc[NB - 1][i][j][e], bias, m, n, c_off, act));
            }
}

// ---------------------------------------------------------------------------------------------------------------------
// Attention of a layer with a sliding window over a ring cache.
// ---------------------------------------------------------------------------------------------------------------------
struct WindowAttn {
    int heads, kv_heads, dk, dv; // query heads, key/value heads, key size, value size
    int window;                  // position i sees j with 0 <= i - j < window
    int ring;                    // cache slots: position j lives in slot j % ring (ring >= window - 1 + rows of a step)
    int ldk, ldv;                // row strides of the key and the value cache (kv_heads * dk, kv_heads * dv when each has rows of its own; a
                                 // latent cache serves both from one row: keys = the whole row, values = its first dv entries)
    int bias_rows;               // rows of the distance table rel[bias_rows][heads]
    float scale, softcap;        // e = softcap * tanh(scale * <q, k> / softcap) + rel[bucket[i - j]][h]   (softcap <= 0: no cap)
    const float *rel;            // [bias_rows][heads] (nullable: no distance bias)
    const int *bucket;           // [window]: table row of every distance the window admits (built on the host in double precision)
    const float *qnorm, *knorm;  // whole-projection RMS norm weights [heads*dk], [kv_heads*dk], used as stored (nullable: no norm)
    int sink;                    // 1: the softmax denominator carries one extra exp(0)
    int gate;                    // 1: the output is multiplied by sigmoid(g), g the fourth block of the fused projection
    int gate_off;                // column of g in a projection row; < 0: behind q | k | v (heads*dk + kv_heads*dk + kv_heads*dv)
    float eps;
    int k_heads;                 // key heads when they differ from the value heads (0: kv_heads): query head h reads key head h / (heads / k_heads).
                                 // Scores mixed over the heads are folded into the query (k_rope_mix_prep): every head then reads ONE key row
                                 // made of all key heads (k_heads = 1, dk = key heads * key size) while the values keep their own heads
    const float *sink_logit;     // [heads] (nullable: 0): with sink, the denominator carries exp(sink_logit[h]) instead of exp(0)
    const float *gate_src;       // the gate is read from row r of this buffer (row stride gate_ld) instead of the query's row (nullable)
    int gate_ld;
    int gate_heads;              // 1: ONE gate per head (g has `heads` entries) instead of one per output entry
    int maps;                    // > 1: every head carries `maps` score maps over the same values.  `heads` then counts (head, map) pairs, pair
                                 // p = head * maps + map reads key slice (value head) * maps + map of a key row [kv_heads][maps][dk] and the
                                 // values of its head; the output keeps one row of dv entries per pair
};
// Row layout of the fused projection output: [q: heads*dk | k: kv_heads*dk | v: kv_heads*dv | g: heads*dv]

// One CTA per row: projection biases, RMS statistics over the WHOLE q and the WHOLE k projection, q normalised in place,
// k / v into the ring.
__global__ void __launch_bounds__(256) k_qk_prep(float *__restrict__ P, int ldp, WindowAttn a, const float *__restrict__ bias, float *__restrict__ kc,
                                                 float *__restrict__ vc, bf16 *__restrict__ kc16, bf16 *__restrict__ vc16, const StepState *__restrict__ st) {
    __shared__ float red[32];
    const int r = blockIdx.x, tid = threadIdx.x;
    const int qd = a.heads * a.dk, kd = a.kv_heads * a.dk, vd = a.kv_heads * a.dv;
    float *q = P + (size_t)r * ldp, *k = q + qd, *v = k + kd;
    const int slot = (st->pos + r) % a.ring;
    if (bias) { // q | k | v biases of the fused projection, added where it is consumed
        for (int i = tid; i < qd + kd + vd; i += 256) q[i] += bias[i];
        __syncthreads();
    }
    float qinv = 1.0f, kinv = 1.0f;
    if (a.qnorm) {
        float ss = 0.0f;
        for (int i = tid; i < qd; i += 256) ss = fmaf(q[i], q[i], ss);
        ss = block_sum(ss, red);
        qinv = 1.0f / sqrtf(ss / (float)qd + a.eps);
    }
    if (a.knorm) {
        float ss = 0.0f;
        for (int i = tid; i < kd; i += 256) ss = fmaf(k[i], k[i], ss);
        ss = block_sum(ss, red);
        kinv = 1.0f / sqrtf(ss / (float)kd + a.eps);
    }
    for (int i = tid; i < qd; i += 256) q[i] = a.qnorm ? q[i] * qinv * a.qnorm[i] : q[i];
    for (int i = tid; i < kd; i += 256) {
        const float kv = a.knorm ? k[i] * kinv * a.knorm[i] : k[i];
        kc[(size_t)slot * kd + i] = kv;
        if (kc16) kc16[(size_t)slot * kd + i] = __float2bfloat16_rn(kv); // BF16 twin row for the tensor-core prefill attention
    }
    for (int i = tid; i < vd; i += 256) {
        vc[(size_t)slot * vd + i] = v[i];
        if (vc16) vc16[(size_t)slot * vd + i] = __float2bfloat16_rn(v[i]);
    }
}

// One CTA per (row, head): scores of the window into shared memory, softmax with the sink term, weighted value sum, gate.
// Scores: a group of dk/4 lanes (at most a warp) owns a key and reads its row with coalesced 128-bit loads; values: a group of
// dv/4 threads owns every groups-th key.  Sizes that are no multiple of 4 take scalar loads.
// gridDim.z > 1 splits the window of a (row, head) over several CTAs; the last one to arrive merges the parts.
// Dynamic shared memory: att_smem_floats(dk, window) floats.
#define LY_ATT_THREADS 256
// Scratch of a launch that splits every (row, head) over gridDim.z CTAs (the decode step: one row, few heads, many SMs):
// per part the unnormalised weighted value sum o[dv] and {maximum, sum of exponentials}; count = arrival counter per (row, head).
struct KeySplit {
    float *o, *ml;
    unsigned *count;
};
__host__ __device__ inline size_t att_smem_floats(int dk, int window) { return (size_t)((dk + 3) / 4 * 4) + window + 4 * LY_ATT_THREADS; }

template <typename OUT_T>
__global__ void __launch_bounds__(LY_ATT_THREADS) k_window_attention(const float *__restrict__ P, int ldp, WindowAttn a, const float *__restrict__ kc,
                                                                     const float *__restrict__ vc, const StepState *__restrict__ st,
                                                                     OUT_T *__restrict__ out, int ldo, KeySplit ks_) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[32];
    __shared__ int s_last;
    const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int splits = gridDim.z, z = blockIdx.z;
    const int qd = a.heads * a.dk, kd = a.kv_heads * a.dk, vd = a.kv_heads * a.dv;
    const int g = h / (a.heads / a.kv_heads);
    const int gk = a.maps > 1 ? g * a.maps + h % a.maps : a.k_heads > 0 ? h / (a.heads / a.k_heads) : g;
    const float sink_v = a.sink_logit ? a.sink_logit[h] : 0.0f;
    const int pos = st->pos + r;
    int lo = pos - a.window + 1 > 0 ? pos - a.window + 1 : 0;
    int nk = pos - lo + 1;
    if (splits > 1) { // this CTA's share of the window; everything below indexes keys as lo + j, j < nk
        const int chunk = (nk + splits - 1) / splits, jb = z * chunk;
        lo += jb;
        nk = nk - jb < chunk ? nk - jb : chunk;
        if (nk < 0) nk = 0;
    }
    float *qs = sm, *sc = sm + (a.dk + 3) / 4 * 4, *part = sc + a.window;
    const float *q = P + (size_t)r * ldp + (size_t)h * a.dk;
    for (int i = tid; i < a.dk; i += LY_ATT_THREADS) qs[i] = q[i];
    __syncthreads();
    float mx = (a.sink && splits == 1) ? sink_v : -INFINITY; // the sink's logit takes part in the maximum (split runs: when the parts are merged)
    {
        const bool vec = (a.dk & 3) == 0 && (a.ldk & 3) == 0;
        int lpk = 32; // lanes per key
        if (vec) { lpk = 1; while (lpk < a.dk / 4 && lpk < 32) lpk <<= 1; }
        const int kpw = 32 / lpk, sub = lane % lpk, ks = lane / lpk;
        const int stride = (LY_ATT_THREADS / 32) * kpw; // keys per CTA-wide step
        auto finish = [&](int j, float d) { // after the lane reduction: cap, bias, store (one lane per key)
            float e = d * a.scale;
            if (a.softcap > 0.0f) e = a.softcap * tanhf(e / a.softcap);
            if (a.rel) e += a.rel[(size_t)a.bucket[pos - lo - j] * a.heads + h];
            sc[j] = e;
            mx = fmaxf(mx, e);
        };
        if (vec && a.dk <= 128) { // one 128-bit chunk per lane and key: four keys in flight per lane
            const bool has = sub < a.dk / 4;
            const float4 qv = has ? *reinterpret_cast<const float4 *>(qs + 4 * sub) : make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j0 = warp * kpw; j0 < nk; j0 += 4 * stride) {
                float4 kv[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int j = j0 + u * stride + ks;
                    kv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (has && j < nk) kv[u] = *reinterpret_cast<const float4 *>(kc + (size_t)((lo + j) % a.ring) * a.ldk + (size_t)gk * a.dk + 4 * sub);
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int j = j0 + u * stride + ks;
                    float d = fmaf(qv.x, kv[u].x, fmaf(qv.y, kv[u].y, fmaf(qv.z, kv[u].z, qv.w * kv[u].w)));
                    for (int o = lpk >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                    if (j < nk && sub == 0) finish(j, d);
                }
            }
        } else {
            for (int j0 = warp * kpw; j0 < nk; j0 += stride) {
                const int j = j0 + ks;
                float d = 0.0f;
                if (j < nk) {
                    const float *kr = kc + (size_t)((lo + j) % a.ring) * a.ldk + (size_t)gk * a.dk;
                    if (vec) {
                        for (int c = sub; c < a.dk / 4; c += lpk) {
                            const float4 kv = *reinterpret_cast<const float4 *>(kr + 4 * c), qv = *reinterpret_cast<const float4 *>(qs + 4 * c);
                            d = fmaf(qv.x, kv.x, d); d = fmaf(qv.y, kv.y, d); d = fmaf(qv.z, kv.z, d); d = fmaf(qv.w, kv.w, d);
                        }
                    } else {
                        for (int i = sub; i < a.dk; i += lpk) d = fmaf(qs[i], kr[i], d);
                    }
                }
                for (int o = lpk >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                if (j < nk && sub == 0) finish(j, d);
            }
        }
    }
    mx = block_max(mx, red);
    float sum = 0.0f;
    for (int j = tid; j < nk; j += LY_ATT_THREADS) {
        const float w = expf(sc[j] - mx);
        sc[j] = w;
        sum += w;
    }
    sum = block_sum(sum, red); // also orders the sc[] writes before the reads below
    const float inv = splits > 1 ? 1.0f : 1.0f / (sum + (a.sink ? expf(sink_v - mx) : 0.0f)); // split runs keep the unnormalised sum
    const size_t cell = (size_t)r * a.heads + h; // (row, head)
    float *my_o = splits > 1 ? ks_.o + (cell * splits + z) * a.dv : nullptr;
    const float *gate = (a.gate_src ? a.gate_src + (size_t)r * a.gate_ld : P + (size_t)r * ldp) + (a.gate_off >= 0 ? a.gate_off : qd + kd + vd) +
                        (a.gate_heads ? (size_t)h : (size_t)h * a.dv);
    const int gs = a.gate_heads ? 0 : 1; // stride of the gate over the output entries of a head
    const int vw = ((a.dv & 3) == 0 && (a.ldv & 3) == 0) ? 4 : 1; // value elements per thread
    int tpk = (a.dv + vw - 1) / vw;                             // threads per key
    if (tpk > LY_ATT_THREADS) tpk = LY_ATT_THREADS;
    const int groups = LY_ATT_THREADS / tpk, grp = tid / tpk, dl = tid % tpk;
    for (int db = 0; db < a.dv; db += tpk * vw) {
        const int d = db + dl * vw;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (grp < groups && d < a.dv) {
#pragma unroll 4
            for (int j = grp; j < nk; j += groups) {
                const float *vr = vc + (size_t)((lo + j) % a.ring) * a.ldv + (size_t)g * a.dv + d;
                const float w = sc[j];
                if (vw == 4) {
                    const float4 v = *reinterpret_cast<const float4 *>(vr);
                    acc[0] = fmaf(w, v.x, acc[0]); acc[1] = fmaf(w, v.y, acc[1]); acc[2] = fmaf(w, v.z, acc[2]); acc[3] = fmaf(w, v.w, acc[3]);
                } else acc[0] = fmaf(w, vr[0], acc[0]);
            }
        }
        __syncthreads(); // part is reused per value block
#pragma unroll
        for (int e = 0; e < 4; e++) part[e * LY_ATT_THREADS + tid] = acc[e];
        __syncthreads();
        if (grp == 0 && d < a.dv) {
            for (int e = 0; e < vw; e++) {
                float o = 0.0f;
                for (int k = 0; k < groups; k++) o += part[e * LY_ATT_THREADS + k * tpk + dl];
                if (splits > 1) { my_o[d + e] = o; continue; }
                o *= inv;
                if (a.gate) o *= 1.0f / (1.0f + expf(-gate[(d + e) * gs]));
                store_out<OUT_T>(out + (size_t)r * ldo + (size_t)h * a.dv + d + e, o);
            }
        }
    }
    if (splits == 1) return;
    // the last CTA of this (row, head) to arrive merges the parts: maximum over the parts (and the sink), rescaled sums
    if (tid == 0) { ks_.ml[(cell * splits + z) * 2] = mx; ks_.ml[(cell * splits + z) * 2 + 1] = sum; }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(ks_.count + cell, 1u) == (unsigned)splits - 1u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float M = a.sink ? sink_v : -INFINITY;
    for (int k = 0; k < splits; k++) M = fmaxf(M, __ldcg(ks_.ml + (cell * splits + k) * 2));
    float Lsum = a.sink ? expf(sink_v - M) : 0.0f;
    for (int k = 0; k < splits; k++) {
        const float mk = __ldcg(ks_.ml + (cell * splits + k) * 2);
        if (mk != -INFINITY) Lsum += __ldcg(ks_.ml + (cell * splits + k) * 2 + 1) * expf(mk - M);
    }
    for (int d = tid; d < a.dv; d += LY_ATT_THREADS) {
        float o = 0.0f;
        for (int k = 0; k < splits; k++) {
            const float mk = __ldcg(ks_.ml + (cell * splits + k) * 2);
            if (mk != -INFINITY) o += __ldcg(ks_.o + (cell * splits + k) * a.dv + d) * expf(mk - M);
        }
        o /= Lsum;
        if (a.gate) o *= 1.0f / (1.0f + expf(-gate[d * gs]));
        store_out<OUT_T>(out + (size_t)r * ldo + (size_t)h * a.dv + d, o);
    }
    if (tid == 0) ks_.count[cell] = 0u; // ready for the next launch
}

// ---------------------------------------------------------------------------------------------------------------------
// The same attention for a prefill chunk on the tensor cores (BF16 compute mode; instantiated for key / value sizes 64 / 64,
// 128 / 128 and 192 / 128): one CTA per (128 query rows, head), eight
// warps of 16 rows (two warps per scheduler: a lone warp cannot hide the latency of its own dependent instructions).  Keys and values come from the BF16 twin rows of the ring (written by k_qk_prep next to the FP32 rows the
// decode step reads): key tiles of 64 positions travel global -> shared with cp.async, double buffered, so the copy of tile
// i + 1 overlaps the mma.sync m16n8k16 work on tile i; V fragments are read with ldmatrix.trans.  Scores, cap, distance bias,
// mask and the ONLINE softmax stay in FP32 registers.  The sink is the initial state of the running softmax: maximum 0,
// denominator exp(0) = 1, no value.  Dynamic shared memory: att_mma_smem_bytes<DK, DV>(window).
// ---------------------------------------------------------------------------------------------------------------------
#define LY_ATT_MMA_ROWS 128 // query rows per CTA: eight warps of 16 rows share every key tile
#define LY_ATT_MMA_THREADS (LY_ATT_MMA_ROWS * 2)
template <int DK, int DV> __host__ __device__ constexpr size_t att_mma_smem_bytes(int window) {
    return (size_t)(LY_ATT_MMA_ROWS * (DK + 8) * 2) + (size_t)(64 * (DK + 8) * 2) * 2 + (size_t)(64 * (DV + 8) * 2) * 2 + (size_t)window * 4;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned *>(&v);
}
// tanh(x) = 1 - 2 / (1 + exp(2x)) with the hardware exponential: absolute error ~1e-7, far below the BF16 rounding of the
// operands that produced x (the FP32 kernels keep tanhf)
__device__ __forceinline__ float tanh_fast(float x) { return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * x)); }
__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool valid) { // 16 bytes, zero-filled when !valid
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void ldmatrix_x2_trans(unsigned (&r)[2], const void *row) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}

template <int DK, int DV>
__global__ void __launch_bounds__(LY_ATT_MMA_THREADS) k_window_attention_mma(const float *__restrict__ P, int ldp, WindowAttn a, const bf16 *__restrict__ kc16,
                                                                             const bf16 *__restrict__ vc16, const StepState *__restrict__ st, int n,
                                                                             bf16 *__restrict__ out, int ldo, float *__restrict__ out32 = nullptr) {
    extern __shared__ __align__(16) unsigned char smraw[];
    constexpr int BM = LY_ATT_MMA_ROWS;
    constexpr int QT = BM * (DK + 8) * 2, KT = 64 * (DK + 8) * 2, VT = 64 * (DV + 8) * 2; // bytes of the Q tile, one K tile, one V tile
    bf16(*Qs)[DK + 8] = reinterpret_cast<bf16(*)[DK + 8]>(smraw);
    float *sbias = reinterpret_cast<float *>(smraw + QT + 2 * KT + 2 * VT);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int h = blockIdx.y, r0 = blockIdx.x * BM;
    const int kd = a.ldk, vd = a.ldv, qd = a.heads * DK; // row strides of the BF16 twin rings = those of the FP32 rings
    const int kvh = h / (a.heads / a.kv_heads);
    const int kh = a.maps > 1 ? kvh * a.maps + h % a.maps : a.k_heads > 0 ? h / (a.heads / a.k_heads) : kvh;
    const float sink_v = a.sink_logit ? a.sink_logit[h] : 0.0f;
    const int pos0 = st->pos;
    const int rows = n - r0 < BM ? n - r0 : BM;
    const int q_lo = pos0 + r0, q_hi = pos0 + r0 + rows - 1;
    const int k_lo = q_lo - a.window + 1 > 0 ? q_lo - a.window + 1 : 0;
    auto load_tile = [&](int buf, int kt0) {
        bf16(*Kd)[DK + 8] = reinterpret_cast<bf16(*)[DK + 8]>(smraw + QT + buf * KT);
        bf16(*Vd)[DV + 8] = reinterpret_cast<bf16(*)[DV + 8]>(smraw + QT + 2 * KT + buf * VT);
        const int slot0 = kt0 % a.ring; // one division per tile; rows wrap by subtraction (by division only in rings below 64 slots)
        for (int e = tid; e < 64 * (DK / 8); e += LY_ATT_MMA_THREADS) {
            const int r = e / (DK / 8), c = (e % (DK / 8)) * 8;
            const bool ok = kt0 + r <= q_hi;
            int sl = slot0 + r;
            if (sl >= a.ring) sl = a.ring >= 64 ? sl - a.ring : sl % a.ring;
            cp_async16(&Kd[r][c], kc16 + (ok ? (size_t)sl * kd + (size_t)kh * DK + c : 0), ok);
        }
        for (int e = tid; e < 64 * (DV / 8); e += LY_ATT_MMA_THREADS) {
            const int r = e / (DV / 8), c = (e % (DV / 8)) * 8;
            const bool ok = kt0 + r <= q_hi;
            int sl = slot0 + r;
            if (sl >= a.ring) sl = a.ring >= 64 ? sl - a.ring : sl % a.ring;
            cp_async16(&Vd[r][c], vc16 + (ok ? (size_t)sl * vd + (size_t)kvh * DV + c : 0), ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_tile(0, k_lo);
    // distance -> bias of this head, for the distances this tile of rows can see
    {
        const int dmax = q_hi - k_lo + 1 < a.window ? q_hi - k_lo + 1 : a.window;
        for (int d = tid; d < dmax; d += LY_ATT_MMA_THREADS) sbias[d] = a.rel ? a.rel[(size_t)a.bucket[d] * a.heads + h] : 0.0f;
    }
    // Q tile -> BF16
    for (int e = tid; e < BM * (DK / 4); e += LY_ATT_MMA_THREADS) {
        const int r = e / (DK / 4), c = (e % (DK / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows) v = *reinterpret_cast<const float4 *>(P + (size_t)(r0 + r) * ldp + (size_t)h * DK + c);
        *reinterpret_cast<uint2 *>(&Qs[r][c]) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
    }
    __syncthreads();
    unsigned qf[DK / 16][4];
    {
        const int r = warp * 16 + g;
#pragma unroll
        for (int kk = 0; kk < DK / 16; kk++) {
            qf[kk][0] = *reinterpret_cast<const unsigned *>(&Qs[r][kk * 16 + 2 * t]);
            qf[kk][1] = *reinterpret_cast<const unsigned *>(&Qs[r + 8][kk * 16 + 2 * t]);
            qf[kk][2] = *reinterpret_cast<const unsigned *>(&Qs[r][kk * 16 + 2 * t + 8]);
            qf[kk][3] = *reinterpret_cast<const unsigned *>(&Qs[r + 8][kk * 16 + 2 * t + 8]);
        }
    }
    float o[DV / 8][4];
#pragma unroll
    for (int j = 0; j < DV / 8; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[j][e] = 0.0f;
    float mrow[2], lrow[2];
    mrow[0] = mrow[1] = a.sink ? sink_v : -INFINITY; // the sink: a running softmax that starts at (maximum z, denominator exp(z - z))
    lrow[0] = lrow[1] = a.sink ? 1.0f : 0.0f;
    const int prow[2] = {pos0 + r0 + warp * 16 + g, pos0 + r0 + warp * 16 + g + 8}; // positions of this thread's two rows
    const bool vrow[2] = {warp * 16 + g < rows, warp * 16 + g + 8 < rows};
    const int w_lo = pos0 + r0 + warp * 16, w_hi = w_lo + 15; // positions of this warp's rows
    const float inv_cap = a.softcap > 0.0f ? 1.0f / a.softcap : 0.0f;
    int buf = 0;
    for (int kt0 = k_lo; kt0 <= q_hi; kt0 += 64, buf ^= 1) {
        if (kt0 + 64 <= q_hi) {
            load_tile(buf ^ 1, kt0 + 64); // the other buffer was released by the barrier that ended the previous iteration
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // a warp whose rows see no key of this tile (all later, or all beyond the window) skips the arithmetic
        if (kt0 <= w_hi && kt0 + 63 > w_lo - a.window) {
            bf16(*Ks)[DK + 8] = reinterpret_cast<bf16(*)[DK + 8]>(smraw + QT + buf * KT);
            bf16(*Vs)[DV + 8] = reinterpret_cast<bf16(*)[DV + 8]>(smraw + QT + 2 * KT + buf * VT);
            // S = Q K^T for this warp's 16 rows x 64 keys
            float sc[8][4];
#pragma unroll
            for (int j = 0; j < 8; j++) {
#pragma unroll
                for (int e = 0; e < 4; e++) sc[j][e] = 0.0f;
#pragma unroll
                for (int kk = 0; kk < DK / 16; kk++) {
                    unsigned bfr[2];
                    bfr[0] = *reinterpret_cast<const unsigned *>(&Ks[j * 8 + g][kk * 16 + 2 * t]);
                    bfr[1] = *reinterpret_cast<const unsigned *>(&Ks[j * 8 + g][kk * 16 + 2 * t + 8]);
                    mma_bf16_16816(sc[j], qf[kk], bfr);
                }
            }
            // cap, bias, mask; tile maximum per row
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int rr = e >> 1, pj = kt0 + j * 8 + 2 * t + (e & 1), dist = prow[rr] - pj;
                    float v = sc[j][e] * a.scale;
                    if (a.softcap > 0.0f) v = a.softcap * tanh_fast(v * inv_cap);
                    if (vrow[rr] && dist >= 0 && dist < a.window) v += sbias[dist];
                    else v = -INFINITY;
                    sc[j][e] = v;
                    tmax[rr] = fmaxf(tmax[rr], v);
                }
            float corr[2], muse[2];
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 1));
                tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 2));
                const float mnew = fmaxf(mrow[rr], tmax[rr]);
                muse[rr] = mnew == -INFINITY ? 0.0f : mnew;
                corr[rr] = mrow[rr] == -INFINITY ? 0.0f : __expf(mrow[rr] - muse[rr]);
                mrow[rr] = mnew;
                lrow[rr] *= corr[rr];
            }
            float psum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < 8; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float pv = __expf(sc[j][e] - muse[e >> 1]); // exp(-inf) = 0 for masked entries
                    sc[j][e] = pv;
                    psum[e >> 1] += pv;
                }
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                psum[rr] += __shfl_xor_sync(0xffffffffu, psum[rr], 1);
                psum[rr] += __shfl_xor_sync(0xffffffffu, psum[rr], 2);
                lrow[rr] += psum[rr];
            }
#pragma unroll
            for (int j = 0; j < DV / 8; j++) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
            // O += P V: the score fragments are the A operand as they stand; V[key][d] becomes the B operand through ldmatrix.trans
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                unsigned pf[4];
                pf[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
                pf[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
                pf[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
                pf[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
                for (int j = 0; j < DV / 8; j++) {
                    unsigned bfr[2];
                    ldmatrix_x2_trans(bfr, &Vs[kk * 16 + (lane & 15)][j * 8]);
                    mma_bf16_16816(o[j], pf, bfr);
                }
            }
        }
        __syncthreads(); // every warp is done with this buffer before the next iteration's copy lands in it
    }
    // normalise, gate, store
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
        if (!vrow[rr]) continue;
        const int r = r0 + warp * 16 + g + rr * 8;
        const float inv = lrow[rr] > 0.0f ? 1.0f / lrow[rr] : 0.0f;
        const float *gate = (a.gate_src ? a.gate_src + (size_t)r * a.gate_ld : P + (size_t)r * ldp) + (a.gate_off >= 0 ? a.gate_off : qd + kd + vd) +
                            (a.gate_heads ? (size_t)h : (size_t)h * DV);
        const float ghead = a.gate && a.gate_heads ? 1.0f / (1.0f + expf(-gate[0])) : 1.0f;
#pragma unroll
        for (int j = 0; j < DV / 8; j++) {
            const int d = j * 8 + 2 * t;
            float v0 = o[j][2 * rr] * inv * ghead, v1 = o[j][2 * rr + 1] * inv * ghead;
            if (a.gate && !a.gate_heads) {
                const float2 gv = *reinterpret_cast<const float2 *>(gate + d);
                v0 *= 1.0f / (1.0f + expf(-gv.x));
                v1 *= 1.0f / (1.0f + expf(-gv.y));
            }
            if (out32) *reinterpret_cast<float2 *>(out32 + (size_t)r * ldo + (size_t)h * DV + d) = make_float2(v0, v1); // FP32 results (what a later subtraction reads)
            else *reinterpret_cast<unsigned *>(out + (size_t)r * ldo + (size_t)h * DV + d) = pack_bf16(v0, v1);
        }
    }
}

} // namespace ly
