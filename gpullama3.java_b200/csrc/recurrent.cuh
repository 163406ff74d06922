// recurrent.cuh -- device kernels of the layered plans' fourth family of mechanisms (first user: Dinuzen), beside those of
// layered.cuh, latent.cuh and delta.cuh and sharing their projection, attention, router and grouping kernels:
//   * k_outnorm_rows     the OUTNORM block's row kernel: x += ls * GN(y; w) with GN an RMS norm in `groups` equal consecutive parts
//                        on the sublayer's OUTPUT (y a plain row, or a mixture of experts assembled here: routing weights on the
//                        experts' results, identity experts, a sigmoid-gated shared expert); the depth average x <- sum_j dwa[j] X_j
//                        over the kept results of all earlier layers; the embedding gather; the gathered final norm; for a single
//                        row also the token shift of the next mixer;
//   * k_shift_rows       token shift of a chunk: h[t] = x[t] + (x[t-1] - x[t]) * shift, the row before the chunk from the state;
//   * k_conv_rows        causal convolution per channel over a ring of its own inputs (bias on the input and on the output, optional
//                        SiLU), any cut of the sequence into launches;
//   * k_rglru_scan       real-gated linear recurrent unit: a = exp(-8 sigmoid(r) softplus(lam)), S <- a S + sqrt(1 - a^2) sigmoid(i) u,
//                        output S * gelu_tanh(y): a two-level scan over the rows of a chunk (up to 32 row groups per CTA);
//   * k_ssd_scan         state-space recurrence with a matrix state per head, S <- exp(-exp(A) dt) S + dt B x^T, y = S^T C + D x,
//                        state columns in registers;
//   * k_gated_group_norm y * silu(z), RMS norm in groups, weight;
//   * k_slice_norm_rope  RMS norm of every key_dim slice of q and k with one weight, table-driven rotation, key / value rows into the ring;
//   * k_diff_combine     differential attention: o = a1 - lambda a2, o / rms(o) * (1 - diff) per head;
//   * k_act_rows         activation over FP32 rows into the operand buffer of the next GEMM.
// Norm statistics, gates, decays, states, rotation and the residual sum are FP32 in both compute modes.
#pragma once
#include "layered.cuh"
#include "latent.cuh"
#include "delta.cuh"

namespace ly {

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

struct OutNormArgs {
    float *x;              // [n][E] residual stream
    const bf16 *emb;       // embedding table [vocab][E]: x = emb[token] (nullable)
    const int *tokens;     // [n] (nullable: the step's own token)
    const StepState *st;
    const float *y;        // [n][E] sublayer output (nullable)
    // mixture of experts (ys != nullptr): y = sum_k wts[r * top + k] * (ids[r * top + k] < n_real ? ys[row of slot r * top + k] : x[r])
    //                                         + sigmoid(sg[r * sg_ld]) * shared[r]
    const float *ys;       // per-slot expert results [slots][E]
    const int *ys_map;     // (nullable) slot s lives in row ys_map[s] of ys
    const int *ids;
    const float *wts;
    int top, n_real;
    const float *shared;   // [n][E] (nullable)
    const float *sg;       // gate logit of the shared expert, one per row
    int sg_ld;
    const float *w, *ls;   // [E] norm weight and layer scale of the sublayer that produced y
    int groups;
    float eps;
    int E, n;
    float *save_prev;      // [E] (nullable): the last row's x BEFORE the update becomes the previous row of the next call's token shift
    float *stash;          // kept results X_j: [j][stash_rows][E]
    long long stash_stride;
    int stash_idx;         // >= 0: the row after the update is X_idx and is kept
    const float *dwa;      // [stash_idx + 1] (nullable): x <- sum_j dwa[j] X_j
    float *trace;          // [n][E]: copy of x as this kernel leaves it (nullable)
    const float *shift;    // [E] (nullable; single-row launches only): out = x + (prev - x) * shift
    const float *prev;     // [E] previous row of that shift (zeros at position 0 whatever it holds)
    const float *w_out;    // [E] (nullable): out = GN(x; w_out)
    const int *gather;     // output row r is computed from x row gather[r] (read-only use: no update then)
    float *out32;          // [n][E] (any of out32 / out16, or none)
    bf16 *out16;
};

// Per part sums of squares of v [E] (parts of E / groups entries) -> inv[g] = 1 / sqrt(mean + eps).  inv: shared memory.
// Several parts of a multiple of 32 entries (E <= 32 * LY_GROUP_WARP_SUMS): every warp leaves the sum of each 32 consecutive entries it
// visits, then a warp per part adds that part's sums -- two barriers whatever the number of parts, a fixed order of additions.
// Other shapes: one block reduction per part.
#define LY_GROUP_WARP_SUMS 512
__device__ __forceinline__ void group_inv_rms(const float *v, int E, int groups, float eps, float *inv, float *red) {
    const int part = E / groups;
    if (groups > 1 && part % 32 == 0 && E <= 32 * LY_GROUP_WARP_SUMS) {
        __shared__ float wsum[LY_GROUP_WARP_SUMS];
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5, per = part / 32;
        for (int i0 = warp * 32; i0 < E; i0 += nw * 32) {
            const float t = v[i0 + lane];
            const float ss = warp_sum(t * t);
            if (lane == 0) wsum[i0 >> 5] = ss;
        }
        __syncthreads();
        for (int g = warp; g < groups; g += nw) {
            float ss = 0.0f;
            for (int k = lane; k < per; k += 32) ss += wsum[g * per + k];
            ss = warp_sum(ss);
            if (lane == 0) inv[g] = 1.0f / sqrtf(ss / (float)part + eps);
        }
        __syncthreads();
        return;
    }
    for (int g = 0; g < groups; g++) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < part; i += blockDim.x) { const float t = v[g * part + i]; ss = fmaf(t, t, ss); }
        ss = block_sum(ss, red);
        if (threadIdx.x == 0) inv[g] = 1.0f / sqrtf(ss / (float)part + eps);
    }
    __syncthreads();
}

#define LY_OUTNORM_MAX_GROUPS 256
#define LY_OUTNORM_SLOTS 64  // chosen experts / depth weights kept in shared memory (more: read where they are)
// One CTA of NTH threads per row.  Dynamic shared memory: 2 * E floats.
template <int NTH>
__global__ void __launch_bounds__(NTH, 1) k_outnorm_rows(OutNormArgs a) {
    extern __shared__ __align__(16) float smo[];
    __shared__ float red[32];
    __shared__ float inv[LY_OUTNORM_MAX_GROUPS];
    __shared__ long long s_row[LY_OUTNORM_SLOTS]; // offset of a chosen expert's result row (-1: an identity expert)
    __shared__ float s_wt[LY_OUTNORM_SLOTS], s_dwa[LY_OUTNORM_SLOTS];
    const int r = blockIdx.x, tid = threadIdx.x, E = a.E;
    constexpr int nth = NTH;
    float *row = smo, *yv = smo + E;
    const size_t src = (size_t)(a.gather ? a.gather[r] : r) * E, dst = (size_t)r * E;
    // the row's few indices and weights first: everything after them is independent loads
    const bool slots = a.ys && a.top <= LY_OUTNORM_SLOTS, depth = a.stash_idx >= 0 && a.dwa && a.stash_idx < LY_OUTNORM_SLOTS;
    if (slots && tid < a.top) {
        const size_t e = (size_t)r * a.top + tid;
        s_row[tid] = a.ids[e] < a.n_real ? (long long)((a.ys_map ? (size_t)a.ys_map[e] : e) * E) : -1;
        s_wt[tid] = a.wts[e];
    }
    if (depth && tid <= a.stash_idx) s_dwa[tid] = a.dwa[tid];
    if (a.emb) {
        const int token = a.tokens ? a.tokens[r] : a.st->token;
        const bf16 *e = a.emb + (size_t)token * E;
        for (int i = tid; i < E; i += nth) row[i] = __bfloat162float(e[i]);
    } else {
        for (int i = tid; i < E; i += nth) row[i] = a.x[src + i];
    }
    if (a.save_prev && r == a.n - 1)
        for (int i = tid; i < E; i += nth) a.save_prev[i] = row[i];
    const bool add = a.y || a.ys;
    if (add) {
        __syncthreads();
        if (a.ys) {
            const float sgv = a.shared ? sigmoidf_(a.sg[(size_t)r * a.sg_ld]) : 0.0f;
            if (slots && NTH >= 1024) { // a single wide row: per entry, the chosen experts' loads are issued eight at a time before the first is used
                for (int i = tid; i < E; i += nth) {
                    float s = a.shared ? sgv * a.shared[src + i] : 0.0f;
                    for (int k0 = 0; k0 < a.top; k0 += 8) {
                        float v[8];
#pragma unroll
                        for (int u = 0; u < 8; u++) v[u] = k0 + u < a.top ? (s_row[k0 + u] >= 0 ? __ldg(a.ys + s_row[k0 + u] + i) : row[i]) : 0.0f;
#pragma unroll
                        for (int u = 0; u < 8; u++) if (k0 + u < a.top) s = fmaf(s_wt[k0 + u], v[u], s);
                    }
                    yv[i] = s;
                }
            } else if (slots) { // many rows: one chosen expert per pass over the row, the loads of a pass are independent and the CTAs many
                for (int i = tid; i < E; i += nth) yv[i] = a.shared ? sgv * a.shared[src + i] : 0.0f;
                for (int k = 0; k < a.top; k++) {
                    const float wk = s_wt[k];
                    const float *v = s_row[k] >= 0 ? a.ys + s_row[k] : row;
#pragma unroll 4
                    for (int i = tid; i < E; i += nth) yv[i] = fmaf(wk, v[i], yv[i]);
                }
            } else {
                for (int i = tid; i < E; i += nth) {
                    float s = a.shared ? sgv * a.shared[src + i] : 0.0f;
                    for (int k = 0; k < a.top; k++) {
                        const size_t e = (size_t)r * a.top + k;
                        const float v = a.ids[e] < a.n_real ? a.ys[(a.ys_map ? (size_t)a.ys_map[e] : e) * E + i] : row[i];
                        s = fmaf(a.wts[e], v, s);
                    }
                    yv[i] = s;
                }
            }
        } else {
            for (int i = tid; i < E; i += nth) yv[i] = a.y[src + i];
        }
        __syncthreads();
        group_inv_rms(yv, E, a.groups, a.eps, inv, red);
        const int part = E / a.groups;
        for (int i = tid; i < E; i += nth) row[i] = fmaf(a.ls[i], yv[i] * inv[i / part] * a.w[i], row[i]);
    } else if (depth) __syncthreads();
    if (a.stash_idx >= 0) { // every thread touches its own entries of the row only: no barrier between the passes
        const float *dw = depth ? s_dwa : a.dwa;
        float *mine = a.stash + (size_t)a.stash_idx * a.stash_stride + src;
        for (int i = tid; i < E; i += nth) mine[i] = row[i];
        if (dw && NTH >= 1024) { // a single wide row: per entry, the earlier results' loads are issued eight at a time
            const float wl = dw[a.stash_idx];
            const float *s0 = a.stash + src;
            for (int i = tid; i < E; i += nth) {
                float acc = row[i] * wl;
                for (int j0 = 0; j0 < a.stash_idx; j0 += 8) {
                    float v[8];
#pragma unroll
                    for (int u = 0; u < 8; u++) v[u] = j0 + u < a.stash_idx ? __ldg(s0 + (size_t)(j0 + u) * a.stash_stride + i) : 0.0f;
#pragma unroll
                    for (int u = 0; u < 8; u++) if (j0 + u < a.stash_idx) acc = fmaf(dw[j0 + u], v[u], acc);
                }
                row[i] = acc;
            }
        } else if (dw) { // many rows: one earlier result per pass
            const float wl = dw[a.stash_idx];
            for (int i = tid; i < E; i += nth) row[i] *= wl;
            for (int j = 0; j < a.stash_idx; j++) {
                const float wj = dw[j];
                const float *sj = a.stash + (size_t)j * a.stash_stride + src;
#pragma unroll 4
                for (int i = tid; i < E; i += nth) row[i] = fmaf(wj, __ldg(sj + i), row[i]);
            }
        }
    }
    if (!a.gather && (a.emb || add || a.stash_idx >= 0))
        for (int i = tid; i < E; i += nth) a.x[src + i] = row[i];
    if (a.trace)
        for (int i = tid; i < E; i += nth) a.trace[src + i] = row[i];
    if (!a.out32 && !a.out16) return;
    if (a.w_out) {
        __syncthreads();
        group_inv_rms(row, E, a.groups, a.eps, inv, red);
    }
    const int part = E / a.groups;
    const bool first = a.shift && a.st->pos == 0;
    for (int i = tid; i < E; i += nth) {
        float v = row[i];
        if (a.w_out) v = v * inv[i / part] * a.w_out[i];
        else if (a.shift) v = fmaf((first ? 0.0f : a.prev[i]) - v, a.shift[i], v);
        if (a.out32) a.out32[dst + i] = v;
        if (a.out16) a.out16[dst + i] = __float2bfloat16_rn(v);
    }
}

// Token shift of a chunk of n rows at positions st->pos ..: out[t] = x[t] + (x[t-1] - x[t]) * shift; the row before the chunk is
// `prev` (kept by an earlier call), zeros at position 0.  grid (n), 256 threads.
__global__ void __launch_bounds__(256) k_shift_rows(const float *__restrict__ x, int E, const float *__restrict__ shift, const float *__restrict__ prev,
                                                    const StepState *__restrict__ st, float *__restrict__ out32, bf16 *__restrict__ out16) {
    const int r = blockIdx.x;
    const bool zero = r == 0 && st->pos == 0;
    const float *p = r > 0 ? x + (size_t)(r - 1) * E : prev;
    for (int i = threadIdx.x; i < E; i += 256) {
        const float v = x[(size_t)r * E + i];
        const float h = fmaf((zero ? 0.0f : p[i]) - v, shift[i], v);
        if (out32) out32[(size_t)r * E + i] = h;
        if (out16) out16[(size_t)r * E + i] = __float2bfloat16_rn(h);
    }
}

// Activation over FP32 rows: out[r][i] = act(in[r * ldi + i]), i < F.  grid (n), 256 threads.
__global__ void __launch_bounds__(256) k_act_rows(const float *__restrict__ in, int ldi, int F, int act, bf16 *__restrict__ out16, int ldo) {
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < F; i += 256) out16[(size_t)r * ldo + i] = __float2bfloat16_rn(act_apply(act, in[(size_t)r * ldi + i]));
}

// ---------------------------------------------------------------------------------------------------------------------
// Causal convolution per channel.  Channel c of row r (position p = st->pos + r) reads the inputs in(p - taps + 1 .. p) with
// in(q) = P[q's row][c_off + c] + bias_in[c]: from the rows of this launch where they belong to it, else from the ring `cstate`
// (position q in slot q % cring, written by earlier launches; cring >= taps - 1 + rows of a launch); positions before the start
// of the sequence count as zero.  out = act(sum_m w[c][m] in(p - taps + 1 + m) + bias_out[c]).  grid (ceil(n / LY_CONV_ROWS), ceil(C / 256)).
// ---------------------------------------------------------------------------------------------------------------------
struct ConvArgs {
    int C, taps, cring;
    const float *w;        // [C][taps], the last tap belongs to the current token
    const float *bias_in;  // [C] (nullable)
    const float *bias_out; // [C] (nullable)
    int silu;              // 1: SiLU on the result
};
#define LY_CONV_ROWS 4 // consecutive rows of a channel per thread: their loads are independent and in flight together
__global__ void __launch_bounds__(256) k_conv_rows(const float *__restrict__ P, int ldp, int c_off, ConvArgs a, float *__restrict__ cstate, float *__restrict__ out32, int ldo,
                                                   bf16 *__restrict__ out16, int ldo16, const StepState *__restrict__ st, int n) {
    const int r0 = blockIdx.x * LY_CONV_ROWS, c = blockIdx.y * 256 + threadIdx.x;
    if (c >= a.C) return;
    const float bi = a.bias_in ? a.bias_in[c] : 0.0f, bo = a.bias_out ? a.bias_out[c] : 0.0f;
    float acc[LY_CONV_ROWS];
#pragma unroll
    for (int i = 0; i < LY_CONV_ROWS; i++) acc[i] = bo;
    for (int m = 0; m < a.taps; m++) {
        const int back = a.taps - 1 - m;
        const float wm = a.w[(size_t)c * a.taps + m];
#pragma unroll
        for (int i = 0; i < LY_CONV_ROWS; i++) {
            const int r = r0 + i, pos = st->pos + r;
            if (r >= n || pos - back < 0) continue;
            const float x = back <= r ? P[(size_t)(r - back) * ldp + c_off + c] + bi : cstate[(size_t)((pos - back) % a.cring) * a.C + c];
            acc[i] = fmaf(wm, x, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < LY_CONV_ROWS; i++) {
        const int r = r0 + i, pos = st->pos + r;
        if (r >= n) break;
        // a later launch reads at most taps - 1 rows back
        if (r + a.taps > n) cstate[(size_t)(pos % a.cring) * a.C + c] = P[(size_t)r * ldp + c_off + c] + bi;
        float v = acc[i];
        if (a.silu) v = v / (1.0f + expf(-v));
        if (out32) out32[(size_t)r * ldo + c] = v;
        if (out16) out16[(size_t)r * ldo16 + c] = __float2bfloat16_rn(v);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Real-gated linear recurrent unit over W channels in `blocks` diagonal blocks of bs = W / blocks.
//   U [n][ldu]: convolved input u;  G [n][ldg] = [block][r logits (bs) | i logits (bs)] without their biases (gate_bias has the same layout);
//   PY [n][ldp]: the other branch before its bias and GELU.
//   a = exp(-8 sigmoid(r) softplus(lam)),  S <- a S + sqrt(1 - a^2) sigmoid(i) u  (from S = 0 at position 0),  out = S * gelu_tanh(PY + y_bias).
// CTA = CW channels x `groups` row groups (blockDim = CW * groups).  A chunk of many rows is scanned on two levels: every group
// folds its rows into (product of a, accumulated input) from a zero state, the groups' carries are chained through shared
// memory, then every group runs its rows again from its true incoming state and writes them; a group of at most RGLRU_KEEP rows
// keeps its coefficients in registers between the two passes.  Few rows: one group, one pass.
// ---------------------------------------------------------------------------------------------------------------------
struct RglruArgs {
    int W, blocks;
    const float *gate_bias; // [blocks][2 * bs]
    const float *lam;       // [W]
    const float *y_bias;    // [W]
};
#define RGLRU_MAX_GROUPS 32
#define RGLRU_KEEP 16
template <int CW, int MAXG> // MAXG = 1: the one-group form only (a launch of CW threads)
__global__ void __launch_bounds__(CW * MAXG) k_rglru_scan(const float *__restrict__ U, int ldu, const float *__restrict__ G, int ldg, const float *__restrict__ PY, int ldp,
                                                                      RglruArgs a, float *__restrict__ S, int n, const StepState *__restrict__ st, float *__restrict__ out32,
                                                                      bf16 *__restrict__ out16, int ldo) {
    __shared__ float cA[MAXG][CW], cB[MAXG][CW];
    const int cl = threadIdx.x % CW, g = threadIdx.x / CW, c = blockIdx.x * CW + cl, groups = blockDim.x / CW;
    const bool live = c < a.W;
    const int bs = a.W / a.blocks, blk = live ? c / bs : 0, j = live ? c % bs : 0;
    const int go = blk * 2 * bs + j; // column of this channel's r logit in a G row; the i logit sits bs further
    const float rb = live ? a.gate_bias[go] : 0.0f, ib = live ? a.gate_bias[go + bs] : 0.0f;
    const float sp8 = live ? 8.0f * softplusf_(a.lam[c]) : 0.0f, yb = live ? a.y_bias[c] : 0.0f;
    const int chunk = (n + groups - 1) / groups, t0 = g * chunk, t1 = t0 + chunk < n ? t0 + chunk : n;
    auto coef = [&](int t, float &av, float &bv) {
        const float *gr = G + (size_t)t * ldg + go;
        const float la = -sp8 * sigmoidf_(gr[0] + rb);
        av = expf(la);
        bv = sqrtf(-expm1f(2.0f * la)) * sigmoidf_(gr[bs] + ib) * U[(size_t)t * ldu + c]; // 1 - a^2 = -expm1(2 log a)
    };
    auto emit = [&](int t, float s) {
        const float o = s * act_apply(ACT_GELU_TANH, PY[(size_t)t * ldp + c] + yb);
        if (out32) out32[(size_t)t * ldo + c] = o;
        if (out16) out16[(size_t)t * ldo + c] = __float2bfloat16_rn(o);
    };
    float s = (st->pos == 0 || !live) ? 0.0f : S[c];
    if (groups == 1) {
        if (!live) return;
        for (int t = 0; t < n; t++) {
            float av, bv;
            coef(t, av, bv);
            s = fmaf(av, s, bv);
            emit(t, s);
        }
        S[c] = s;
        return;
    }
    if constexpr (MAXG == 1) return;
    const bool keep = chunk <= RGLRU_KEEP;
    float ka[RGLRU_KEEP], kb[RGLRU_KEEP], ku[RGLRU_KEEP], kp[RGLRU_KEEP];
    float A = 1.0f, B = 0.0f;
    if (live) {
        if (keep) { // all of the group's loads (both gate logits, the input, the other branch) are in flight before the first is used
#pragma unroll
            for (int i = 0; i < RGLRU_KEEP; i++) {
                const bool in = t0 + i < t1;
                const size_t t = in ? t0 + i : 0;
                ka[i] = in ? __ldg(G + t * ldg + go) : 0.0f;
                kb[i] = in ? __ldg(G + t * ldg + go + bs) : 0.0f;
                ku[i] = in ? __ldg(U + t * ldu + c) : 0.0f;
                kp[i] = in ? __ldg(PY + t * ldp + c) : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < RGLRU_KEEP; i++)
                if (t0 + i < t1) {
                    const float la = -sp8 * sigmoidf_(ka[i] + rb);
                    ka[i] = expf(la);
                    kb[i] = sqrtf(-expm1f(2.0f * la)) * sigmoidf_(kb[i] + ib) * ku[i];
                    kp[i] = act_apply(ACT_GELU_TANH, kp[i] + yb);
                    A *= ka[i];
                    B = fmaf(ka[i], B, kb[i]);
                }
        } else {
            for (int t = t0; t < t1; t++) {
                float av, bv;
                coef(t, av, bv);
                A *= av;
                B = fmaf(av, B, bv);
            }
        }
    }
    cA[g][cl] = A; cB[g][cl] = B;
    __syncthreads();
    if (!live) return;
    for (int k = 0; k < g; k++) s = fmaf(cA[k][cl], s, cB[k][cl]);
    if (keep) {
#pragma unroll
        for (int i = 0; i < RGLRU_KEEP; i++)
            if (t0 + i < t1) {
                s = fmaf(ka[i], s, kb[i]);
                const float o = s * kp[i];
                if (out32) out32[(size_t)(t0 + i) * ldo + c] = o;
                if (out16) out16[(size_t)(t0 + i) * ldo + c] = __float2bfloat16_rn(o);
            }
    } else {
        for (int t = t0; t < t1; t++) {
            float av, bv;
            coef(t, av, bv);
            s = fmaf(av, s, bv);
            emit(t, s);
        }
    }
    if (t1 == n && t0 < n) S[c] = s;
}

// ---------------------------------------------------------------------------------------------------------------------
// State-space recurrence with a matrix state per head.  XBC [n][ldx] = [x: heads * P | B: groups * N | C: groups * N] (convolved,
// SiLU applied), DT [n][lddt]: dt before its bias and softplus.  Per head h (group h / (heads / groups)):
//   dt = softplus(DT + dt_bias),  S <- exp(-exp(a_log) dt) S + dt B x^T  (S [N][P], zero at position 0),  y = S^T C + D x.
// grid (heads, ceil(P / SSD_COLS)), SSD_THREADS threads: sixteen lanes share a state column, lane `slice` holds R of its rows (see ssd_rows)
// in registers (R = ceil(N / 16) rounded up to a power of two; rows beyond N stay zero); tokens are staged 8 or 16 at a time
// in shared memory (double buffered).  The state is kept in the kernel's own order: ssd_state_floats() floats per layer run.
// ---------------------------------------------------------------------------------------------------------------------
struct SsdArgs {
    int heads, groups, N, P;
    const float *a_log, *dt_bias, *D; // [heads]
};
#define SSD_COLS 16
#define SSD_THREADS (SSD_COLS * 16)
#define SSD_TB_OF(R) ((R) >= 16 ? 8 : 16) // tokens per staged batch: two buffers of B and C rows stay below 48 KB of static shared memory
__host__ __device__ inline int ssd_reg_rows(int N) { const int q = (N + 15) / 16; return q <= 1 ? 1 : q <= 2 ? 2 : q <= 4 ? 4 : q <= 8 ? 8 : q <= 16 ? 16 : 0; }
__host__ __device__ inline size_t ssd_state_floats(int heads, int N, int P) { return (size_t)heads * ((P + SSD_COLS - 1) / SSD_COLS) * ssd_reg_rows(N) * SSD_THREADS; }

// The R state rows of lane `slice` out of a staged token's 16 R rows: for R a multiple of 4 the rows (16 k + slice) * 4 + j, j < 4,
// k < R / 4 (sixteen lanes read consecutive 16-byte words: no bank conflicts), else the rows slice * R + i.
template <int R>
__device__ __forceinline__ void ssd_rows(const float *tile, int slice, float (&v)[R]) {
    if constexpr (R % 4 == 0) {
#pragma unroll
        for (int k = 0; k < R / 4; k++) {
            const float4 q = *reinterpret_cast<const float4 *>(tile + (16 * k + slice) * 4);
            v[4 * k] = q.x; v[4 * k + 1] = q.y; v[4 * k + 2] = q.z; v[4 * k + 3] = q.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < R; i++) v[i] = tile[slice * R + i];
    }
}

// Tokens are staged SSD_TB_OF(R) at a time through two shared-memory buffers with cp.async: the next batch's B, C, x and dt land
// while this one is computed.  Lane t of every sixteen turns token t's dt into (step, decay) once per batch; the column's lanes
// fetch them with a shuffle.
template <int R>
__global__ void __launch_bounds__(SSD_THREADS) k_ssd_scan(const float *__restrict__ XBC, int ldx, const float *__restrict__ DT, int lddt, SsdArgs a, float *__restrict__ S, int n,
                                                          const StepState *__restrict__ st, float *__restrict__ Y, int ldy) {
    constexpr int RW = R * 16;                  // staged state rows per token (rows beyond N are zero)
    constexpr int SSD_TB = SSD_TB_OF(R);
    constexpr int LB = SSD_TB * R / 16;         // elements of a batch's B (or C) tile per thread
    __shared__ __align__(16) float Bs[2][SSD_TB][RW], Cs[2][SSD_TB][RW];
    __shared__ float xs[2][SSD_TB][SSD_COLS], draw[2][16];
    const int h = blockIdx.x, tid = threadIdx.x, slice = tid & 15, cc = tid >> 4, col = blockIdx.y * SSD_COLS + cc;
    const int grp = h / (a.heads / a.groups);
    const int xo = h * a.P, bo = a.heads * a.P + grp * a.N, co = a.heads * a.P + a.groups * a.N + grp * a.N;
    float *Sg = S + ((size_t)h * gridDim.y + blockIdx.y) * R * SSD_THREADS + tid;
    float s[R];
    const bool fresh = st->pos == 0;
#pragma unroll
    for (int i = 0; i < R; i++) s[i] = fresh ? 0.0f : Sg[(size_t)i * SSD_THREADS];
    const float na = -expf(a.a_log[h]), dtb = a.dt_bias[h], Dh = a.D[h];
    const int xt = tid / SSD_COLS, xi = tid % SSD_COLS, xg = blockIdx.y * SSD_COLS + xi;
    // element e = tid + k * SSD_THREADS of a batch's [SSD_TB][RW] tile: token e / RW, state row e % RW
    auto fetch = [&](int t0, int buf) {
        const int nt = n - t0 < SSD_TB ? n - t0 : SSD_TB;
#pragma unroll
        for (int k = 0; k < LB; k++) {
            const int e = tid + k * SSD_THREADS, t = e / RW, i = e % RW;
            const bool ok = t < nt && i < a.N;
            const float *row = XBC + (size_t)(t0 + (ok ? t : 0)) * ldx;
            cp_async4(&Bs[buf][0][0] + e, ok ? row + bo + i : XBC, ok);
            cp_async4(&Cs[buf][0][0] + e, ok ? row + co + i : XBC, ok);
        }
        if (xt < SSD_TB) {
            const bool ok = xt < nt && xg < a.P;
            cp_async4(&xs[buf][xt][xi], ok ? XBC + (size_t)(t0 + xt) * ldx + xo + xg : XBC, ok);
        }
        if (tid < 16) cp_async4(&draw[buf][tid], tid < nt ? DT + (size_t)(t0 + tid) * lddt + h : DT, tid < nt);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(0, 0);
    int buf = 0;
    for (int t0 = 0; t0 < n; t0 += SSD_TB, buf ^= 1) {
        const int nt = n - t0 < SSD_TB ? n - t0 : SSD_TB;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads(); // this batch has landed for every thread, and the other buffer's batch is consumed
        if (t0 + SSD_TB < n) fetch(t0 + SSD_TB, buf ^ 1);
        const float my_dt = softplusf_(draw[buf][slice] + dtb), my_dec = expf(na * my_dt); // token `slice` of the batch
        int tb = 0;
        for (; tb + 4 <= nt; tb += 4) { // four tokens: four independent read-out sums, reduced over the sixteen lanes with five shuffles
            float acc[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int t = tb + u;
                const float dA = __shfl_sync(0xffffffffu, my_dec, t, 16), dx = __shfl_sync(0xffffffffu, my_dt, t, 16) * xs[buf][t][cc];
                float bv[R], cv[R];
                ssd_rows<R>(Bs[buf][t], slice, bv);
                ssd_rows<R>(Cs[buf][t], slice, cv);
                float ac = 0.0f;
#pragma unroll
                for (int i = 0; i < R; i++) {
                    s[i] = fmaf(dA, s[i], dx * bv[i]);
                    ac = fmaf(s[i], cv[i], ac);
                }
                acc[u] = ac;
            }
            const bool hi8 = slice & 8, hi4 = slice & 4;
            float p0 = hi8 ? acc[2] : acc[0], p1 = hi8 ? acc[3] : acc[1];
            p0 += __shfl_xor_sync(0xffffffffu, hi8 ? acc[0] : acc[2], 8);
            p1 += __shfl_xor_sync(0xffffffffu, hi8 ? acc[1] : acc[3], 8);
            float v = hi4 ? p1 : p0;
            v += __shfl_xor_sync(0xffffffffu, hi4 ? p0 : p1, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            const int t = tb + (slice >> 2); // lanes 0, 4, 8, 12 of a column hold the sums of tokens tb .. tb + 3
            if ((slice & 3) == 0 && col < a.P) Y[(size_t)(t0 + t) * ldy + xo + col] = fmaf(Dh, xs[buf][t][cc], v);
        }
        for (int t = tb; t < nt; t++) {
            const float dA = __shfl_sync(0xffffffffu, my_dec, t, 16), xv = xs[buf][t][cc], dx = __shfl_sync(0xffffffffu, my_dt, t, 16) * xv;
            float bv[R], cv[R];
            ssd_rows<R>(Bs[buf][t], slice, bv);
            ssd_rows<R>(Cs[buf][t], slice, cv);
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < R; i++) {
                s[i] = fmaf(dA, s[i], dx * bv[i]);
                acc = fmaf(s[i], cv[i], acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            if (slice == 0 && col < a.P) Y[(size_t)(t0 + t) * ldy + xo + col] = fmaf(Dh, xv, acc);
        }
    }
#pragma unroll
    for (int i = 0; i < R; i++) Sg[(size_t)i * SSD_THREADS] = s[i];
}

// out = GN(y * silu(z); w) with GN an RMS norm in `groups` equal consecutive parts of the row (n_in entries).  One CTA per row (any
// multiple of 32 threads), dynamic shared memory: n_in floats.
__global__ void __launch_bounds__(1024) k_gated_group_norm(const float *__restrict__ Yv, int ldy, const float *__restrict__ Z, int ldz, const float *__restrict__ w, int n_in,
                                                          int groups, float eps, float *__restrict__ out32, bf16 *__restrict__ out16, int ldo) {
    extern __shared__ __align__(16) float gv[];
    __shared__ float red[32];
    __shared__ float inv[LY_OUTNORM_MAX_GROUPS];
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < n_in; i += blockDim.x) {
        const float z = Z[(size_t)r * ldz + i];
        gv[i] = Yv[(size_t)r * ldy + i] * (z / (1.0f + expf(-z)));
    }
    __syncthreads();
    group_inv_rms(gv, n_in, groups, eps, inv, red);
    const int part = n_in / groups;
    for (int i = threadIdx.x; i < n_in; i += blockDim.x) {
        const float v = gv[i] * inv[i / part] * w[i];
        if (out32) out32[(size_t)r * ldo + i] = v;
        if (out16) out16[(size_t)r * ldo + i] = __float2bfloat16_rn(v);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Attention preparation with a norm per slice.  Projection row [q: q_slices * dk | k: k_slices * dk | v: v_width] (has_kv == 0: q
// only; the layer reads another layer's rings).  Every dk slice is divided by its root mean square (+ eps inside the root) and
// multiplied by qnorm / knorm [dk], then its first rope_dims entries turn by the table's angles of the row's position.  q stays in
// place, k and v go to the ring slot of the position (FP32 + optional BF16 twin rows).  One CTA per row, a warp per slice.
// ---------------------------------------------------------------------------------------------------------------------
struct SliceNormRopeArgs {
    int q_slices, k_slices, dk, v_width, has_kv;
    const float *qnorm, *knorm; // [dk]
    const float *cs;            // rotation table [positions][rope_dims / 2][2] = (cos, sin), magnitude factor included
    int rope_dims, rope_layout;
    float eps;
    int ring;
};
__global__ void __launch_bounds__(256) k_slice_norm_rope(float *__restrict__ P, int ldp, SliceNormRopeArgs a, float *__restrict__ kc, float *__restrict__ vc, bf16 *__restrict__ kc16,
                                                         bf16 *__restrict__ vc16, const StepState *__restrict__ st) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = st->pos + r, half = a.rope_dims / 2, slot = pos % a.ring;
    const int kd = a.k_slices * a.dk, qd = a.q_slices * a.dk;
    float *p = P + (size_t)r * ldp;
    const float *cs = a.cs + (size_t)pos * half * 2;
    const int slices = a.q_slices + (a.has_kv ? a.k_slices : 0);
    for (int s = warp; s < slices; s += 8) {
        const bool isq = s < a.q_slices;
        float *src = p + (size_t)s * a.dk;
        const float *w = isq ? a.qnorm : a.knorm;
        float ss = 0.0f;
        for (int i = lane; i < a.dk; i += 32) ss = fmaf(src[i], src[i], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)a.dk + a.eps);
        float *d32 = isq ? src : kc + (size_t)slot * kd + (size_t)(s - a.q_slices) * a.dk;
        bf16 *d16 = (!isq && kc16) ? kc16 + (size_t)slot * kd + (size_t)(s - a.q_slices) * a.dk : nullptr;
        __syncwarp();
        for (int i = lane; i < half; i += 32) {
            int u, v;
            rope_pair_index(i, a.rope_dims, a.rope_layout, u, v);
            const float xu = src[u] * inv * w[u], xv = src[v] * inv * w[v];
            const float co = cs[2 * i], si = cs[2 * i + 1];
            const float ru = xu * co - xv * si, rv = xv * co + xu * si;
            d32[u] = ru; d32[v] = rv;
            if (d16) { d16[u] = __float2bfloat16_rn(ru); d16[v] = __float2bfloat16_rn(rv); }
        }
        for (int i = a.rope_dims + lane; i < a.dk; i += 32) {
            const float x = src[i] * inv * w[i];
            d32[i] = x;
            if (d16) d16[i] = __float2bfloat16_rn(x);
        }
    }
    if (a.has_kv)
        for (int i = threadIdx.x; i < a.v_width; i += 256) {
            const float v = p[qd + kd + i];
            vc[(size_t)slot * a.v_width + i] = v;
            if (vc16) vc16[(size_t)slot * a.v_width + i] = __float2bfloat16_rn(v);
        }
}

// Differential attention: A [n][heads][2][dv] = per head the results of map 1 and map 2; o = a1 - lambda a2, normalised to o / sqrt(mean(o^2) + eps)
// over the head's dv values times out_scale.  One CTA per row, a warp per head.
__global__ void __launch_bounds__(256) k_diff_combine(const float *__restrict__ A, int lda, int heads, int dv, float lambda, float out_scale, float eps, float *__restrict__ out32,
                                                      bf16 *__restrict__ out16, int ldo) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int h = warp; h < heads; h += 8) {
        const float *a1 = A + (size_t)r * lda + (size_t)h * 2 * dv, *a2 = a1 + dv;
        float ss = 0.0f;
        for (int i = lane; i < dv; i += 32) { const float o = fmaf(-lambda, a2[i], a1[i]); ss = fmaf(o, o, ss); }
        ss = warp_sum(ss);
        const float inv = out_scale / sqrtf(ss / (float)dv + eps);
        for (int i = lane; i < dv; i += 32) {
            const float o = fmaf(-lambda, a2[i], a1[i]) * inv;
            if (out32) out32[(size_t)r * ldo + (size_t)h * dv + i] = o;
            if (out16) out16[(size_t)r * ldo + (size_t)h * dv + i] = __float2bfloat16_rn(o);
        }
    }
}

} // namespace ly
