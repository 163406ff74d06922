// delta.cuh -- device kernels of the two mixers of pre-norm layered plans (B200_BLOCK_PRENORM).  First user: Lerosun.
//
//   * k_rope_mix_prep   windowed attention with rotated, head-mixed scores: projection biases, value rows = the keys BEFORE the
//                       rotation (or a value projection of their own), table-driven rotation of the leading entries of every
//                       query / key head, key / value rows into the window ring, and the head mixing FOLDED INTO THE QUERY:
//                           e'_h(i, j) = sum_m T[h][m] t_m <q_i^m, k_j^g(m)> = < q'_i^h , [k_j^0 | k_j^1 | ...] >,
//                           q'_i^h = [ sum_{m in group 0} T[h][m] t_m q_i^m | sum_{m in group 1} ... | ... ]
//                       so every head attends with ONE query of (key heads x key size) entries over the whole key row and the
//                       attention kernels of layered.cuh need no mixing pass (WindowAttn::k_heads = 1).  Without a mixing
//                       matrix the query is only scaled by its head's temperature;
//   * k_delta_prep      gated delta rule, everything in front of the recurrence: causal convolution of the q | k | v channels over
//                       a ring of earlier inputs, SiLU, unit vectors per q / k head, beta = sigmoid, decay = exp(-exp(A) softplus);
//   * k_delta_rule_reg  the recurrence S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q with the state in registers: eight
//                       lanes share a state column, the rows of a chunk run in sequence, columns in parallel over warps and CTAs;
//   * k_delta_rule      the same for key sizes above 128: one thread per state column, the state tile in shared memory;
//   * k_head_norm_gate  per-head RMS norm of the read-out, weight, SiLU gate.
// Rotation, scores, decays, gates, unit norms and the state are FP32 in both compute modes; fmaf is explicit because the
// translation unit is compiled with -fmad=false.
#pragma once
#include "latent.cuh"

namespace ly {

struct RopeMixArgs {
    int heads, kv_heads, dk, dv; // query heads, key/value heads, key size, value size (value_from_key: dv == dk)
    int rope_dims, rope_layout;  // the first rope_dims entries of every head turn (0: none)
    const float *cs;             // [position][rope_dims / 2][2] = (cos, sin)
    const float *temp;           // [heads] (nullable)
    const float *talk;           // [heads][heads] (nullable): mixing matrix T
    int value_from_key;
    int ring;                    // position j lives in slot j % ring
};

// grid (rows, ceil(heads / hpc) + 1), 128 threads (hpc = query heads per CTA: ROPE_MIX_HEADS for a chunk of rows, 1 for the decode step's single row); dynamic shared memory: max(heads, kv_heads) * dk floats.  P row:
// [q: heads*dk | k: kv_heads*dk | v: kv_heads*dv (absent with value_from_key) | ...].  A query-side CTA biases and rotates ALL query heads
// of the row into shared memory (every mixed query needs them all; the row in P stays as projected) and writes the queries of its
// hpc heads: heads * (talk ? kv_heads * dk : dk) entries per Q row (ldq).  The last CTA of a row owns the key side: bias,
// value row = unrotated key (or the value projection), rotation, key row.
#define ROPE_MIX_THREADS 128
#define ROPE_MIX_HEADS 4
__global__ void __launch_bounds__(ROPE_MIX_THREADS) k_rope_mix_prep(const float *__restrict__ P, int ldp, RopeMixArgs a, const float *__restrict__ bias, float *__restrict__ Q, int ldq,
                                                                    float *__restrict__ kc, float *__restrict__ vc, bf16 *__restrict__ kc16, bf16 *__restrict__ vc16,
                                                                    const StepState *__restrict__ st, int hpc) {
    extern __shared__ __align__(16) float xs[];
    const int r = blockIdx.x, tid = threadIdx.x;
    const int qd = a.heads * a.dk, kd = a.kv_heads * a.dk, vd = a.kv_heads * a.dv;
    const float *p = P + (size_t)r * ldp;
    const int pos = st->pos + r, slot = pos % a.ring, half = a.rope_dims / 2;
    const float *cs = a.cs + (size_t)pos * half * 2;
    const bool key_side = blockIdx.y == gridDim.y - 1;
    // this CTA's vectors, biased: all query heads, or all key heads
    const int off = key_side ? qd : 0, len = key_side ? kd : qd, nh = key_side ? a.kv_heads : a.heads;
    for (int i = tid; i < len; i += ROPE_MIX_THREADS) xs[i] = p[off + i] + (bias ? bias[off + i] : 0.0f);
    __syncthreads();
    if (key_side) {
        for (int i = tid; i < vd; i += ROPE_MIX_THREADS) {
            const float v = a.value_from_key ? xs[i] : p[qd + kd + i] + (bias ? bias[qd + kd + i] : 0.0f);
            vc[(size_t)slot * vd + i] = v;
            if (vc16) vc16[(size_t)slot * vd + i] = __float2bfloat16_rn(v);
        }
        __syncthreads(); // the values above are the unrotated keys
    }
    for (int e = tid; e < nh * half; e += ROPE_MIX_THREADS) {
        const int hd = e / half, i = e % half;
        int u, w;
        rope_pair_index(i, a.rope_dims, a.rope_layout, u, w);
        float *x = xs + (size_t)hd * a.dk;
        const float co = cs[2 * i], si = cs[2 * i + 1];
        const float xu = x[u], xw = x[w];
        x[u] = fmaf(xu, co, -(xw * si));
        x[w] = fmaf(xw, co, xu * si);
    }
    __syncthreads();
    if (key_side) {
        for (int i = tid; i < kd; i += ROPE_MIX_THREADS) {
            kc[(size_t)slot * kd + i] = xs[i];
            if (kc16) kc16[(size_t)slot * kd + i] = __float2bfloat16_rn(xs[i]);
        }
        return;
    }
    const int h0 = blockIdx.y * hpc, h1 = h0 + hpc < a.heads ? h0 + hpc : a.heads;
    if (a.talk) {
        const int group = a.heads / a.kv_heads;
        float *qo = Q + (size_t)r * ldq + (size_t)h0 * kd;
        for (int e = tid; e < (h1 - h0) * kd; e += ROPE_MIX_THREADS) {
            const int h = h0 + e / kd, c = e % kd, kv = c / a.dk, d = c % a.dk;
            float s = 0.0f;
            for (int m = kv * group; m < (kv + 1) * group; m++) s = fmaf(a.talk[h * a.heads + m] * (a.temp ? a.temp[m] : 1.0f), xs[(size_t)m * a.dk + d], s);
            qo[e] = s;
        }
    } else {
        float *qo = Q + (size_t)r * ldq;
        for (int e = h0 * a.dk + tid; e < h1 * a.dk; e += ROPE_MIX_THREADS) qo[e] = a.temp ? xs[e] * a.temp[e / a.dk] : xs[e];
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Gated delta rule.
// ---------------------------------------------------------------------------------------------------------------------
struct DeltaArgs {
    int heads, kv_heads, dk, dv; // value heads, query/key heads, key size, value size
    int taps;                    // convolution taps; tap taps - 1 belongs to the current token
    int cring;                   // slots of the ring of convolution inputs: position j in slot j % cring (cring >= taps - 1 + rows of a step)
    const float *conv_w;         // [2 * kv_heads * dk + heads * dv][taps]: q | k | v channels
    const float *a_log, *dt_bias; // [heads]
    float unit_eps;              // inside the root of the unit-vector normalisation
};
// Row layout of the fused projection: [q: kv_heads*dk | k: kv_heads*dk | v: heads*dv | b: heads | a: heads | g: heads*dv]
// Row layout of the prepared buffer D (ldd): [q unit / sqrt(dk) | k unit | v | beta: heads | decay: heads]
__host__ __device__ inline int delta_channels(const DeltaArgs &a) { return 2 * a.kv_heads * a.dk + a.heads * a.dv; }

// grid (rows, 2 * kv_heads + heads + 1), 128 threads; dynamic shared memory: max(dk, dv) floats.  CTA (r, u) owns one unit of the row:
// a query head, a key head (convolution, SiLU, unit vector), a value head (convolution, SiLU), or -- the last unit -- beta and decay
// of all heads.  A row at position p reads the inputs of positions p - taps + 1 .. p: from the rows of this launch where they belong
// to it, else from the ring (written by earlier launches; positions before the start of the sequence count as zero).  Every unit
// leaves its own input channels in the ring.
#define DELTA_PREP_THREADS 128
__global__ void __launch_bounds__(DELTA_PREP_THREADS) k_delta_prep(const float *__restrict__ P, int ldp, DeltaArgs a, float *__restrict__ cstate, float *__restrict__ D, int ldd,
                                                                   const StepState *__restrict__ st) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[32];
    const int r = blockIdx.x, u = blockIdx.y, tid = threadIdx.x;
    const int C = delta_channels(a), qk = a.kv_heads * a.dk;
    const int pos = st->pos + r;
    const float *p = P + (size_t)r * ldp;
    float *d = D + (size_t)r * ldd;
    if (u == 2 * a.kv_heads + a.heads) {
        for (int h = tid; h < a.heads; h += DELTA_PREP_THREADS) {
            d[C + h] = 1.0f / (1.0f + expf(-p[C + h]));
            const float z = p[C + a.heads + h] + a.dt_bias[h];
            const float sp = fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z)));
            d[C + a.heads + h] = expf(-expf(a.a_log[h]) * sp);
        }
        return;
    }
    const bool unit_vec = u < 2 * a.kv_heads;
    const int c0 = unit_vec ? u * a.dk : 2 * qk + (u - 2 * a.kv_heads) * a.dv, len = unit_vec ? a.dk : a.dv;
    float ss = 0.0f;
    for (int i = tid; i < len; i += DELTA_PREP_THREADS) {
        const int c = c0 + i;
        float acc = 0.0f;
        for (int m = 0; m < a.taps; m++) {
            const int back = a.taps - 1 - m;
            if (pos - back < 0) continue;
            const float x = back <= r ? P[(size_t)(r - back) * ldp + c] : cstate[(size_t)((pos - back) % a.cring) * C + c];
            acc = fmaf(a.conv_w[(size_t)c * a.taps + m], x, acc);
        }
        cstate[(size_t)(pos % a.cring) * C + c] = p[c];
        const float y = acc / (1.0f + expf(-acc));
        if (unit_vec) { row[i] = y; ss = fmaf(y, y, ss); }
        else d[c] = y;
    }
    if (!unit_vec) return;
    ss = block_sum(ss, red);
    float inv = 1.0f / sqrtf(ss + a.unit_eps);
    if (u < a.kv_heads) inv *= 1.0f / sqrtf((float)a.dk);
    for (int i = tid; i < len; i += DELTA_PREP_THREADS) d[c0 + i] = row[i] * inv;
}

// grid (heads, column tiles), DELTA_COLS threads: thread j owns column j of the head's state S [dk][dv]; the tile S[:, cols] stays
// in shared memory over the n rows of the launch.  Dynamic shared memory: (dk * DELTA_COLS + 4 * dk) floats.  pos == 0 starts
// from a zero state whatever the buffer holds (a new sequence needs no clearing).
#define DELTA_COLS 64
__host__ __device__ inline size_t delta_rule_smem_floats(int dk) { return (size_t)dk * DELTA_COLS + 4 * (size_t)dk; }

__global__ void __launch_bounds__(DELTA_COLS) k_delta_rule(const float *__restrict__ D, int ldd, DeltaArgs a, float *__restrict__ S, int n, float *__restrict__ O, int ldo,
                                                           const StepState *__restrict__ st) {
    extern __shared__ __align__(16) float sm[];
    const int h = blockIdx.x, j0 = blockIdx.y * DELTA_COLS, tid = threadIdx.x, j = j0 + tid;
    const int dk = a.dk, dv = a.dv, g = h / (a.heads / a.kv_heads), C = delta_channels(a);
    float *Ss = sm, *kq = sm + (size_t)dk * DELTA_COLS; // kq: two buffers of [k (dk) | q (dk)]
    float *Sg = S + (size_t)h * dk * dv;
    const bool live = j < dv;
    const bool fresh = st->pos == 0;
    for (int i = 0; i < dk; i++) Ss[i * DELTA_COLS + tid] = (live && !fresh) ? Sg[(size_t)i * dv + j] : 0.0f;
    auto stage = [&](int t, int buf) {
        const float *d = D + (size_t)t * ldd;
        float *dst = kq + (size_t)buf * 2 * dk;
        for (int i = tid; i < dk; i += DELTA_COLS) {
            dst[i] = d[(size_t)(a.kv_heads + g) * dk + i];
            dst[dk + i] = d[(size_t)g * dk + i];
        }
    };
    stage(0, 0);
    __syncthreads();
    for (int t = 0; t < n; t++) {
        const int buf = t & 1;
        if (t + 1 < n) stage(t + 1, buf ^ 1); // the other buffer was last read in iteration t - 1, before its closing barrier
        const float *ks = kq + (size_t)buf * 2 * dk, *qs = ks + dk;
        const float *d = D + (size_t)t * ldd;
        const float beta = d[C + h], decay = d[C + a.heads + h];
        const float vj = live ? d[2 * a.kv_heads * dk + (size_t)h * dv + j] : 0.0f;
        float rd = 0.0f;
        for (int i = 0; i < dk; i++) rd = fmaf(Ss[i * DELTA_COLS + tid], ks[i], rd);
        const float u = beta * (vj - decay * rd);
        float o = 0.0f;
        for (int i = 0; i < dk; i++) {
            const float s = fmaf(ks[i], u, decay * Ss[i * DELTA_COLS + tid]);
            Ss[i * DELTA_COLS + tid] = s;
            o = fmaf(s, qs[i], o);
        }
        if (live) O[(size_t)t * ldo + (size_t)h * dv + j] = o;
        __syncthreads();
    }
    if (live)
        for (int i = 0; i < dk; i++) Sg[(size_t)i * dv + j] = Ss[i * DELTA_COLS + tid];
}

// The same recurrence with the state in REGISTERS (key sizes up to 16 * R, R = 1, 2, 4 or 8): grid (heads, column tiles of DR_COLS),
// DR_THREADS threads.  A column of S is shared by DR_SLICES = 16 neighbouring lanes, lane s holding rows s * R .. s * R + R - 1; the two
// products S^T k and S^T q are R multiply-adds per lane (four partial sums) and a four-step shuffle.  Columns are independent and a
// warp owns two of them completely, so the only block-wide step is staging DR_TB tokens of k, q, v, beta and decay in shared memory
// at a time (cp.async, double buffered: the next block lands while this one is computed; slices of eight padded by four floats: the
// 128-bit reads of a quarter warp fall on distinct banks) and writing their read-outs back coalesced.  Within a token the chain
// S^T k -> shuffles -> u -> S is what the next token waits for; the read-out's shuffles ride one token behind, interleaved with it.
// Sixteen lanes per column rather than eight: the per-token chain gets shorter and every scheduler has two warps to alternate
// between.  The state buffer is private to this kernel: [head][tile][R][thread].
#define DR_COLS 16
#define DR_SLICES 16
#define DR_THREADS (DR_COLS * DR_SLICES)
#define DR_TB 8
__host__ __device__ inline int delta_reg_rows(int dk) { return dk <= 16 ? 1 : dk <= 32 ? 2 : dk <= 64 ? 4 : dk <= 128 ? 8 : 0; } // 0: the shared-memory kernel
__host__ __device__ inline size_t delta_state_floats(int heads, int dk, int dv) {
    const int R = delta_reg_rows(dk);
    return R ? (size_t)heads * ((dv + DR_COLS - 1) / DR_COLS) * R * DR_THREADS : (size_t)heads * dk * dv;
}

__device__ __forceinline__ void cp_async4(void *dst, const void *src, bool valid) { // 4 bytes, zero-filled when !valid
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int nbytes = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(nbytes) : "memory");
}

template <int R>
__global__ void __launch_bounds__(DR_THREADS) k_delta_rule_reg(const float *__restrict__ D, int ldd, DeltaArgs a, float *__restrict__ S, int n, float *__restrict__ O, int ldo,
                                                               const StepState *__restrict__ st) {
    constexpr int RP = R > 4 ? R + 4 : R, KR = DR_SLICES * RP; // floats per slice / per token in shared memory
    __shared__ __align__(16) float ks[2][DR_TB][KR], qs[2][DR_TB][KR];
    __shared__ float vs[2][DR_TB][DR_COLS], bd[2][DR_TB][2], os[DR_TB][DR_COLS];
    const int h = blockIdx.x, tile = blockIdx.y, j0 = tile * DR_COLS, tid = threadIdx.x, lane = tid & 31;
    const int c = (tid >> 5) * (32 / DR_SLICES) + lane / DR_SLICES, s = lane % DR_SLICES;
    const int dk = a.dk, dv = a.dv, g = h / (a.heads / a.kv_heads), C = delta_channels(a);
    float *Sg = S + ((size_t)h * gridDim.y + tile) * R * DR_THREADS + tid;
    float Sr[R];
    const bool fresh = st->pos == 0;
    // the tokens of block t0 travel global -> shared asynchronously while the previous block is computed
    auto stage = [&](int buf, int t0) {
        const int nb = n - t0 < DR_TB ? n - t0 : DR_TB;
        for (int e = tid; e < nb * DR_SLICES * R; e += DR_THREADS) {
            const int t = e / (DR_SLICES * R), i = e % (DR_SLICES * R); // key row i belongs to slice i / R
            const float *d = D + (size_t)(t0 + t) * ldd;
            const int at = (i / R) * RP + i % R;
            const bool ok = i < dk;
            cp_async4(&ks[buf][t][at], ok ? d + (size_t)(a.kv_heads + g) * dk + i : D, ok);
            cp_async4(&qs[buf][t][at], ok ? d + (size_t)g * dk + i : D, ok);
        }
        for (int e = tid; e < nb * DR_COLS; e += DR_THREADS) {
            const int t = e / DR_COLS, cc = e % DR_COLS;
            const bool ok = j0 + cc < dv;
            cp_async4(&vs[buf][t][cc], ok ? D + (size_t)(t0 + t) * ldd + 2 * a.kv_heads * dk + (size_t)h * dv + j0 + cc : D, ok);
        }
        if (tid < nb * 2) cp_async4(&bd[buf][tid >> 1][tid & 1], D + (size_t)(t0 + (tid >> 1)) * ldd + C + (tid & 1) * a.heads + h, true);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
#pragma unroll
    for (int i = 0; i < R; i++) Sr[i] = fresh ? 0.0f : Sg[(size_t)i * DR_THREADS];
    int buf = 0;
    for (int t0 = 0; t0 < n; t0 += DR_TB, buf ^= 1) {
        const int nb = n - t0 < DR_TB ? n - t0 : DR_TB;
        if (t0 + DR_TB < n) {
            stage(buf ^ 1, t0 + DR_TB); // that buffer was last read before the barrier that ended the previous iteration
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        auto load = [&](int t, float (&kr)[R], float (&qr)[R]) {
            if (R >= 4) {
#pragma unroll
                for (int i = 0; i < R; i += 4) {
                    *reinterpret_cast<float4 *>(&kr[i]) = *reinterpret_cast<const float4 *>(&ks[buf][t][s * RP + i]);
                    *reinterpret_cast<float4 *>(&qr[i]) = *reinterpret_cast<const float4 *>(&qs[buf][t][s * RP + i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < R; i++) { kr[i] = ks[buf][t][s * RP + i]; qr[i] = qs[buf][t][s * RP + i]; }
            }
        };
        float ka[R], qa[R], kb[R], qb[R]; // two register sets: the next token's k and q load while the current one's shuffles run
        load(0, ka, qa);
        float op = 0.0f; // read-out of the previous token, summed over the slices one shuffle step behind the current token's S^T k
        auto token = [&](int t, const float (&kr)[R], const float (&qr)[R], float (&kn)[R], float (&qn)[R]) {
            const float beta = bd[buf][t][0], decay = bd[buf][t][1], v = vs[buf][t][c];
            float r4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < R; i++) r4[i & 3] = fmaf(Sr[i], kr[i], r4[i & 3]);
            if (t + 1 < nb) load(t + 1, kn, qn); // in flight during the shuffles below
            float rd = (r4[0] + r4[1]) + (r4[2] + r4[3]);
#pragma unroll
            for (int m = 1; m < DR_SLICES; m <<= 1) {
                const float x = __shfl_xor_sync(0xffffffffu, rd, m), y = __shfl_xor_sync(0xffffffffu, op, m);
                rd += x;
                op += y;
            }
            if (s == 0 && t > 0) os[t - 1][c] = op;
            const float u = beta * (v - decay * rd);
            float o4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < R; i++) {
                Sr[i] = fmaf(kr[i], u, decay * Sr[i]);
                o4[i & 3] = fmaf(Sr[i], qr[i], o4[i & 3]);
            }
            op = (o4[0] + o4[1]) + (o4[2] + o4[3]);
        };
        for (int t = 0; t < nb; t += 2) {
            token(t, ka, qa, kb, qb);
            if (t + 1 < nb) token(t + 1, kb, qb, ka, qa);
        }
#pragma unroll
        for (int m = 1; m < DR_SLICES; m <<= 1) op += __shfl_xor_sync(0xffffffffu, op, m);
        if (s == 0) os[nb - 1][c] = op;
        __syncthreads();
        for (int e = tid; e < nb * DR_COLS; e += DR_THREADS) {
            const int t = e / DR_COLS, cc = e % DR_COLS;
            if (j0 + cc < dv) O[(size_t)(t0 + t) * ldo + (size_t)h * dv + j0 + cc] = os[t][cc];
        }
        // os is rewritten only after the barrier that follows the next block's wait
    }
#pragma unroll
    for (int i = 0; i < R; i++) Sg[(size_t)i * DR_THREADS] = Sr[i];
}

// One CTA per row, one warp per head: y = o / sqrt(mean(o^2) + eps) * w[d] * silu(gate[h][d]).
__global__ void __launch_bounds__(256) k_head_norm_gate(const float *__restrict__ O, int ldo, const float *__restrict__ G, int ldg, const float *__restrict__ w, int heads, int dv,
                                                        float eps, float *__restrict__ out32, bf16 *__restrict__ out16, int ldout) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int h = warp; h < heads; h += 8) {
        const float *o = O + (size_t)r * ldo + (size_t)h * dv, *g = G + (size_t)r * ldg + (size_t)h * dv;
        float ss = 0.0f;
        for (int i = lane; i < dv; i += 32) ss = fmaf(o[i], o[i], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
        for (int i = lane; i < dv; i += 32) {
            const float z = g[i];
            const float y = o[i] * inv * w[i] * (z / (1.0f + expf(-z)));
            if (out32) out32[(size_t)r * ldout + (size_t)h * dv + i] = y;
            if (out16) out16[(size_t)r * ldout + (size_t)h * dv + i] = __float2bfloat16_rn(y);
        }
    }
}

} // namespace ly
