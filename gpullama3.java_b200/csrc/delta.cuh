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
//   * k_delta_rule      the recurrence S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, one thread per state column,
//                       rows of a chunk in sequence, the state tile resident in shared memory for the whole chunk;
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

// One CTA per row.  P row: [q: heads*dk | k: kv_heads*dk | v: kv_heads*dv (absent with value_from_key) | ...]; q and k are
// rotated in place.  Q row (ldq): heads * (talk ? kv_heads * dk : dk) entries.
__global__ void __launch_bounds__(256) k_rope_mix_prep(float *__restrict__ P, int ldp, RopeMixArgs a, const float *__restrict__ bias, float *__restrict__ Q, int ldq,
                                                       float *__restrict__ kc, float *__restrict__ vc, bf16 *__restrict__ kc16, bf16 *__restrict__ vc16,
                                                       const StepState *__restrict__ st) {
    const int r = blockIdx.x, tid = threadIdx.x;
    const int qd = a.heads * a.dk, kd = a.kv_heads * a.dk, vd = a.kv_heads * a.dv, pv = a.value_from_key ? 0 : vd;
    float *q = P + (size_t)r * ldp, *k = q + qd;
    const float *v = a.value_from_key ? k : k + kd;
    const int pos = st->pos + r, slot = pos % a.ring;
    if (bias) {
        for (int i = tid; i < qd + kd + pv; i += 256) q[i] += bias[i];
        __syncthreads();
    }
    for (int i = tid; i < vd; i += 256) {
        vc[(size_t)slot * vd + i] = v[i];
        if (vc16) vc16[(size_t)slot * vd + i] = __float2bfloat16_rn(v[i]);
    }
    if (a.rope_dims > 0) {
        __syncthreads(); // the values above are read from the unrotated keys
        const int half = a.rope_dims / 2;
        const float *cs = a.cs + (size_t)pos * half * 2;
        for (int e = tid; e < (a.heads + a.kv_heads) * half; e += 256) {
            const int hd = e / half, i = e % half;
            int u, w;
            rope_pair_index(i, a.rope_dims, a.rope_layout, u, w);
            float *x = q + (size_t)hd * a.dk; // the key heads follow the query heads in the row
            const float co = cs[2 * i], si = cs[2 * i + 1];
            const float xu = x[u], xw = x[w];
            x[u] = fmaf(xu, co, -(xw * si));
            x[w] = fmaf(xw, co, xu * si);
        }
    }
    __syncthreads();
    for (int i = tid; i < kd; i += 256) {
        kc[(size_t)slot * kd + i] = k[i];
        if (kc16) kc16[(size_t)slot * kd + i] = __float2bfloat16_rn(k[i]);
    }
    float *qo = Q + (size_t)r * ldq;
    if (a.talk) {
        const int group = a.heads / a.kv_heads, row = kd;
        for (int e = tid; e < a.heads * row; e += 256) {
            const int h = e / row, c = e % row, kv = c / a.dk, d = c % a.dk;
            float s = 0.0f;
            for (int m = kv * group; m < (kv + 1) * group; m++) s = fmaf(a.talk[h * a.heads + m] * (a.temp ? a.temp[m] : 1.0f), q[(size_t)m * a.dk + d], s);
            qo[e] = s;
        }
    } else {
        for (int e = tid; e < qd; e += 256) qo[e] = a.temp ? q[e] * a.temp[e / a.dk] : q[e];
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

// One CTA per row; dynamic shared memory: delta_channels floats.  A row at position p reads the inputs of positions p - taps + 1
// .. p: from the rows of this launch where they belong to it, else from the ring (written by earlier launches; positions before
// the start of the sequence count as zero).  Every row leaves its own input in the ring.
__global__ void __launch_bounds__(256) k_delta_prep(const float *__restrict__ P, int ldp, DeltaArgs a, float *__restrict__ cstate, float *__restrict__ D, int ldd,
                                                    const StepState *__restrict__ st) {
    extern __shared__ __align__(16) float row[];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = delta_channels(a), qk = a.kv_heads * a.dk;
    const int pos = st->pos + r;
    const float *p = P + (size_t)r * ldp;
    for (int c = tid; c < C; c += 256) {
        float acc = 0.0f;
        for (int m = 0; m < a.taps; m++) {
            const int back = a.taps - 1 - m;
            if (pos - back < 0) continue;
            const float x = back <= r ? P[(size_t)(r - back) * ldp + c] : cstate[(size_t)((pos - back) % a.cring) * C + c];
            acc = fmaf(a.conv_w[(size_t)c * a.taps + m], x, acc);
        }
        cstate[(size_t)(pos % a.cring) * C + c] = p[c];
        row[c] = acc / (1.0f + expf(-acc));
    }
    __syncthreads();
    float *d = D + (size_t)r * ldd;
    // q heads then k heads: one warp per head
    for (int hd = warp; hd < 2 * a.kv_heads; hd += 8) {
        const float *x = row + (size_t)hd * a.dk;
        float ss = 0.0f;
        for (int i = lane; i < a.dk; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        float inv = 1.0f / sqrtf(ss + a.unit_eps);
        if (hd < a.kv_heads) inv *= 1.0f / sqrtf((float)a.dk);
        for (int i = lane; i < a.dk; i += 32) d[(size_t)hd * a.dk + i] = x[i] * inv;
    }
    for (int c = 2 * qk + tid; c < C; c += 256) d[c] = row[c];
    for (int h = tid; h < a.heads; h += 256) {
        d[C + h] = 1.0f / (1.0f + expf(-p[C + h]));
        const float z = p[C + a.heads + h] + a.dt_bias[h];
        const float sp = fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z)));
        d[C + a.heads + h] = expf(-expf(a.a_log[h]) * sp);
    }
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
