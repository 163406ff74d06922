// latent.cuh -- device kernels of the layered plans' second family of mechanisms (first user: Latusun), beside those of
// layered.cuh and sharing its projection and attention kernels:
//   * k_block_norm_rows  the PARALLEL block's row kernel: x += mult * (a + sum of the feed-forward's per-slot results), then
//                        TWO norms of the same x (layer norm with weight and bias, one pair per branch) in one pass; also the
//                        embedding gather and the gathered final norm;
//   * k_latent_prep      latent attention: RMS norm of the key/value latent, rotation of the shared key part and of every
//                        head's rotated query part (table-driven: half-split or interleaved pairs, any blend of frequencies),
//                        cache write [latent | rotated shared key part];
//   * k_moe_route        router logits in FP32, sigmoid scores and selection of the `top` largest per row;
//   * k_moe_group        slots sorted by expert into tiles of 64 for the grouped projection kernels (GemmView);
//   * k_softcap          x <- cap * tanh(x / cap) over a logits buffer.
// The latent attention itself runs through k_window_attention: with W_uk folded into the query (q' = W_uk^T q_u per head)
// and W_uv applied to the attention's output, every head attends over the SAME cached row: keys = [latent | shared key part],
// values = latent -- one key/value "head" of size rank + dr / rank, never expanded per head.
// Norm statistics, router, softmax, rotation and the residual sum are FP32.
#pragma once
#include "layered.cuh"

namespace ly {

struct BlockNormArgs {
    float *x;             // [n][E] residual stream
    const bf16 *emb;      // embedding table [vocab][E]: x = emb_scale * emb[token] (nullable)
    const int *tokens;    // [n] (nullable: the step's own token)
    const StepState *st;
    float emb_scale;
    const float *add_a;   // [n][E] (nullable): mixer output of the previous layer
    const float *add_b;   // [n * add_b_terms][E] (nullable): feed-forward results, row r owns entries r * terms .. r * terms + terms - 1
    const int *add_b_map; // (nullable) entry e lives in row add_b_map[e] of add_b (results left in expert-sorted order)
    int add_b_terms;
    float add_mult;       // x += add_mult * (a + sum b)
    float *trace;         // [n][E]: copy of x after the update (nullable)
    const float *w1, *b1; // first norm (nullable: no output); b nullable
    float *out1_32;
    bf16 *out1_16;
    const float *w2, *b2; // second norm of the same x (nullable)
    float *out2_32;
    bf16 *out2_16;
    const int *gather;    // output row r is computed from x row gather[r] (no update then)
    int rms;              // 0: (x - mean) / sqrt(var + eps) * w + b;  1: x / sqrt(mean x^2 + eps) * w + b
    float eps;
    int E;
};

__global__ void __launch_bounds__(LY_NORM_THREADS) k_block_norm_rows(BlockNormArgs a) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[32];
    const int r = blockIdx.x, tid = threadIdx.x, E = a.E;
    const size_t src = (size_t)(a.gather ? a.gather[r] : r) * E, dst = (size_t)r * E;
    if (a.emb) {
        const int token = a.tokens ? a.tokens[r] : a.st->token;
        const bf16 *e = a.emb + (size_t)token * E;
        for (int i = tid; i < E; i += LY_NORM_THREADS) row[i] = __bfloat162float(e[i]) * a.emb_scale;
    } else {
        for (int i = tid; i < E; i += LY_NORM_THREADS) row[i] = a.x[src + i];
    }
    if (a.add_a || a.add_b) {
        for (int i = tid; i < E; i += LY_NORM_THREADS) {
            float s = a.add_a ? a.add_a[src + i] : 0.0f;
            for (int k = 0; k < a.add_b_terms; k++) {
                const size_t e = (size_t)r * a.add_b_terms + k;
                s += a.add_b[(a.add_b_map ? (size_t)a.add_b_map[e] : e) * E + i];
            }
            row[i] = fmaf(a.add_mult, s, row[i]);
        }
    }
    if (!a.gather && (a.emb || a.add_a || a.add_b))
        for (int i = tid; i < E; i += LY_NORM_THREADS) a.x[src + i] = row[i];
    if (a.trace)
        for (int i = tid; i < E; i += LY_NORM_THREADS) a.trace[src + i] = row[i];
    if (!a.w1 && !a.w2) return;
    float mean = 0.0f;
    if (!a.rms) {
        float s = 0.0f;
        for (int i = tid; i < E; i += LY_NORM_THREADS) s += row[i];
        mean = block_sum(s, red) / (float)E;
    }
    float ss = 0.0f;
    for (int i = tid; i < E; i += LY_NORM_THREADS) { const float d = row[i] - mean; ss = fmaf(d, d, ss); }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)E + a.eps);
    for (int i = tid; i < E; i += LY_NORM_THREADS) {
        const float u = (row[i] - mean) * inv;
        if (a.w1) {
            const float v = fmaf(u, a.w1[i], a.b1 ? a.b1[i] : 0.0f);
            if (a.out1_32) a.out1_32[dst + i] = v;
            if (a.out1_16) a.out1_16[dst + i] = __float2bfloat16_rn(v);
        }
        if (a.w2) {
            const float v = fmaf(u, a.w2[i], a.b2 ? a.b2[i] : 0.0f);
            if (a.out2_32) a.out2_32[dst + i] = v;
            if (a.out2_16) a.out2_16[dst + i] = __float2bfloat16_rn(v);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Latent attention, the part between the fused projection and the attention kernel.  One CTA per row.
// Projection row: [q: heads x (dk unrotated | dr rotated)] at q_off, [latent' (rank) | shared key part (dr)] at kv_off.
// ---------------------------------------------------------------------------------------------------------------------
struct LatentArgs {
    int heads, dk, dr, rank;
    int q_off, kv_off;   // kv_off < 0: the layer reads another layer's cache and writes none
    const float *cnorm;  // [rank] weight of the latent's RMS norm
    const float *cs;     // rotation table [positions][rope_dims / 2][2] = (cos, sin), magnitude factor included
    int rope_dims;       // the first rope_dims entries of a rotated part turn, the rest pass unchanged
    int rope_layout;     // 0: pair (i, i + rope_dims / 2);  1: pair (2i, 2i + 1)
    float eps;
};

__device__ __forceinline__ void rope_pair_index(int i, int dims, int layout, int &u, int &v) {
    if (layout) { u = 2 * i; v = 2 * i + 1; }
    else { u = i; v = i + dims / 2; }
}

// cache [ring][rank + dr];  Q [n][heads * (rank + dr)]: this kernel fills the rotated tail of every head, the folded-key
// product fills the first rank entries;  qu16 (nullable) [n][heads * dk]: BF16 copy of the unrotated query parts.
// The rotated query parts are also written back into the projection row (the expanded-key prefill reads [q_u | rot q_r] there).
// cache16 (nullable): BF16 twin of the cache row.
__global__ void __launch_bounds__(256) k_latent_prep(float *__restrict__ P, int ldp, LatentArgs a, float *__restrict__ cache, bf16 *__restrict__ cache16, int ring,
                                                     float *__restrict__ Q, bf16 *__restrict__ qu16, const StepState *__restrict__ st) {
    __shared__ float red[32];
    const int r = blockIdx.x, tid = threadIdx.x;
    const int pos = st->pos + r, half = a.rope_dims / 2, kw = a.rank + a.dr;
    float *p = P + (size_t)r * ldp;
    const float *cs = a.cs + (size_t)pos * half * 2;
    if (a.kv_off >= 0) {
        const float *c = p + a.kv_off, *kr = c + a.rank;
        float ss = 0.0f;
        for (int i = tid; i < a.rank; i += 256) ss = fmaf(c[i], c[i], ss);
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)a.rank + a.eps);
        float *row = cache + (size_t)(pos % ring) * kw;
        for (int i = tid; i < a.rank; i += 256) row[i] = c[i] * inv * a.cnorm[i];
        for (int i = tid; i < half; i += 256) {
            int u, v;
            rope_pair_index(i, a.rope_dims, a.rope_layout, u, v);
            const float co = cs[2 * i], si = cs[2 * i + 1];
            row[a.rank + u] = kr[u] * co - kr[v] * si;
            row[a.rank + v] = kr[v] * co + kr[u] * si;
        }
        for (int i = a.rope_dims + tid; i < a.dr; i += 256) row[a.rank + i] = kr[i];
        if (cache16) {
            __syncthreads();
            bf16 *row16 = cache16 + (size_t)(pos % ring) * kw;
            for (int i = tid; i < kw; i += 256) row16[i] = __float2bfloat16_rn(row[i]);
        }
    }
    const int hw = a.dk + a.dr;
    float *q = Q + (size_t)r * a.heads * kw;
    for (int e = tid; e < a.heads * half; e += 256) {
        const int h = e / half, i = e % half;
        int u, v;
        rope_pair_index(i, a.rope_dims, a.rope_layout, u, v);
        float *qr = p + a.q_off + (size_t)h * hw + a.dk;
        const float co = cs[2 * i], si = cs[2 * i + 1];
        const float ru = qr[u] * co - qr[v] * si, rv = qr[v] * co + qr[u] * si;
        q[(size_t)h * kw + a.rank + u] = qr[u] = ru;
        q[(size_t)h * kw + a.rank + v] = qr[v] = rv;
    }
    const int rest = a.dr - a.rope_dims;
    for (int e = tid; e < a.heads * rest; e += 256) {
        const int h = e / rest, i = a.rope_dims + e % rest;
        q[(size_t)h * kw + a.rank + i] = p[a.q_off + (size_t)h * hw + a.dk + i];
    }
    if (qu16)
        for (int e = tid; e < a.heads * a.dk; e += 256) {
            const int h = e / a.dk, d = e % a.dk;
            qu16[(size_t)r * a.heads * a.dk + e] = __float2bfloat16_rn(p[a.q_off + (size_t)h * hw + d]);
        }
}

// ---------------------------------------------------------------------------------------------------------------------
// Mixture of experts: router and grouping.
// ---------------------------------------------------------------------------------------------------------------------
// How the router's logits become expert ids and weights.  softmax == 0: scores sigmoid(z), the `top` largest, weight = score.
// softmax == 1: scores s = softmax(z) over all router outputs, the `top` largest of s + correction are chosen, weight =
// s / (sum of the chosen s + 1e-20) * scale.  Router outputs n_real .. are identity experts: they all get the id n_real.
struct RouteMode {
    int softmax;
    const float *correction; // [experts] (softmax mode)
    int n_real;              // experts with weights (<= experts)
    float scale;
};

// One warp: z [experts] logits in shared memory (overwritten), sbuf [experts] scratch; ids / wts [top] in order of falling choice
// score (the lowest index wins a tie).
__device__ __forceinline__ void route_select(float *z, float *sbuf, int experts, int top, const RouteMode &m, int *ids, float *wts, int lane) {
    if (m.softmax) {
        float mx = -INFINITY;
        for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z[e]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.0f;
        for (int e = lane; e < experts; e += 32) { const float w = expf(z[e] - mx); sbuf[e] = w; sum += w; }
        sum = warp_sum(sum);
        for (int e = lane; e < experts; e += 32) { const float sc = sbuf[e] / sum; sbuf[e] = sc; z[e] = sc + m.correction[e]; }
        __syncwarp();
    }
    float tot = 0.0f;
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int bi = experts;
        for (int e = lane; e < experts; e += 32)
            if (z[e] > best) { best = z[e]; bi = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (lane == 0) {
            const int id = bi < experts ? bi : 0;
            ids[k] = id < m.n_real ? id : m.n_real;
            const float w = m.softmax ? (bi < experts ? sbuf[bi] : 0.0f) : 1.0f / (1.0f + expf(-best));
            wts[k] = w;
            tot += w;
            if (bi < experts) z[bi] = -INFINITY; // taken
        }
        __syncwarp();
    }
    if (m.softmax && lane == 0)
        for (int k = 0; k < top; k++) wts[k] = wts[k] / (tot + 1e-20f) * m.scale;
}

// Router: logits z_e = <Wr[e], x> accumulated in FP32 (x FP32 or its BF16 rounding, Wr BF16), then route_select; ids / wts
// [n][top].  Wr may carry `extra` further rows behind the experts' whose logits go to extra_out [n][extra] (a gate computed
// from the same input).  Four warps per CTA: with rows_per_cta == 4 every warp owns a row, with rows_per_cta == 1 the four
// warps share the rows of one token (what the plan launches: four times the warps in flight, and the kernel is bound by the
// latency of its loads; the router matrix is small and stays in L2).
// Dynamic shared memory: rows_per_cta * (E + 2 * (experts + extra)) floats.
template <typename IN_T>
__global__ void __launch_bounds__(128) k_moe_route(const IN_T *__restrict__ X, const bf16 *__restrict__ Wr, int n, int E, int experts, int top, int rows_per_cta,
                                                   int *__restrict__ ids, float *__restrict__ wts, RouteMode m, int extra, float *__restrict__ extra_out) {
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool shared_row = rows_per_cta == 1;
    const int r = shared_row ? blockIdx.x : blockIdx.x * 4 + warp;
    const int zw = 2 * (experts + extra);
    float *xs = sm + (shared_row ? 0 : (size_t)warp * E), *z = sm + (size_t)rows_per_cta * E + (shared_row ? 0 : (size_t)warp * zw);
    if (r < n) {
        if (shared_row) for (int i = tid; i < E; i += 128) xs[i] = (float)X[(size_t)r * E + i];
        else for (int i = lane; i < E; i += 32) xs[i] = (float)X[(size_t)r * E + i];
    }
    if (shared_row) __syncthreads(); else __syncwarp();
    if (r < n) {
        const bool vec = (E & 7) == 0 && (((size_t)Wr) & 15) == 0;
        for (int e = shared_row ? warp : 0; e < experts + extra; e += shared_row ? 4 : 1) {
            const float acc = dot_row_bf16(Wr + (size_t)e * E, xs, E, lane, vec); // 128-bit weight loads, FP32 accumulation
            if (lane == 0) z[e] = acc;
        }
    }
    if (shared_row) __syncthreads(); else __syncwarp();
    if (r >= n || (shared_row && warp != 0)) return;
    for (int e = lane; e < extra; e += 32) extra_out[(size_t)r * extra + e] = z[experts + e];
    route_select(z, z + experts + extra, experts, top, m, ids + (size_t)r * top, wts + (size_t)r * top, lane);
}

// The decode step spreads the router's rows over several CTAs (k_matvec_bf16) and selects here: one warp, logits z [experts]
// in, route_select out.  Dynamic shared memory: 2 * experts floats.
__global__ void __launch_bounds__(32) k_moe_topk(const float *__restrict__ Z, int experts, int top, int *__restrict__ ids, float *__restrict__ wts, RouteMode m) {
    extern __shared__ __align__(16) float z[];
    const int lane = threadIdx.x;
    for (int e = lane; e < experts; e += 32) z[e] = Z[e];
    __syncwarp();
    route_select(z, z + experts, experts, top, m, ids, wts, lane);
}

// One CTA: the slots 0 .. n_slots - 1 (slot = row * top + k, expert ids[slot]) sorted by expert into `perm`, and the list of
// tiles (at most 64 slots of one expert each) the grouped projections run over; unused tiles get group -1.
// Dynamic shared memory: 3 * experts ints.
// Ids n_real .. experts - 1 are experts without weights (the identity): their slots are sorted like the others but their tiles get group -1.
__global__ void __launch_bounds__(1024) k_moe_group(const int *__restrict__ ids, int n_slots, int experts, int max_tiles, int *__restrict__ perm,
                                                    int *__restrict__ tile_group, int *__restrict__ tile_row0, int *__restrict__ tile_rows, int n_real) {
    extern __shared__ int smi[];
    int *count = smi, *offs = smi + experts, *cursor = smi + 2 * experts;
    const int tid = threadIdx.x;
    for (int e = tid; e < experts; e += 1024) count[e] = cursor[e] = 0;
    __syncthreads();
    for (int s = tid; s < n_slots; s += 1024) atomicAdd(&count[ids[s]], 1);
    __syncthreads();
    if (tid == 0) {
        int o = 0, t = 0;
        for (int e = 0; e < experts; e++) {
            offs[e] = o;
            for (int b = 0; b < count[e] && t < max_tiles; b += 64, t++) {
                tile_group[t] = e < n_real ? e : -1;
                tile_row0[t] = o + b;
                tile_rows[t] = count[e] - b < 64 ? count[e] - b : 64;
            }
            o += count[e];
        }
        for (; t < max_tiles; t++) { tile_group[t] = -1; tile_row0[t] = 0; tile_rows[t] = 0; }
    }
    __syncthreads();
    // the order of an expert's slots inside `perm` depends on the scheduling; no result does (a row's products are
    // accumulated in the same order wherever the row sits in its tile)
    for (int s = tid; s < n_slots; s += 1024) {
        const int e = ids[s];
        perm[offs[e] + atomicAdd(&cursor[e], 1)] = s;
    }
}

// Expanded keys of a prefill chunk: the rotated shared key part of cached row j (BF16 twin, [.][kw], entries rank ..) goes behind
// every head's unrotated key in KX [rows][heads * (dk + dr)].
__global__ void __launch_bounds__(256) k_latent_spread(const bf16 *__restrict__ cache16, int kw, int rank, int dr, int heads, int dk, bf16 *__restrict__ KX, int rows) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x, per = (long long)heads * dr;
    if (i >= per * rows) return;
    const int j = (int)(i / per), h = (int)(i % per) / dr, e = (int)(i % per) % dr;
    KX[((size_t)j * heads + h) * (dk + dr) + dk + e] = cache16[(size_t)j * kw + rank + e];
}

// The same grouping for the tcgen05 projections: every expert's slots padded to whole 128-row tiles, so that a tile belongs to one
// expert.  srt [max_tiles * 128]: slot of every padded row (-1: padding); slot_row [n_slots]: the inverse; row_scale: the slot's
// routing weight (0 for padding); tile_group [max_tiles]: expert of every tile, -1 beyond the last.  Dynamic shared memory: 3 * experts ints.
// Slots of ids >= n_real (experts without weights) get no row (slot_row -1); unit_scale: row_scale is 1 for every real row (the
// routing weight is applied to the expert's output, elsewhere).
__global__ void __launch_bounds__(1024) k_moe_group_padded(const int *__restrict__ ids, const float *__restrict__ wts, int n_slots, int experts, int max_tiles,
                                                           int *__restrict__ srt, int *__restrict__ slot_row, float *__restrict__ row_scale, int *__restrict__ tile_group,
                                                           int n_real, int unit_scale) {
    extern __shared__ int smi[];
    int *count = smi, *offs = smi + experts, *cursor = smi + 2 * experts;
    const int tid = threadIdx.x;
    for (int e = tid; e < experts; e += 1024) count[e] = cursor[e] = 0;
    for (int r = tid; r < max_tiles * 128; r += 1024) { srt[r] = -1; row_scale[r] = 0.0f; }
    __syncthreads();
    for (int s = tid; s < n_slots; s += 1024) atomicAdd(&count[ids[s]], 1);
    __syncthreads();
    if (tid == 0) {
        int t = 0;
        for (int e = 0; e < n_real; e++) {
            offs[e] = t * 128;
            for (int b = 0; b < count[e] && t < max_tiles; b += 128) tile_group[t++] = e;
        }
        for (; t < max_tiles; t++) tile_group[t] = -1;
    }
    __syncthreads();
    for (int s = tid; s < n_slots; s += 1024) {
        const int e = ids[s];
        if (e >= n_real) { slot_row[s] = -1; continue; }
        const int row = offs[e] + atomicAdd(&cursor[e], 1);
        if (row < max_tiles * 128) { srt[row] = s; row_scale[row] = unit_scale ? 1.0f : wts[s]; }
        slot_row[s] = row;
    }
}

// Rows of A (one per token) into expert-sorted order: padded row r reads token srt[r] / top; padding rows are zero.  E % 8 == 0.
__global__ void __launch_bounds__(128) k_moe_gather(const bf16 *__restrict__ A, int E, int top, const int *__restrict__ srt, const int *__restrict__ tile_group,
                                                    bf16 *__restrict__ AS) {
    const int row = blockIdx.x;
    if (tile_group[row >> 7] < 0) return;
    const int slot = srt[row];
    int4 *dst = reinterpret_cast<int4 *>(AS + (size_t)row * E);
    const int4 *src = slot >= 0 ? reinterpret_cast<const int4 *>(A + (size_t)(slot / top) * E) : nullptr;
    for (int i = threadIdx.x; i < E / 8; i += 128) dst[i] = src ? src[i] : make_int4(0, 0, 0, 0);
}

// The same after the expansions ran on the tcgen05 GEMM (FP32 results KXF [rows][heads * dk], VXF [rows][heads * dv]): BF16 keys
// [W_uk c_j | rot r_j] per head and BF16 values.  One CTA per cached row.
__global__ void __launch_bounds__(256) k_latent_pack(const float *__restrict__ KXF, const float *__restrict__ VXF, const bf16 *__restrict__ cache16, int kw, int rank, int dr,
                                                     int heads, int dk, int dv, bf16 *__restrict__ KX, bf16 *__restrict__ VX) {
    const int j = blockIdx.x, tid = threadIdx.x, DK = dk + dr;
    const float *kf = KXF + (size_t)j * heads * dk, *vf = VXF + (size_t)j * heads * dv;
    bf16 *kx = KX + (size_t)j * heads * DK, *vx = VX + (size_t)j * heads * dv;
    for (int e = tid; e < heads * DK; e += 256) {
        const int h = e / DK, d = e % DK;
        kx[e] = d < dk ? __float2bfloat16_rn(kf[h * dk + d]) : cache16[(size_t)j * kw + rank + d - dk];
    }
    for (int e = tid; e < heads * dv; e += 256) vx[e] = __float2bfloat16_rn(vf[e]);
}

__global__ void __launch_bounds__(256) k_softcap(float *__restrict__ x, long long n, float cap) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

} // namespace ly
