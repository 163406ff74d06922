// layered_plan.cuh -- host side of layered plans (included by plan.cu after its helpers): weight upload, the per-run window
// ring caches, the decode graph and the chunked prefill of models given as a list of layer specifications.
//
// Execution order.  The layer list is unrolled into RUNS: a loop block [start, stop) that executes `times` passes over the same
// weights contributes times * (stop - start) runs, and every run owns a key/value ring of its own (same weights, different
// history).  A pass starts with x += x0 (the embedding output; not on the first pass) and x += step[pass].
//
// Cache.  A run's ring has `ring` slots; position j lives in slot j % ring.  With ring >= window - 1 + (rows of one step) a
// step never overwrites a key one of its own rows still needs, so memory is bounded by the window, not by the context; a
// position is only ever read through an index range derived from the CURRENT position, so recycled slots and a new request
// starting at position 0 need no clearing.
//
// Kernel sequence of one run (decode: one row, captured once into a CUDA graph driven by the device-resident StepState;
// prefill: n rows per launch): norm (post-norm + residual of the previous sublayer, pass prologue, pre-norm) -> fused
// q|k|v|gate projection (+bias) -> whole-projection q/k norm + ring write -> window attention (+gate) -> output projection ->
// norm -> gated feed-forward projection (activation in the epilogue) -> down projection.
//
// Three block kinds share the plan: the sandwich block above (B200_BLOCK_SANDWICH), the pre-norm block (B200_BLOCK_PRENORM: the
// same sequence with x += s * y in place of the post-norm, RMS norms that carry one number, a normalised embedding, and loop
// passes without a prologue) and the parallel block of latent_plan.cuh (B200_BLOCK_PARALLEL: latent attention and a mixture of
// experts reading two norms of the same residual row).  Sandwich and pre-norm layers choose their mixer per layer: windowed
// attention (optionally with rotation, values taken from the keys, head temperatures and head-mixed scores: k_rope_mix_prep
// replaces k_qk_prep) or the gated delta rule (k_delta_prep -> k_delta_rule -> k_head_norm_gate), whose recurrent state and
// convolution inputs live per RUN next to the rings.
#pragma once
#include "layered.cuh"
#include "latent.cuh"
#include "delta.cuh"
#include "recurrent.cuh"

struct LyLayer {
    b200_layer_spec s{};
    int qd = 0, kd = 0, vd = 0, gd = 0, P = 0; // fused projection: q | k | v | gate rows
    int Pn = 0;                                // rows of the fused projection that carry weights (P may be padded with zero rows)
    ly::bf16 *w_proj = nullptr, *w_o = nullptr, *w_gu = nullptr, *w_down = nullptr;
    float *b_proj = nullptr;
    float *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr, *qnorm = nullptr, *knorm = nullptr, *rel = nullptr;
    int *bucket = nullptr;
    // latent attention (B200_MIXER_LATENT_ATTENTION): columns of q, [latent' | shared key part] and gate in a projection row; cache row
    // kw = kv_rank + rot_dim; folded query row qw = heads * kw; attention output in latent space lw = heads * kv_rank
    int q_off = 0, kv_off = -1, g_off = -1, kw = 0, qw = 0, lw = 0;
    ly::bf16 *w_ukT = nullptr, *w_uv = nullptr; // [heads][kv_rank][key_dim] (W_uk transposed per head at upload), [heads][value_dim][kv_rank]
    ly::bf16 *w_uk = nullptr;                   // [heads * key_dim][kv_rank] as stored: the BF16 prefill that expands keys per head reads it
    bool expand = false;                        // BF16 prefill through expanded keys / values and the tensor-core attention kernel
    float *cnorm = nullptr;
    const float *rope = nullptr;                // [context][rope_dims / 2][2], shared between layers with the same rotation
    // parallel block: biases of the two layer norms; mixture of experts: router [experts][width], w_gu = [experts][2 ff][width],
    // w_down = [experts][width][ff]
    float *ln1_b = nullptr, *ln2_b = nullptr;
    ly::bf16 *w_router = nullptr;
    // TMA descriptors of the tensor-core prefill (BF16 compute mode, shapes the tcgen05 GEMM tiles cover); *_ok = usable
    CUtensorMap m_proj, m_o, m_gate, m_up, m_down, m_att, m_h;
    CUtensorMap m_xk_b, m_xv_b, m_xk_c, m_xv_c; // key / value expansion of the BF16 prefill on the tcgen05 GEMM: W_uk, W_uv, FP32 results
    bool tc_expand = false;
    CUtensorMap m_moe_gate, m_moe_up, m_moe_down, m_moe_h; // mixture of experts on the tcgen05 GEMM: all experts' matrices in one map each
    bool tc_moe = false;
    bool tc_proj = false, tc_o = false, tc_gu = false, tc_down = false;
    // windowed attention with rotation / head temperature / head mixing (k_rope_mix_prep): pv = value rows and gr = gate rows of the
    // fused projection; the query the attention kernels read has heads * dk_eff entries (dk_eff = kv_heads * key_dim when the head
    // mixing is folded into it, k_heads = key heads the attention kernel indexes)
    int pv = 0, gr = 0, dk_eff = 0, k_heads = 0;
    bool mixprep = false;
    float *temp = nullptr, *talk = nullptr, *sink_logit = nullptr;
    float *ls1 = nullptr, *ls2 = nullptr; // pre-norm block: layer scales
    // gated delta rule: convolution weights of the q | k | v channels, per-head constants, weight of the read-out norm
    float *conv_w = nullptr, *a_log = nullptr, *dt_bias = nullptr, *onorm = nullptr;
    int dC = 0; // convolved channels = 2 * kv_heads * key_dim + heads * value_dim
    // OUTNORM block: token shift, depth average weights; differential attention; recurrent unit (stacked gate matrices [blocks][r | i rows][in],
    // their biases, branch biases); state-space recurrence; mixture of experts with correction and a shared expert; plain feed-forward (w_gu = up)
    float *shift = nullptr, *dwa = nullptr;
    float diff_lambda = 0.0f;
    ly::bf16 *w_gates = nullptr;
    float *gate_bias = nullptr, *lam = nullptr, *x_bias = nullptr, *y_bias = nullptr, *conv_b = nullptr, *ssd_d = nullptr;
    float *correction = nullptr;
    ly::bf16 *w_sgu = nullptr, *w_sdown = nullptr;
    CUtensorMap m_sgate, m_sup, m_sdown, m_sh;
    bool tc_sgu = false, tc_sdown = false;
};
struct LyRun {
    int layer = 0, pass = -1;
    bool first = false; // first layer of a loop pass
    float *kc = nullptr, *vc = nullptr;
    ly::bf16 *kc16 = nullptr, *vc16 = nullptr; // BF16 twin rows (BF16 plans whose head sizes the tensor-core attention takes)
    CUtensorMap m_lat;                         // latent attention: the latent columns of the BF16 twin rows as a GEMM operand
    bool tc_lat = false;
    int kw = 0, vw = 0;                        // floats per cache row (latent attention: one cache, kw = kv_rank + rot_dim, vc == nullptr)
    bool own = true;                           // false: kc is the cache of the run this layer reads (kv_from)
    float *S = nullptr, *cstate = nullptr;     // gated delta rule: state [heads][key_dim][value_dim]; ring of convolution inputs [cring][channels]
    size_t s_floats = 0, c_floats = 0;         // sizes of S and cstate
    float *prev = nullptr;                     // token shift: the row the run's mixer read last, before its shift
};
struct Layered {
    b200_layered_config c{};
    std::vector<LyLayer> layers;
    std::vector<LyRun> runs;
    ly::bf16 *emb = nullptr, *head = nullptr;
    float *final_norm = nullptr, *step = nullptr;
    int cap = 1, ring = 0, max_window = 1, logit_rows = 1;
    int maxP = 0, maxO = 0, maxF = 0;
    bool f32 = false, has_loop = false;
    float *X = nullptr, *X0 = nullptr, *Y = nullptr, *PROJ = nullptr, *A32 = nullptr, *ATT32 = nullptr, *H32 = nullptr, *LOG = nullptr;
    ly::bf16 *A16 = nullptr, *ATT16 = nullptr, *H16 = nullptr;
    int *tok = nullptr, *rows = nullptr;
    StepState *st_pf = nullptr;
    float *trace = nullptr; // [runs][cap][width], allocated on first use
    int smem_max = 0;
    ly::KeySplit split{nullptr, nullptr, nullptr}; // scratch of the decode attention's key splits (B200_LAYERED_SPLITS=1 turns them off)
    int max_splits = 8;
    int cap_pad = 1; // rows of the activation buffers: cap, padded to whole 256-row GEMM tiles in BF16 mode
    bool tc = false, tc_head = false;
    bool att_mma = true; // BF16 prefill attention on the tensor cores for key/value sizes 64 and 128 (B200_LAYERED_ATT=simt: the FP32 kernel)
    CUtensorMap m_a, m_head, m_proj_c, m_y_c, m_log_c;
    // parallel block / latent attention / mixture of experts
    float *final_norm_b = nullptr;
    float *A2_32 = nullptr, *Q = nullptr, *LAT32 = nullptr, *YS = nullptr, *moe_wts = nullptr, *ZR = nullptr;
    ly::bf16 *A2_16 = nullptr, *QU16 = nullptr, *LAT16 = nullptr;
    float *KXF = nullptr, *VXF = nullptr;      // FP32 results of the tcgen05 expansions, rows padded to whole 128-row tiles
    ly::bf16 *KX16 = nullptr, *VX16 = nullptr; // keys / values of one layer expanded per head for a prefill chunk: [context][heads * size]
    int maxKX = 0, maxVX = 0, pf_pos = 0;      // pf_pos: first position of the chunk being enqueued
    // expert-sorted, tile-padded operands of the tcgen05 expert projections (BF16 prefill)
    ly::bf16 *AS16 = nullptr, *HS16 = nullptr;
    float *YSP = nullptr, *row_scale = nullptr;
    int *srt = nullptr, *slot_row = nullptr, *tile_group128 = nullptr;
    int max_tiles128 = 0;
    CUtensorMap m_as, m_ysp;
    int *moe_ids = nullptr, *moe_perm = nullptr, *tile_group = nullptr, *tile_row0 = nullptr, *tile_rows = nullptr;
    int maxQ = 0, maxL = 0, maxQU = 0, maxTop = 0, maxExperts = 0, max_tiles = 0, max_att_dv = 1;
    std::vector<std::pair<std::vector<float>, float *>> rope_tables; // (key, device table)
    // pre-norm block / gated delta rule
    float w_off = 1.0f;   // what the norm kernels add to a norm weight (sandwich: weights are deviations from one)
    bool prenorm = false;
    float *emb_norm = nullptr;
    float *DLT = nullptr, *DO = nullptr; // prepared q | k | v | beta | decay rows and read-out rows of a delta layer, [cap][...]
    int maxD = 0, maxDO = 0, cring = 0, max_taps = 0;
    // OUTNORM block: kept layer results X_j [layers + 1][cap][width], the shared expert's result, its gate logits, BF16 twin of a convolved row
    bool outnorm = false;
    float *STASH = nullptr, *SH = nullptr, *SGL = nullptr;
    ly::bf16 *U16 = nullptr;
    int max_att_heads = 1;
    CUtensorMap m_sh_c;
};

// What ly_project needs to take the tcgen05 route: operand and result descriptors (nullptr = CUDA-core / mma.sync kernels).
struct LyTc {
    const CUtensorMap *a = nullptr, *b = nullptr, *b2 = nullptr, *c = nullptr;
};

static int ly_vec_f32(b200_plan *p, const b200_tensor *tensors, int nt, const std::string &name, int64_t n, float **dst, bool required = true) {
    const b200_tensor *t = find(tensors, nt, name);
    if (!t) {
        if (!required) { *dst = nullptr; return B200_OK; }
        return fail(p, B200_ERR_BAD_ARG, "missing tensor %s", name.c_str());
    }
    if (n_elems(t) != n) return fail(p, B200_ERR_BAD_ARG, "tensor %s has %lld elements, expected %lld", name.c_str(), (long long)n_elems(t), (long long)n);
    std::vector<float> h((size_t)n);
    if (t->ggml_type == B200_GGML_BF16) {
        const uint16_t *s = (const uint16_t *)t->data;
        for (int64_t i = 0; i < n; i++) { uint32_t u = (uint32_t)s[i] << 16; memcpy(&h[i], &u, 4); }
    } else if (t->ggml_type == B200_GGML_F32) memcpy(h.data(), t->data, (size_t)n * 4);
    else return fail(p, B200_ERR_UNSUPPORTED, "tensor %s: type %d (vectors are BF16 or F32)", name.c_str(), t->ggml_type);
    int rc;
    if ((rc = dalloc(p, dst, (size_t)n * 4))) return rc;
    CK(cudaMemcpy(*dst, h.data(), (size_t)n * 4, cudaMemcpyHostToDevice));
    return B200_OK;
}

// A tensor that holds ONE number (BF16 or F32, any rank), repeated n times: a norm whose weight is the same for all coordinates.
static int ly_scalar_vec(b200_plan *p, const b200_tensor *tensors, int nt, const std::string &name, int64_t n, float **dst) {
    const b200_tensor *t = find(tensors, nt, name);
    if (!t) return fail(p, B200_ERR_BAD_ARG, "missing tensor %s", name.c_str());
    if (n_elems(t) != 1) return fail(p, B200_ERR_BAD_ARG, "tensor %s has %lld elements, expected one number", name.c_str(), (long long)n_elems(t));
    float v;
    if (t->ggml_type == B200_GGML_BF16) { uint32_t u = (uint32_t)(*(const uint16_t *)t->data) << 16; memcpy(&v, &u, 4); }
    else if (t->ggml_type == B200_GGML_F32) memcpy(&v, t->data, 4);
    else return fail(p, B200_ERR_UNSUPPORTED, "tensor %s: type %d (numbers are BF16 or F32)", name.c_str(), t->ggml_type);
    std::vector<float> h((size_t)n, v);
    int rc;
    if ((rc = dalloc(p, dst, (size_t)n * 4))) return rc;
    CK(cudaMemcpy(*dst, h.data(), (size_t)n * 4, cudaMemcpyHostToDevice));
    return B200_OK;
}

// rows x cols BF16 matrix into dst at row offset row_off, through the plan's upload pipeline
static int ly_mat(b200_plan *p, const b200_tensor *tensors, int nt, const std::string &name, int rows, int cols, ly::bf16 *dst, int row_off) {
    const b200_tensor *t = find(tensors, nt, name);
    if (!t) return fail(p, B200_ERR_BAD_ARG, "missing tensor %s", name.c_str());
    if (t->ggml_type != B200_GGML_BF16) return fail(p, B200_ERR_UNSUPPORTED, "tensor %s: type %d (layered plans take BF16 matrices)", name.c_str(), t->ggml_type);
    if (t->n_dims != 2 || t->dims[0] != cols || t->dims[1] != rows)
        return fail(p, B200_ERR_BAD_ARG, "tensor %s is not [%d][%d]", name.c_str(), rows, cols);
    const size_t bytes = (size_t)rows * cols * 2;
    if (p->up.on) return up_h2d(p, dst + (size_t)row_off * cols, t->data, bytes);
    CK(cudaMemcpy(dst + (size_t)row_off * cols, t->data, bytes, cudaMemcpyHostToDevice));
    p->up.h2d_bytes += (int64_t)bytes;
    return B200_OK;
}

// Distance -> table row: exact below rows/2, logarithmic up to `far`, the last row beyond (evaluated in double on the host).
static int ly_bucket(int n, int rows, double far) {
    const int half = rows / 2;
    if (n < half) return n;
    const int b = half + (int)floor(log((double)n / half) / log(far / half) * (rows - half));
    return b < rows - 1 ? b : rows - 1;
}

static void ly_free(b200_plan *p) {
    delete p->ly;
    p->ly = nullptr;
}

static size_t ly_att_smem(int dk, int window) { return ly::att_smem_floats(dk, window) * 4; }
static size_t ly_att_smem(const b200_layer_spec &s, int ring) {
    (void)ring;
    // latent attention attends over the cached row [latent | shared key part] with one key/value head; head-mixed scores over a row of all key heads
    return ly_att_smem(s.mixer == B200_MIXER_LATENT_ATTENTION ? s.kv_rank + s.rot_dim : s.head_mix ? s.kv_heads * s.key_dim : s.key_dim, s.window);
}

// Instances of the tensor-core prefill attention: (key size, value size) = (64, 64), (128, 128), (192, 128); 0 = none.
static int ly_mma_kind(int dk, int dv) {
    return dk == 64 && dv == 64 ? 1 : dk == 128 && dv == 128 ? 2 : dk == 192 && dv == 128 ? 3 : dk == 128 && dv == 64 ? 4 : dk == 256 && dv == 128 ? 5 : 0;
}
static size_t ly_mma_smem(int kind, int window) {
    return kind == 1 ? ly::att_mma_smem_bytes<64, 64>(window) : kind == 2 ? ly::att_mma_smem_bytes<128, 128>(window) : kind == 3 ? ly::att_mma_smem_bytes<192, 128>(window)
         : kind == 4 ? ly::att_mma_smem_bytes<128, 64>(window) : ly::att_mma_smem_bytes<256, 128>(window);
}
static int ly_launch_mma(b200_plan *p, int kind, int n, int heads, int window, const float *P, int ldp, const ly::WindowAttn &wa, const ly::bf16 *k16, const ly::bf16 *v16,
                         const StepState *st, ly::bf16 *out, int ldo, float *out32 = nullptr) {
    const dim3 grid((n + LY_ATT_MMA_ROWS - 1) / LY_ATT_MMA_ROWS, heads), block(LY_ATT_MMA_THREADS);
    const size_t sm = ly_mma_smem(kind, window);
    if (kind == 1) return launch_k(p, false, ly::k_window_attention_mma<64, 64>, grid, block, sm, P, ldp, wa, k16, v16, st, n, out, ldo, out32);
    if (kind == 2) return launch_k(p, false, ly::k_window_attention_mma<128, 128>, grid, block, sm, P, ldp, wa, k16, v16, st, n, out, ldo, out32);
    if (kind == 4) return launch_k(p, false, ly::k_window_attention_mma<128, 64>, grid, block, sm, P, ldp, wa, k16, v16, st, n, out, ldo, out32);
    if (kind == 5) return launch_k(p, false, ly::k_window_attention_mma<256, 128>, grid, block, sm, P, ldp, wa, k16, v16, st, n, out, ldo, out32);
    return launch_k(p, false, ly::k_window_attention_mma<192, 128>, grid, block, sm, P, ldp, wa, k16, v16, st, n, out, ldo, out32);
}

static ly::WindowAttn ly_attn_args(const Layered &Y, const LyLayer &L) {
    ly::WindowAttn a{};
    a.heads = L.s.heads; a.kv_heads = L.s.kv_heads; a.dk = L.s.key_dim; a.dv = L.s.value_dim;
    a.window = L.s.window; a.ring = Y.ring; a.bias_rows = L.s.bias_rows;
    a.ldk = L.kd; a.ldv = L.vd;
    a.scale = L.s.score_scale; a.softcap = L.s.softcap;
    a.rel = L.rel; a.bucket = L.bucket; a.qnorm = L.qnorm; a.knorm = L.knorm;
    a.sink = L.s.sink; a.gate = L.s.gate; a.gate_off = L.qd + L.kd + L.pv; a.eps = Y.c.norm_eps;
    a.sink_logit = L.sink_logit; a.gate_heads = L.s.gate == 2;
    if (L.mixprep) { // the query comes from k_rope_mix_prep's buffer (temperature and head mixing folded in), the gate from the projection row
        a.dk = L.dk_eff; a.k_heads = L.k_heads; a.qnorm = a.knorm = nullptr;
        a.gate_src = Y.PROJ; a.gate_ld = Y.maxP;
    }
    return a;
}

// C[n][N] = A[n][K] W^T with the epilogue EPI; decode (n == 1 through the graph) streams the rows, prefill takes a GEMM:
// the persistent CTA-pair tcgen05 kernel (256-wide tiles) or the single-CTA one (128-wide) of prefill_gemm.cuh when the
// shape fits and the plan computes in BF16, else the any-shape kernels of layered.cuh.
template <int EPI>
static int ly_project(b200_plan *p, bool decode, int n, const float *a32, const ly::bf16 *a16, const ly::bf16 *W, const float *bias, int N, int K,
                      float *c32, ly::bf16 *c16, int ldc, int act, const LyTc *tc = nullptr) {
    Layered &Y = *p->ly;
    if (decode) {
        const int warps = LY_MV_THREADS / 32;
        int grid = (N + warps - 1) / warps;
        return launch_k(p, false, ly::k_matvec_bf16<EPI>, dim3(grid), dim3(LY_MV_THREADS), (size_t)K * 4, W, bias, a32, c32, N, K, act, ly::MvView{});
    }
    if (tc && tc->a && !Y.f32) {
        const int mt2 = (n + 255) / 256 * 2;
        int rc;
        if (EPI == ly::EPI_GATED)
            rc = pg::gemm2_persist_launch<pg::GEMM_GATEUP, 256, pg::GEMM2_PERSIST_STAGES_256>(*tc->a, *tc->b, *tc->b2, *tc->c, c16, ldc, n, mt2, N / 128, K, p->n_sms, p->stream, 1,
                                                                                            pg::FLAVOR_BF16 | (act == B200_ACT_RELU ? pg::FLAVOR_RELU_BF16 : act == B200_ACT_SILU ? pg::FLAVOR_SILU_BF16 : pg::FLAVOR_GELU_BF16));
        else if (N % 256 == 0) {
            // a narrow output (N = width) leaves most SMs idle: split K over the grid and let every split reduce-add its partial
            // product into the zeroed result through TMA, as the GGUF prefill does for its residual GEMMs
            const int ctas = mt2 * (N / 256), nk = K / pg::BK;
            int sp = p->n_sms / ctas;
            if (sp > 4) sp = 4;
            while (sp > 1 && (nk / sp < 8 || (sp - 1) * ((nk + sp - 1) / sp) >= nk)) sp--;
            if (sp > 1) {
                if (cudaMemsetAsync(c32, 0, (size_t)n * ldc * 4, p->stream) != cudaSuccess) return fail(p, B200_ERR_CUDA, "cudaMemsetAsync failed");
                rc = pg::gemm2_launch<pg::GEMM_RESID, 256, pg::GEMM2_STAGES_256>(*tc->a, *tc->b, *tc->b, *tc->c, c32, ldc, n, mt2, N / 256, K, p->stream, sp, pg::FLAVOR_BF16);
            } else
                rc = pg::gemm2_persist_launch<pg::GEMM_F32, 256, pg::GEMM2_PERSIST_STAGES_256>(*tc->a, *tc->b, *tc->b, *tc->c, c32, ldc, n, mt2, N / 256, K, p->n_sms, p->stream, 1, pg::FLAVOR_BF16);
        }
        else
            rc = pg::gemm_launch<pg::GEMM_F32, pg::GEMM_STAGES>(*tc->a, *tc->b, *tc->b, *tc->c, c32, ldc, n, (n + 127) / 128, N / 128, K, p->stream, pg::FLAVOR_BF16);
        return rc ? fail(p, B200_ERR_CUDA, "tensor-core GEMM launch failed (%d)", rc) : B200_OK;
    }
    dim3 grid((N + 63) / 64, (n + 63) / 64);
    if (Y.f32) return launch_k(p, false, ly::k_gemm_f32<EPI, float>, grid, dim3(256), (size_t)0, a32, W, bias, c32, n, N, K, ldc, act, ly::GemmView{});
    if (c16) return launch_k(p, false, ly::k_gemm_bf16<EPI, ly::bf16>, grid, dim3(128), (size_t)0, a16, W, bias, c16, n, N, K, ldc, act, ly::GemmView{});
    return launch_k(p, false, ly::k_gemm_bf16<EPI, float>, grid, dim3(128), (size_t)0, a16, W, bias, c32, n, N, K, ldc, act, ly::GemmView{});
}

#include "latent_plan.cuh"
#include "outnorm_plan.cuh"

// Enqueue the forward of n rows on p->stream.  decode: the single-token step (row 0, position and token from *st).
// with_head (decode only): final norm + classifier into p->logits.  Prefill leaves the finished residual rows in X.
static int ly_enqueue(b200_plan *p, bool decode, int n, const StepState *st, const int *tokens, bool with_head, float *trace, int *launches) {
    Layered &Y = *p->ly;
    if (Y.c.block == B200_BLOCK_PARALLEL) return ly_enqueue_parallel(p, decode, n, st, tokens, with_head, trace, launches);
    if (Y.c.block == B200_BLOCK_OUTNORM) return ly_enqueue_outnorm(p, decode, n, st, tokens, with_head, trace, launches);
    const int E = Y.c.width;
    const bool h16 = !decode && !Y.f32; // prefill in BF16 mode rounds GEMM operands to BF16
    int nl = 0, rc;
    const float *pend_y = nullptr, *pend_w = nullptr;
    float *pend_trace = nullptr;
    auto norm = [&](bool embed, bool add_x0, const float *step, const float *w_pre) {
        ly::NormArgs a{};
        a.x = Y.X; a.x0 = Y.has_loop && !Y.prenorm ? Y.X0 : nullptr;
        a.y = pend_y; a.w_post = pend_w;
        a.w_off = Y.w_off; a.post_plain = Y.prenorm ? 1 : 0; a.w_emb = embed ? Y.emb_norm : nullptr;
        a.emb = embed ? Y.emb : nullptr; a.tokens = tokens; a.st = st; a.emb_scale = Y.c.embedding_scale;
        a.add_x0 = add_x0 ? 1 : 0; a.step = step; a.w_pre = w_pre;
        a.out32 = w_pre && !h16 ? Y.A32 : nullptr; a.out16 = w_pre && h16 ? Y.A16 : nullptr;
        a.gather = nullptr; a.trace = pend_trace; a.eps = Y.c.norm_eps; a.E = E;
        pend_y = pend_w = nullptr; pend_trace = nullptr;
        nl++;
        return launch_k(p, false, ly::k_norm_rows, dim3(n), dim3(LY_NORM_THREADS), (size_t)E * 4, a);
    };
    for (size_t r = 0; r < Y.runs.size(); r++) {
        const LyRun &R = Y.runs[r];
        const LyLayer &L = Y.layers[R.layer];
        // a loop pass of a sandwich block starts with x += x0 (not the first pass) and x += step[pass]; a pre-norm block just repeats
        const bool prologue = R.first && !Y.prenorm;
        if ((rc = norm(r == 0, prologue && R.pass > 0, prologue ? Y.step + (size_t)R.pass * E : nullptr, L.norm1))) return rc;
        LyTc t_proj, t_o, t_gu, t_down;
        if (Y.tc && !decode) {
            if (L.tc_proj) { t_proj.a = &Y.m_a; t_proj.b = &L.m_proj; t_proj.c = &Y.m_proj_c; }
            if (L.tc_o) { t_o.a = &L.m_att; t_o.b = &L.m_o; t_o.c = &Y.m_y_c; }
            if (L.tc_gu) { t_gu.a = &Y.m_a; t_gu.b = &L.m_gate; t_gu.b2 = &L.m_up; t_gu.c = &Y.m_y_c; }
            if (L.tc_down) { t_down.a = &L.m_h; t_down.b = &L.m_down; t_down.c = &Y.m_y_c; }
        }
        // the q, k, v biases are added where the projection is consumed (k_qk_prep), so every projection kernel serves it
        if ((rc = ly_project<ly::EPI_STORE>(p, decode, n, Y.A32, Y.A16, L.w_proj, nullptr, decode ? L.Pn : L.P, E, Y.PROJ, nullptr, Y.maxP, 0, &t_proj))) return rc;
        nl++;
        if (L.s.mixer == B200_MIXER_GATED_DELTA) {
            ly::DeltaArgs da{};
            da.heads = L.s.heads; da.kv_heads = L.s.kv_heads; da.dk = L.s.key_dim; da.dv = L.s.value_dim; da.taps = L.s.conv_taps; da.cring = Y.cring;
            da.conv_w = L.conv_w; da.a_log = L.a_log; da.dt_bias = L.dt_bias; da.unit_eps = 1e-6f;
            const int dmax = L.s.key_dim > L.s.value_dim ? L.s.key_dim : L.s.value_dim;
            if ((rc = launch_k(p, false, ly::k_delta_prep, dim3(n, 2 * L.s.kv_heads + L.s.heads + 1), dim3(DELTA_PREP_THREADS), (size_t)dmax * 4, (const float *)Y.PROJ, Y.maxP, da, R.cstate,
                               Y.DLT, Y.maxD, st))) return rc;
            const dim3 rgrid(L.s.heads, (L.s.value_dim + DR_COLS - 1) / DR_COLS), rblock(DR_THREADS);
            switch (ly::delta_reg_rows(L.s.key_dim)) {
            case 1: rc = launch_k(p, false, ly::k_delta_rule_reg<1>, rgrid, rblock, (size_t)0, (const float *)Y.DLT, Y.maxD, da, R.S, n, Y.DO, Y.maxDO, st); break;
            case 2: rc = launch_k(p, false, ly::k_delta_rule_reg<2>, rgrid, rblock, (size_t)0, (const float *)Y.DLT, Y.maxD, da, R.S, n, Y.DO, Y.maxDO, st); break;
            case 4: rc = launch_k(p, false, ly::k_delta_rule_reg<4>, rgrid, rblock, (size_t)0, (const float *)Y.DLT, Y.maxD, da, R.S, n, Y.DO, Y.maxDO, st); break;
            case 8: rc = launch_k(p, false, ly::k_delta_rule_reg<8>, rgrid, rblock, (size_t)0, (const float *)Y.DLT, Y.maxD, da, R.S, n, Y.DO, Y.maxDO, st); break;
            default: // key sizes above 128: the state tile in shared memory, one thread per column
                rc = launch_k(p, false, ly::k_delta_rule, dim3(L.s.heads, (L.s.value_dim + DELTA_COLS - 1) / DELTA_COLS), dim3(DELTA_COLS), ly::delta_rule_smem_floats(L.s.key_dim) * 4,
                              (const float *)Y.DLT, Y.maxD, da, R.S, n, Y.DO, Y.maxDO, st);
            }
            if (rc) return rc;
            if ((rc = launch_k(p, false, ly::k_head_norm_gate, dim3(n), dim3(256), (size_t)0, (const float *)Y.DO, Y.maxDO, (const float *)(Y.PROJ + L.dC + 2 * L.s.heads), Y.maxP,
                               (const float *)L.onorm, L.s.heads, L.s.value_dim, Y.c.norm_eps, h16 ? (float *)nullptr : Y.ATT32, h16 ? Y.ATT16 : (ly::bf16 *)nullptr, L.gd))) return rc;
            nl += 3;
        } else {
        const ly::WindowAttn wa = ly_attn_args(Y, L);
        const float *qsrc = Y.PROJ; // where the attention kernels read the query rows
        int ldq = Y.maxP;
        if (L.mixprep) {
            ly::RopeMixArgs ra{};
            ra.heads = L.s.heads; ra.kv_heads = L.s.kv_heads; ra.dk = L.s.key_dim; ra.dv = L.s.value_dim; ra.rope_dims = L.s.rope_dims; ra.rope_layout = L.s.rope_layout;
            ra.cs = L.rope; ra.temp = L.temp; ra.talk = L.talk; ra.value_from_key = L.s.value_from_key; ra.ring = Y.ring;
            qsrc = Y.Q; ldq = L.s.heads * L.dk_eff;
            const int hpc = decode ? 1 : ROPE_MIX_HEADS; // one row: a CTA per head; a chunk: several heads share the rotation of the row
            rc = launch_k(p, false, ly::k_rope_mix_prep, dim3(n, (L.s.heads + hpc - 1) / hpc + 1), dim3(ROPE_MIX_THREADS), (size_t)(L.qd > L.kd ? L.qd : L.kd) * 4, (const float *)Y.PROJ, Y.maxP, ra,
                          (const float *)L.b_proj, Y.Q, ldq, R.kc, R.vc, R.kc16, R.vc16, st, hpc);
        } else
            rc = launch_k(p, false, ly::k_qk_prep, dim3(n), dim3(256), (size_t)0, Y.PROJ, Y.maxP, wa, (const float *)L.b_proj, R.kc, R.vc, R.kc16, R.vc16, st);
        if (rc) return rc;
        nl++;
        const size_t asm_ = ly_att_smem(L.s, Y.ring);
        const int mma = ly_mma_kind(L.mixprep ? L.dk_eff : L.s.key_dim, L.s.value_dim);
        if (h16 && R.kc16 && mma)
            rc = ly_launch_mma(p, mma, n, L.s.heads, L.s.window, qsrc, ldq, wa, (const ly::bf16 *)R.kc16, (const ly::bf16 *)R.vc16, st, Y.ATT16, L.gd);
        else if (h16) rc = launch_k(p, false, ly::k_window_attention<ly::bf16>, dim3(n, L.s.heads), dim3(LY_ATT_THREADS), asm_, qsrc, ldq, wa,
                               (const float *)R.kc, (const float *)R.vc, st, Y.ATT16, L.gd, ly::KeySplit{nullptr, nullptr, nullptr});
        else {
            // the decode step has one row and few heads: split every head's window over several CTAs so that the SMs are used
            int sp = 1;
            if (decode && Y.split.o && L.s.window >= 64) { sp = p->n_sms / L.s.heads; if (sp > Y.max_splits) sp = Y.max_splits; if (sp < 1) sp = 1; }
            rc = launch_k(p, false, ly::k_window_attention<float>, dim3(n, L.s.heads, sp), dim3(LY_ATT_THREADS), asm_, qsrc, ldq, wa,
                          (const float *)R.kc, (const float *)R.vc, st, Y.ATT32, L.gd, sp > 1 ? Y.split : ly::KeySplit{nullptr, nullptr, nullptr});
        }
        if (rc) return rc;
        nl++;
        } // windowed attention
        if ((rc = ly_project<ly::EPI_STORE>(p, decode, n, Y.ATT32, Y.ATT16, L.w_o, nullptr, E, L.gd, Y.Y, nullptr, E, 0, &t_o))) return rc;
        nl++;
        pend_y = Y.Y; pend_w = Y.prenorm ? L.ls1 : L.norm1b;
        if (L.s.ff_kind == B200_FF_DENSE_GATED) {
            if ((rc = norm(false, false, nullptr, L.norm2))) return rc;
            const int F = L.s.ff_dim;
            if ((rc = ly_project<ly::EPI_GATED>(p, decode, n, Y.A32, Y.A16, L.w_gu, nullptr, F, E, Y.H32, h16 ? Y.H16 : nullptr, F, L.s.ff_act, &t_gu))) return rc;
            nl++;
            if ((rc = ly_project<ly::EPI_STORE>(p, decode, n, Y.H32, Y.H16, L.w_down, nullptr, E, F, Y.Y, nullptr, E, 0, &t_down))) return rc;
            nl++;
            pend_y = Y.Y; pend_w = Y.prenorm ? L.ls2 : L.norm2b;
        }
        pend_trace = trace ? trace + r * (size_t)Y.cap * E : nullptr;
    }
    if (decode) {
        if (with_head) {
            if ((rc = norm(false, false, nullptr, Y.final_norm))) return rc;
            if ((rc = ly_project<ly::EPI_STORE>(p, true, 1, Y.A32, nullptr, Y.head, nullptr, Y.c.vocab_size, E, p->logits, nullptr, Y.c.vocab_size, 0))) return rc;
            nl++;
        } else if ((rc = norm(false, false, nullptr, nullptr))) return rc;
        if ((rc = launch_k(p, false, k_argmax_advance, dim3(1), dim3(1024), (size_t)0, (const float *)p->logits, Y.c.vocab_size, p->st, (const int *)p->seq_tokens,
                           p->out_ids, with_head ? 1 : 0, (const float *)nullptr, (const int *)nullptr, 0, TraceBuf{nullptr, 0, 0}, p->tp, -1))) return rc;
        nl++;
    } else if ((rc = norm(false, false, nullptr, nullptr))) return rc;
    if (launches) *launches = nl;
    return B200_OK;
}

static int ly_capture(b200_plan *p, bool with_head, cudaGraphExec_t *exec, int *launches) {
    cudaGraph_t g = nullptr;
    CK(cudaStreamBeginCapture(p->stream, cudaStreamCaptureModeThreadLocal));
    int rc = ly_enqueue(p, true, 1, p->st, nullptr, with_head, nullptr, launches);
    cudaError_t e = cudaStreamEndCapture(p->stream, &g);
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    if (e != cudaSuccess) return fail(p, B200_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(p, B200_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    return B200_OK;
}

// Tensor-core prefill of BF16 plans: TMA descriptors for the weight matrices whose shapes the tcgen05 GEMM tiles cover
// (output width a multiple of 128, reduction width a multiple of 64) and for the activation / result buffers.  A layer whose
// shapes do not fit keeps the any-shape kernels; B200_LAYERED_TC=0 turns the route off.
static int ly_tc_init(b200_plan *p) {
    Layered &Y = *p->ly;
    const char *e = getenv("B200_LAYERED_TC");
    if ((e && e[0] == '0') || !pg::encode_fn()) return B200_OK;
    const int E = Y.c.width, V = Y.c.vocab_size;
    const uint64_t rows = (uint64_t)Y.cap_pad;
    auto fits = [](int N, int K) { return N % 128 == 0 && K % 64 == 0; };
    if (E % 64) return B200_OK;
    bool ok = pg::make_map(&Y.m_a, Y.A16, rows, E, pg::BM) == 0 && pg::make_map_c(&Y.m_y_c, Y.Y, rows, E) == 0;
    if (ok && Y.maxP % 4 == 0) ok = pg::make_map_c(&Y.m_proj_c, Y.PROJ, rows, Y.maxP) == 0;
    if (!ok) return B200_OK;
    for (LyLayer &L : Y.layers) {
        const int F = L.s.ff_dim;
        L.tc_proj = fits(L.P, E) && Y.maxP % 4 == 0 && pg::make_map(&L.m_proj, L.w_proj, L.P, E, 128) == 0;
        L.tc_o = fits(E, L.gd) && pg::make_map(&L.m_o, L.w_o, E, L.gd, 128) == 0 && pg::make_map(&L.m_att, Y.ATT16, rows, L.gd, pg::BM) == 0;
        if (Y.outnorm) continue; // its feed-forwards: ly_outnorm_tc_init
        if (L.w_gu && L.s.ff_kind == B200_FF_DENSE_GATED) {
            L.tc_gu = fits(F, E) && pg::make_map(&L.m_gate, L.w_gu, F, E, 128) == 0 &&
                      pg::make_map(&L.m_up, L.w_gu + (size_t)F * E, F, E, 128) == 0;
            L.tc_down = fits(E, F) && pg::make_map(&L.m_down, L.w_down, E, F, 128) == 0 && pg::make_map(&L.m_h, Y.H16, rows, F, pg::BM) == 0;
        }
    }
    if (Y.KXF) { // key / value expansions: A = latent columns of a cache's BF16 twin rows, B = W_uk / W_uv as stored, C = FP32 scratch
        const uint64_t rowsX = ((uint64_t)Y.ring + 127) / 128 * 128;
        for (LyRun &R : Y.runs) {
            const LyLayer &L = Y.layers[R.layer];
            R.tc_lat = R.own && R.kc16 && L.kw % 8 == 0 && L.s.kv_rank % 64 == 0 && pg::make_map_ld(&R.m_lat, R.kc16, (uint64_t)Y.ring, L.s.kv_rank, L.kw, pg::BM) == 0;
        }
        for (size_t r = 0; r < Y.runs.size(); r++) {
            LyLayer &L = Y.layers[Y.runs[r].layer];
            const LyRun &O = L.s.kv_from >= 0 ? Y.runs[L.s.kv_from] : Y.runs[r];
            const uint64_t nk = (uint64_t)L.s.heads * L.s.key_dim, nv = (uint64_t)L.gd, K = L.s.kv_rank;
            L.tc_expand = L.expand && O.tc_lat && nk % 128 == 0 && nv % 128 == 0 && pg::make_map(&L.m_xk_b, L.w_uk, nk, K, pg::BN) == 0 &&
                          pg::make_map(&L.m_xv_b, L.w_uv, nv, K, pg::BN) == 0 && pg::make_map_c(&L.m_xk_c, Y.KXF, rowsX, nk) == 0 && pg::make_map_c(&L.m_xv_c, Y.VXF, rowsX, nv) == 0;
        }
    }
    if (Y.AS16 && pg::make_map(&Y.m_as, Y.AS16, (uint64_t)Y.max_tiles128 * 128, E, pg::BM) == 0 && pg::make_map_c(&Y.m_ysp, Y.YSP, (uint64_t)Y.max_tiles128 * 128, E) == 0)
        for (LyLayer &L : Y.layers) {
            if (L.s.ff_kind != B200_FF_MOE || L.s.ff_dim % 64) continue;
            const uint64_t F = L.s.ff_dim, X = L.s.ff_experts;
            L.tc_moe = pg::make_map(&L.m_moe_gate, L.w_gu, X * 2 * F, E, pg::BN / 2) == 0 && pg::make_map(&L.m_moe_up, L.w_gu + F * E, X * 2 * F - F, E, pg::BN / 2) == 0 &&
                       pg::make_map(&L.m_moe_down, L.w_down, X * E, F, pg::BN) == 0 && pg::make_map(&L.m_moe_h, Y.HS16, (uint64_t)Y.max_tiles128 * 128, F, pg::BM) == 0;
        }
    if (Y.outnorm) ly_outnorm_tc_init(p);
    Y.tc_head = fits(V, E) && pg::make_map(&Y.m_head, Y.head, V, E, 128) == 0 && pg::make_map_c(&Y.m_log_c, Y.LOG, 256, V) == 0;
    Y.tc = true;
    return B200_OK;
}

static int ly_build(b200_plan *p, const b200_layered_config *cfg, const b200_layer_spec *specs, const b200_tensor *tensors, int nt) {
    Layered *Yp = new Layered();
    p->ly = Yp;
    Layered &Y = *Yp;
    Y.c = *cfg;
    const b200_layered_config &c = Y.c;
    if (c.arch != B200_ARCH_PIBIDRA && c.arch != B200_ARCH_LATUSUN && c.arch != B200_ARCH_LEROSUN && c.arch != B200_ARCH_DINUZEN) return fail(p, B200_ERR_UNSUPPORTED, "unknown layered arch %d", c.arch);
    if (c.block != B200_BLOCK_SANDWICH && c.block != B200_BLOCK_PARALLEL && c.block != B200_BLOCK_PRENORM && c.block != B200_BLOCK_OUTNORM) return fail(p, B200_ERR_BAD_ARG, "unknown block kind %d", c.block);
    Y.outnorm = c.block == B200_BLOCK_OUTNORM;
    const bool outn = Y.outnorm;
    if (outn) {
        if (c.loop_times >= 0 && c.loop_stop > c.loop_start) return fail(p, B200_ERR_UNSUPPORTED, "blocks with the norm on the sublayer's output do not loop");
        if (Y.c.norm_groups <= 0) Y.c.norm_groups = 1;
        if (c.width % Y.c.norm_groups || Y.c.norm_groups > LY_OUTNORM_MAX_GROUPS) return fail(p, B200_ERR_BAD_ARG, "width %d in %d norm groups", c.width, Y.c.norm_groups);
    }
    Y.prenorm = c.block == B200_BLOCK_PRENORM;
    Y.w_off = Y.prenorm ? 0.0f : 1.0f;
    const bool par = c.block == B200_BLOCK_PARALLEL;
    if (par && Y.has_loop && c.loop_stop > c.loop_start) return fail(p, B200_ERR_UNSUPPORTED, "parallel blocks do not loop");
    if (c.width <= 0 || c.vocab_size <= 0 || c.n_layers <= 0 || c.context_length <= 0) return fail(p, B200_ERR_BAD_ARG, "width, vocabulary, layers and context must be positive");
    if (c.compute != B200_COMPUTE_BF16 && c.compute != B200_COMPUTE_F32) return fail(p, B200_ERR_BAD_ARG, "compute must be B200_COMPUTE_BF16 or B200_COMPUTE_F32");
    Y.f32 = c.compute == B200_COMPUTE_F32;
    Y.has_loop = c.loop_times >= 0;
    if (Y.c.block == B200_BLOCK_PARALLEL && !(Y.c.residual_mult == Y.c.residual_mult)) return fail(p, B200_ERR_BAD_ARG, "residual multiplier is not a number");
    { const char *e = getenv("B200_LAYERED_ATT"); Y.att_mma = !(e && e[0] == 's'); }
    if (Y.has_loop && (c.loop_start < 0 || c.loop_stop > c.n_layers || c.loop_start > c.loop_stop)) return fail(p, B200_ERR_BAD_ARG, "loop [%d, %d) outside the %d layers", c.loop_start, c.loop_stop, c.n_layers);
    const int E = c.width;
    // the fields of b200_config the shared entry points read
    p->cfg.arch = c.arch; p->cfg.dim = E; p->cfg.n_layers = c.n_layers; p->cfg.vocab_size = c.vocab_size; p->cfg.context_length = c.context_length;
    p->cfg.rms_norm_eps = c.norm_eps; p->cfg.tp_rank = 0; p->cfg.tp_size = 1;
    p->tp.rank = 0; p->tp.n = 1;
    p->wtype = B200_GGML_BF16;
    p->pd_why = "layered plans decode through the CUDA graph";
    p->prefill.why = "layered plans prefill through b200_forward_batch_prefill / b200_forward_batch_logits in the plan's compute mode";

    CK(cudaSetDevice(p->device));
    CK(cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking));
    CK(cudaEventCreate(&p->ev0));
    CK(cudaEventCreate(&p->ev1));
    CK(cudaDeviceGetAttribute(&p->n_sms, cudaDevAttrMultiProcessorCount, p->device));
    CK(cudaDeviceGetAttribute(&Y.smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, p->device));
    int rc;
    Y.cap = p->prefill_batch > 1 ? p->prefill_batch : 1;
    Y.layers.resize(c.n_layers);
    for (int l = 0; l < c.n_layers; l++) {
        LyLayer &L = Y.layers[l];
        L.s = specs[l];
        if (L.s.window > c.context_length) L.s.window = c.context_length; // no position is further back than the context: same result, smaller tables
        const b200_layer_spec &s = L.s;
        if (outn) {
            if ((rc = ly_outnorm_sizes(p, l, L, specs))) return rc;
            continue;
        }
        if (par) {
            // parallel block: latent attention and a mixture of experts (or no feed-forward)
            if (s.mixer != B200_MIXER_LATENT_ATTENTION) return fail(p, B200_ERR_UNSUPPORTED, "layer %d: mixer %d in a parallel block", l, s.mixer);
            L.s.window = c.context_length; // causal over the whole sequence
            if ((rc = ly_latent_sizes(p, l, L, c.n_layers, specs))) return rc;
            if (s.ff_kind != B200_FF_NONE && s.ff_kind != B200_FF_MOE) return fail(p, B200_ERR_UNSUPPORTED, "layer %d: feed-forward kind %d in a parallel block", l, s.ff_kind);
            if (s.ff_kind == B200_FF_MOE) {
                if (s.ff_dim <= 0 || s.ff_experts <= 0 || (size_t)4 * (E + s.ff_experts) * 4 > (size_t)Y.smem_max || s.ff_top <= 0 || s.ff_top > s.ff_experts || (s.ff_act != B200_ACT_GELU_TANH && s.ff_act != B200_ACT_SILU))
                    return fail(p, B200_ERR_BAD_ARG, "layer %d: %d experts of width %d, %d chosen, activation %d", l, s.ff_experts, s.ff_dim, s.ff_top, s.ff_act);
                if (s.ff_dim > Y.maxF) Y.maxF = s.ff_dim;
                if (s.ff_top > Y.maxTop) Y.maxTop = s.ff_top;
                if (s.ff_experts > Y.maxExperts) Y.maxExperts = s.ff_experts;
            }
            if (L.P > Y.maxP) Y.maxP = L.P;
            if (L.gd > Y.maxO) Y.maxO = L.gd;
            if (L.qw > Y.maxQ) Y.maxQ = L.qw;
            if (L.lw > Y.maxL) Y.maxL = L.lw;
            if (s.heads * s.key_dim > Y.maxQU) Y.maxQU = s.heads * s.key_dim;
            if (s.kv_rank > Y.max_att_dv) Y.max_att_dv = s.kv_rank;
            if (L.s.window > Y.max_window) Y.max_window = L.s.window;
            continue;
        }
        if (s.mixer != B200_MIXER_WINDOW_ATTENTION && s.mixer != B200_MIXER_GATED_DELTA) return fail(p, B200_ERR_UNSUPPORTED, "layer %d: mixer %d", l, s.mixer);
        if (s.mixer == B200_MIXER_GATED_DELTA) L.s.window = 1; // a recurrent state, no ring
        if (s.heads <= 0 || s.kv_heads <= 0 || s.heads % s.kv_heads || s.key_dim <= 0 || s.value_dim <= 0 || s.window <= 0)
            return fail(p, B200_ERR_BAD_ARG, "layer %d: heads %d / kv heads %d / key %d / value %d / window %d", l, s.heads, s.kv_heads, s.key_dim, s.value_dim, s.window);
        if (s.ff_kind != B200_FF_NONE && s.ff_kind != B200_FF_DENSE_GATED) return fail(p, B200_ERR_UNSUPPORTED, "layer %d: feed-forward kind %d", l, s.ff_kind);
        if (s.ff_kind == B200_FF_DENSE_GATED && (s.ff_dim <= 0 || (s.ff_act != B200_ACT_GELU_TANH && s.ff_act != B200_ACT_SILU && s.ff_act != B200_ACT_RELU)))
            return fail(p, B200_ERR_BAD_ARG, "layer %d: feed-forward width %d / activation %d", l, s.ff_dim, s.ff_act);
        if (s.ff_kind == B200_FF_DENSE_GATED && s.ff_dim > Y.maxF) Y.maxF = s.ff_dim;
        const bool pad = !Y.f32 && E % 64 == 0; // zero rows up to whole 128-row tiles: the BF16 prefill takes the tcgen05 GEMM; the decode step streams Pn rows
        if (s.mixer == B200_MIXER_GATED_DELTA) {
            if (s.conv_taps < 1 || s.conv_taps > 64) return fail(p, B200_ERR_BAD_ARG, "layer %d: %d convolution taps", l, s.conv_taps);
            L.qd = L.kd = s.kv_heads * s.key_dim; L.vd = L.pv = L.gd = L.gr = s.heads * s.value_dim;
            L.dC = 2 * L.qd + L.vd;
            L.Pn = L.dC + 2 * s.heads + L.gr;
            L.P = pad ? (L.Pn + 127) / 128 * 128 : L.Pn;
            if ((!ly::delta_reg_rows(s.key_dim) && ly::delta_rule_smem_floats(s.key_dim) * 4 > (size_t)Y.smem_max) || (size_t)(s.key_dim > s.value_dim ? s.key_dim : s.value_dim) * 4 > (size_t)Y.smem_max)
                return fail(p, B200_ERR_UNSUPPORTED, "layer %d: a state tile of key size %d or a head of %d values exceeds the shared memory of a CTA", l, s.key_dim, s.value_dim);
            if (L.P > Y.maxP) Y.maxP = L.P;
            if (L.gd > Y.maxO) Y.maxO = L.gd;
            if (L.dC + 2 * s.heads > Y.maxD) Y.maxD = L.dC + 2 * s.heads;
            if (L.gd > Y.maxDO) Y.maxDO = L.gd;
            if (s.conv_taps > Y.max_taps) Y.max_taps = s.conv_taps;
            continue;
        }
        if (s.sink < 0 || s.sink > 2 || s.gate < 0 || s.gate > 2) return fail(p, B200_ERR_BAD_ARG, "layer %d: sink %d / gate %d", l, s.sink, s.gate);
        if (s.rope_dims < 0 || s.rope_dims % 2 || s.rope_dims > s.key_dim || (s.rope_dims > 0 && !(s.rope_base > 0.0f)) || s.yarn_factor != 0.0f)
            return fail(p, B200_ERR_BAD_ARG, "layer %d: rotation of %d of %d entries, base %g", l, s.rope_dims, s.key_dim, (double)s.rope_base);
        if (s.value_from_key && s.value_dim != s.key_dim) return fail(p, B200_ERR_BAD_ARG, "layer %d: values taken from the keys need value size %d = key size %d", l, s.value_dim, s.key_dim);
        L.mixprep = s.rope_dims > 0 || s.value_from_key || s.head_temp || s.head_mix;
        if (L.mixprep && s.qk_norm) return fail(p, B200_ERR_UNSUPPORTED, "layer %d: whole-projection q/k norm together with rotation, key-values, head temperature or head mixing", l);
        if (s.bias_rows < 0 || (s.bias_rows > 0 && (s.bias_rows < 2 || !(s.bias_far > s.bias_rows / 2))))
            return fail(p, B200_ERR_BAD_ARG, "layer %d: distance table of %d rows up to %g", l, s.bias_rows, (double)s.bias_far);
        L.qd = s.heads * s.key_dim; L.kd = s.kv_heads * s.key_dim; L.vd = s.kv_heads * s.value_dim; L.gd = s.heads * s.value_dim;
        L.pv = s.value_from_key ? 0 : L.vd;
        L.gr = s.gate == 2 ? s.heads : s.gate ? L.gd : 0;
        L.P = L.Pn = L.qd + L.kd + L.pv + L.gr;
        if (L.mixprep) {
            if (pad) L.P = (L.Pn + 127) / 128 * 128;
            L.dk_eff = s.head_mix ? L.kd : s.key_dim;
            L.k_heads = s.head_mix ? 1 : s.kv_heads;
            if (s.heads * L.dk_eff > Y.maxQ) Y.maxQ = s.heads * L.dk_eff;
        }
        if (L.P > Y.maxP) Y.maxP = L.P;
        if (L.gd > Y.maxO) Y.maxO = L.gd;
        if (s.window > Y.max_window) Y.max_window = s.window;
        if (s.value_dim > Y.max_att_dv) Y.max_att_dv = s.value_dim;
    }
    {
        int maxK = E > Y.maxO ? E : Y.maxO;
        if (Y.maxF > maxK) maxK = Y.maxF;
        for (const LyLayer &L : Y.layers) if (L.s.kv_rank > maxK) maxK = L.s.kv_rank; // reduction width of the per-head value expansion
        size_t need = (size_t)maxK * 4;
        if (outn && (size_t)2 * E * 4 > need) need = (size_t)2 * E * 4; // the row kernel holds the row and the sublayer's output
        for (const LyLayer &L : Y.layers) if (ly_att_smem(L.s, 0) > need) need = ly_att_smem(L.s, 0);
        if (need > (size_t)Y.smem_max) return fail(p, B200_ERR_UNSUPPORTED, "a row of %zu bytes (widest activation or window) exceeds the %d bytes of shared memory a CTA can hold", need, Y.smem_max);
        static bool attrs = false; // per function and process-wide, like plan.cu's set_smem_attrs
        if (!attrs) {
            CK(set_max_dyn(ly::k_norm_rows, Y.smem_max));
            CK(set_max_dyn(ly::k_block_norm_rows, Y.smem_max));
            CK(set_max_dyn(ly::k_moe_route<float>, Y.smem_max));
            CK(set_max_dyn(ly::k_moe_route<ly::bf16>, Y.smem_max));
            CK(set_max_dyn(ly::k_matvec_bf16<ly::EPI_STORE>, Y.smem_max));
            CK(set_max_dyn(ly::k_matvec_bf16<ly::EPI_GATED>, Y.smem_max));
            CK(set_max_dyn(ly::k_window_attention<float>, Y.smem_max));
            CK(set_max_dyn(ly::k_window_attention<ly::bf16>, Y.smem_max));
            CK(set_max_dyn(ly::k_window_attention_mma<64, 64>, Y.smem_max));
            CK(set_max_dyn(ly::k_window_attention_mma<128, 128>, Y.smem_max));
            CK(set_max_dyn(ly::k_window_attention_mma<192, 128>, Y.smem_max));
            CK(set_max_dyn(ly::k_window_attention_mma<128, 64>, Y.smem_max));
            CK(set_max_dyn(ly::k_window_attention_mma<256, 128>, Y.smem_max));
            CK(set_max_dyn(ly::k_delta_prep, Y.smem_max));
            CK(set_max_dyn(ly::k_rope_mix_prep, Y.smem_max));
            CK(set_max_dyn(ly::k_delta_rule, Y.smem_max));
            CK(set_max_dyn(ly::k_outnorm_rows<LY_NORM_THREADS>, Y.smem_max));
            CK(set_max_dyn(ly::k_outnorm_rows<1024>, Y.smem_max));
            CK(set_max_dyn(ly::k_gated_group_norm, Y.smem_max));
            CK(set_max_dyn(ly::k_matvec_bf16<ly::EPI_ACT>, Y.smem_max));
            attrs = true;
        }
    }
    // Latent attention, BF16 prefill: layers whose per-head key size (unrotated + rotated) and value size are an instance of the
    // tensor-core attention kernel expand keys and values per head for the chunk and run it; all others attend in the folded form
    if (par && !Y.f32 && Y.att_mma && Y.cap > 1 && Y.maxP % 4 == 0)
        for (LyLayer &L : Y.layers) {
            const int DK = L.s.key_dim + L.s.rot_dim;
            const int kind = ly_mma_kind(DK, L.s.value_dim);
            L.expand = kind && ly_mma_smem(kind, L.s.window) <= (size_t)Y.smem_max && (!L.s.gate || L.g_off % 2 == 0) && L.s.key_dim % 8 == 0;
            if (L.expand) {
                if (L.s.heads * DK > Y.maxKX) Y.maxKX = L.s.heads * DK;
                if (L.gd > Y.maxVX) Y.maxVX = L.gd;
            }
        }
    // ring: a step of `cap` rows must not overwrite keys its first rows still see; never more slots than positions
    {
        long long want = (long long)Y.max_window - 1 + Y.cap;
        Y.ring = (int)(want < c.context_length ? want : c.context_length);
        if (Y.ring < 1) Y.ring = 1;
    }
    // unroll the loop into runs
    for (int l = 0; l < c.n_layers;) {
        if (Y.has_loop && l == c.loop_start && c.loop_stop > c.loop_start) {
            for (int t = 0; t < c.loop_times; t++)
                for (int k = c.loop_start; k < c.loop_stop; k++) { LyRun R; R.layer = k; R.pass = t; R.first = k == c.loop_start; Y.runs.push_back(R); }
            l = c.loop_stop;
            continue;
        }
        LyRun R; R.layer = l++; Y.runs.push_back(R);
    }
    if (Y.runs.empty()) return fail(p, B200_ERR_BAD_ARG, "the loop leaves no layer to run");

    const auto t_up0 = std::chrono::steady_clock::now();
    if ((rc = up_init(p, 256))) return rc;
    struct UpGuard { b200_plan *pl; ~UpGuard() { up_destroy(pl); } } guard{p};
    if ((rc = dalloc(p, &Y.emb, (size_t)c.vocab_size * E * 2))) return rc;
    if ((rc = ly_mat(p, tensors, nt, "embed", c.vocab_size, E, Y.emb, 0))) return rc;
    if ((rc = dalloc(p, &Y.head, (size_t)c.vocab_size * E * 2))) return rc;
    if ((rc = ly_mat(p, tensors, nt, "head", c.vocab_size, E, Y.head, 0))) return rc;
    if (outn) {
        if ((rc = ly_vec_f32(p, tensors, nt, "final.norm", E, &Y.final_norm))) return rc;
    } else if (Y.prenorm) {
        if ((rc = ly_scalar_vec(p, tensors, nt, "final.norm", E, &Y.final_norm))) return rc;
        if ((rc = ly_scalar_vec(p, tensors, nt, "embed.norm", E, &Y.emb_norm))) return rc;
    } else if ((rc = ly_vec_f32(p, tensors, nt, "final.norm", E, &Y.final_norm))) return rc;
    if (par && (rc = ly_vec_f32(p, tensors, nt, "final.norm.b", E, &Y.final_norm_b))) return rc;
    if (Y.has_loop && c.loop_times > 0 && !Y.prenorm)
        if ((rc = ly_vec_f32(p, tensors, nt, "loop.step", (int64_t)c.loop_times * E, &Y.step))) return rc;
    for (int l = 0; l < c.n_layers; l++) {
        LyLayer &L = Y.layers[l];
        const b200_layer_spec &s = L.s;
        const std::string pre = "l" + std::to_string(l) + ".", mx = pre + "mix.", ff = pre + "mlp.";
        if (par) {
            if ((rc = ly_latent_upload(p, l, L, tensors, nt))) return rc;
            continue;
        }
        if (outn) {
            if ((rc = ly_outnorm_upload(p, l, L, tensors, nt))) return rc;
            continue;
        }
        if (Y.prenorm) {
            if ((rc = ly_scalar_vec(p, tensors, nt, pre + "norm1", E, &L.norm1))) return rc;
            if ((rc = ly_vec_f32(p, tensors, nt, pre + "ls1", E, &L.ls1))) return rc;
        } else {
            if ((rc = ly_vec_f32(p, tensors, nt, pre + "norm1", E, &L.norm1))) return rc;
            if ((rc = ly_vec_f32(p, tensors, nt, pre + "norm1b", E, &L.norm1b))) return rc;
        }
        if ((rc = dalloc(p, &L.w_proj, (size_t)L.P * E * 2))) return rc;
        if (L.P > L.Pn) CK(cudaMemset(L.w_proj + (size_t)L.Pn * E, 0, (size_t)(L.P - L.Pn) * E * 2));
        if ((rc = ly_mat(p, tensors, nt, mx + "q", L.qd, E, L.w_proj, 0))) return rc;
        if ((rc = ly_mat(p, tensors, nt, mx + "k", L.kd, E, L.w_proj, L.qd))) return rc;
        if (L.pv > 0 && (rc = ly_mat(p, tensors, nt, mx + "v", L.pv, E, L.w_proj, L.qd + L.kd))) return rc;
        if (s.mixer == B200_MIXER_GATED_DELTA) {
            // fused projection rows: q | k | v | b | a | g; the convolution weights of the q | k | v channels in one table
            if ((rc = ly_mat(p, tensors, nt, mx + "b", s.heads, E, L.w_proj, L.dC))) return rc;
            if ((rc = ly_mat(p, tensors, nt, mx + "a", s.heads, E, L.w_proj, L.dC + s.heads))) return rc;
            if ((rc = ly_mat(p, tensors, nt, mx + "g", L.gr, E, L.w_proj, L.dC + 2 * s.heads))) return rc;
            std::vector<float> cw((size_t)L.dC * s.conv_taps);
            const char *nm[3] = {"q.conv", "k.conv", "v.conv"};
            const int off[3] = {0, L.qd, 2 * L.qd}, len[3] = {L.qd, L.kd, L.vd};
            for (int k = 0; k < 3; k++) {
                const b200_tensor *t = find(tensors, nt, mx + nm[k]);
                if (!t || t->ggml_type != B200_GGML_BF16 || t->n_dims != 2 || t->dims[0] != s.conv_taps || t->dims[1] != len[k])
                    return fail(p, B200_ERR_BAD_ARG, "tensor %s%s: BF16 [%d][%d] expected", mx.c_str(), nm[k], len[k], s.conv_taps);
                const uint16_t *src = (const uint16_t *)t->data;
                for (int64_t i = 0; i < (int64_t)len[k] * s.conv_taps; i++) { uint32_t u = (uint32_t)src[i] << 16; memcpy(&cw[(size_t)off[k] * s.conv_taps + i], &u, 4); }
            }
            if ((rc = dalloc(p, &L.conv_w, cw.size() * 4))) return rc;
            CK(cudaMemcpy(L.conv_w, cw.data(), cw.size() * 4, cudaMemcpyHostToDevice));
            if ((rc = ly_vec_f32(p, tensors, nt, mx + "A_log", s.heads, &L.a_log))) return rc;
            if ((rc = ly_vec_f32(p, tensors, nt, mx + "dt_bias", s.heads, &L.dt_bias))) return rc;
            if ((rc = ly_vec_f32(p, tensors, nt, mx + "norm", s.value_dim, &L.onorm))) return rc;
        } else {
        if (s.gate && (rc = ly_mat(p, tensors, nt, mx + "g", L.gr, E, L.w_proj, L.qd + L.kd + L.pv))) return rc;
        if (s.head_temp && (rc = ly_vec_f32(p, tensors, nt, mx + "temp", s.heads, &L.temp))) return rc;
        if (s.head_mix && (rc = ly_vec_f32(p, tensors, nt, mx + "talk", (int64_t)s.heads * s.heads, &L.talk))) return rc;
        if (s.sink == 2 && (rc = ly_vec_f32(p, tensors, nt, mx + "sink", s.heads, &L.sink_logit))) return rc;
        if (s.rope_dims > 0 && (rc = ly_rope_table(p, s, c.context_length, &L.rope))) return rc;
        { // biases of q, k, v in one vector; the gate has none
            std::vector<float> b((size_t)L.P, 0.0f);
            const char *nm[3] = {"q.b", "k.b", "v.b"};
            const int off[3] = {0, L.qd, L.qd + L.kd}, len[3] = {L.qd, L.kd, L.pv};
            bool any = false;
            for (int k = 0; k < 3; k++) {
                if (len[k] == 0) continue;
                const b200_tensor *t = find(tensors, nt, mx + nm[k]);
                if (!t) { if (s.qkv_bias) return fail(p, B200_ERR_BAD_ARG, "missing tensor %s%s", mx.c_str(), nm[k]); continue; }
                if (n_elems(t) != len[k] || t->ggml_type != B200_GGML_BF16) return fail(p, B200_ERR_BAD_ARG, "tensor %s%s: %d BF16 values expected", mx.c_str(), nm[k], len[k]);
                const uint16_t *src = (const uint16_t *)t->data;
                for (int i = 0; i < len[k]; i++) { uint32_t u = (uint32_t)src[i] << 16; memcpy(&b[off[k] + i], &u, 4); }
                any = true;
            }
            if (any && s.qkv_bias) {
                if ((rc = dalloc(p, &L.b_proj, (size_t)L.P * 4))) return rc;
                CK(cudaMemcpy(L.b_proj, b.data(), (size_t)L.P * 4, cudaMemcpyHostToDevice));
            }
        }
        if (s.qk_norm) {
            if ((rc = ly_vec_f32(p, tensors, nt, mx + "q.norm", L.qd, &L.qnorm))) return rc;
            if ((rc = ly_vec_f32(p, tensors, nt, mx + "k.norm", L.kd, &L.knorm))) return rc;
        }
        if (s.bias_rows > 0) {
            if ((rc = ly_vec_f32(p, tensors, nt, mx + "rel", (int64_t)s.bias_rows * s.heads, &L.rel))) return rc;
            std::vector<int> bk((size_t)s.window);
            for (int n = 0; n < s.window; n++) bk[n] = ly_bucket(n, s.bias_rows, (double)s.bias_far);
            if ((rc = dalloc(p, &L.bucket, (size_t)s.window * 4))) return rc;
            CK(cudaMemcpy(L.bucket, bk.data(), (size_t)s.window * 4, cudaMemcpyHostToDevice));
        }
        } // windowed attention
        if ((rc = dalloc(p, &L.w_o, (size_t)E * L.gd * 2))) return rc;
        if ((rc = ly_mat(p, tensors, nt, mx + "o", E, L.gd, L.w_o, 0))) return rc;
        if (s.ff_kind == B200_FF_DENSE_GATED) {
            const int F = s.ff_dim;
            if (Y.prenorm) {
                if ((rc = ly_scalar_vec(p, tensors, nt, pre + "norm2", E, &L.norm2))) return rc;
                if ((rc = ly_vec_f32(p, tensors, nt, pre + "ls2", E, &L.ls2))) return rc;
            } else {
                if ((rc = ly_vec_f32(p, tensors, nt, pre + "norm2", E, &L.norm2))) return rc;
                if ((rc = ly_vec_f32(p, tensors, nt, pre + "norm2b", E, &L.norm2b))) return rc;
            }
            if ((rc = dalloc(p, &L.w_gu, (size_t)2 * F * E * 2))) return rc;
            if ((rc = ly_mat(p, tensors, nt, ff + "gate", F, E, L.w_gu, 0))) return rc;
            if ((rc = ly_mat(p, tensors, nt, ff + "up", F, E, L.w_gu, F))) return rc;
            if ((rc = dalloc(p, &L.w_down, (size_t)E * F * 2))) return rc;
            if ((rc = ly_mat(p, tensors, nt, ff + "down", E, F, L.w_down, 0))) return rc;
        }
    }
    if (p->up.on) CK(cudaStreamSynchronize(p->up.copy));
    p->up.total_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_up0).count();

    // per-run rings
    Y.cring = Y.max_taps > 0 ? Y.max_taps - 1 + Y.cap : 0;
    for (LyRun &R : Y.runs) {
        const LyLayer &L = Y.layers[R.layer];
        if (outn) {
            if ((rc = ly_outnorm_run(p, R, L))) return rc;
            continue;
        }
        if (L.s.mixer == B200_MIXER_LATENT_ATTENTION) {
            // one cache of [latent | rotated shared key part] rows; a layer that reads another layer's cache points at it (runs = layers here)
            R.kw = L.kw;
            if (L.s.kv_from >= 0) { R.own = false; R.kc = Y.runs[L.s.kv_from].kc; R.kc16 = Y.runs[L.s.kv_from].kc16; continue; }
            if ((rc = dalloc(p, &R.kc, (size_t)Y.ring * L.kw * 4))) return rc;
            CK(cudaMemset(R.kc, 0, (size_t)Y.ring * L.kw * 4));
            if (Y.maxKX > 0) { // BF16 twin rows: the A operand of the per-chunk key / value expansion
                if ((rc = dalloc(p, &R.kc16, (size_t)Y.ring * L.kw * 2))) return rc;
                CK(cudaMemset(R.kc16, 0, (size_t)Y.ring * L.kw * 2));
            }
            continue;
        }
        if (L.s.mixer == B200_MIXER_GATED_DELTA) {
            // the run's recurrent state and its ring of convolution inputs (position j in slot j % cring)
            const size_t sb = ly::delta_state_floats(L.s.heads, L.s.key_dim, L.s.value_dim) * 4, cb = (size_t)Y.cring * L.dC * 4;
            R.s_floats = sb / 4; R.c_floats = cb / 4;
            if ((rc = dalloc(p, &R.S, sb))) return rc;
            if ((rc = dalloc(p, &R.cstate, cb))) return rc;
            CK(cudaMemset(R.S, 0, sb));
            CK(cudaMemset(R.cstate, 0, cb));
            continue;
        }
        R.kw = L.kd; R.vw = L.vd;
        if ((rc = dalloc(p, &R.kc, (size_t)Y.ring * L.kd * 4))) return rc;
        if ((rc = dalloc(p, &R.vc, (size_t)Y.ring * L.vd * 4))) return rc;
        CK(cudaMemset(R.kc, 0, (size_t)Y.ring * L.kd * 4));
        CK(cudaMemset(R.vc, 0, (size_t)Y.ring * L.vd * 4));
        // tensor-core prefill attention: BF16 plans, key = value size 64 or 128, a window whose tiles fit shared memory
        const int kind = ly_mma_kind(L.mixprep ? L.dk_eff : L.s.key_dim, L.s.value_dim);
        if (!Y.f32 && Y.att_mma && Y.cap > 1 && kind && ly_mma_smem(kind, L.s.window) <= (size_t)Y.smem_max && Y.maxP % 4 == 0) {
            if ((rc = dalloc(p, &R.kc16, (size_t)Y.ring * L.kd * 2))) return rc;
            if ((rc = dalloc(p, &R.vc16, (size_t)Y.ring * L.vd * 2))) return rc;
            CK(cudaMemset(R.kc16, 0, (size_t)Y.ring * L.kd * 2));
            CK(cudaMemset(R.vc16, 0, (size_t)Y.ring * L.vd * 2));
        }
    }
    // activations
    Y.logit_rows = Y.cap < 128 ? Y.cap : 128;
    Y.cap_pad = Y.f32 ? Y.cap : (Y.cap + 255) / 256 * 256;
    const size_t cap = (size_t)Y.cap_pad, rows32 = Y.f32 ? cap : 1;
    const int maxF = Y.maxF > 0 ? Y.maxF : 1;
    const size_t slots = Y.maxTop > 0 ? (size_t)Y.maxTop : 1; // feed-forward rows per token (a mixture of experts: one per chosen expert)
    if ((rc = dalloc(p, &Y.X, cap * E * 4))) return rc;
    if (Y.has_loop && !Y.prenorm && (rc = dalloc(p, &Y.X0, cap * E * 4))) return rc;
    if (!par && Y.maxQ > 0 && (rc = dalloc(p, &Y.Q, cap * Y.maxQ * 4))) return rc;
    if (outn) {
        if (Y.c.depth_average && (rc = dalloc(p, &Y.STASH, (size_t)(c.n_layers + 1) * Y.cap * E * 4))) return rc;
        if (Y.maxTop > 0 && ((rc = dalloc(p, &Y.SH, cap * E * 4)) || (rc = dalloc(p, &Y.SGL, cap * 4)))) return rc;
        if (!Y.f32 && Y.maxD > 0 && (rc = dalloc(p, &Y.U16, cap * Y.maxD * 2))) return rc;
        if (Y.maxDO > 0 && !Y.DO && (rc = dalloc(p, &Y.DO, cap * Y.maxDO * 4))) return rc;
    }
    if (Y.maxD > 0 && ((rc = dalloc(p, &Y.DLT, cap * Y.maxD * 4)) || (rc = dalloc(p, &Y.DO, cap * (Y.maxDO > 0 ? Y.maxDO : 1) * 4)))) return rc;
    if ((rc = dalloc(p, &Y.Y, cap * E * 4))) return rc;
    if ((rc = dalloc(p, &Y.PROJ, cap * Y.maxP * 4))) return rc;
    if ((rc = dalloc(p, &Y.A32, rows32 * E * 4))) return rc;
    if ((rc = dalloc(p, &Y.ATT32, rows32 * Y.maxO * 4))) return rc;
    if ((rc = dalloc(p, &Y.H32, rows32 * slots * maxF * 4))) return rc;
    if (!Y.f32) {
        if ((rc = dalloc(p, &Y.A16, cap * E * 2))) return rc;
        if ((rc = dalloc(p, &Y.ATT16, cap * Y.maxO * 2))) return rc;
        if ((rc = dalloc(p, &Y.H16, cap * slots * maxF * 2))) return rc;
    }
    if (par || outn) {
        if (Y.maxKX > 0) {
            if ((rc = dalloc(p, &Y.KX16, (size_t)Y.ring * Y.maxKX * 2))) return rc;
            if ((rc = dalloc(p, &Y.VX16, (size_t)Y.ring * Y.maxVX * 2))) return rc;
            const size_t rowsX = ((size_t)Y.ring + 127) / 128 * 128;
            if ((rc = dalloc(p, &Y.KXF, rowsX * Y.maxKX * 4))) return rc;
            if ((rc = dalloc(p, &Y.VXF, rowsX * Y.maxVX * 4))) return rc;
        }
        if (par && (rc = dalloc(p, &Y.A2_32, rows32 * E * 4))) return rc;
        if (par && (rc = dalloc(p, &Y.Q, cap * Y.maxQ * 4))) return rc;
        if (par && (rc = dalloc(p, &Y.LAT32, rows32 * Y.maxL * 4))) return rc;
        if (par && !Y.f32) {
            if ((rc = dalloc(p, &Y.A2_16, cap * E * 2))) return rc;
            if ((rc = dalloc(p, &Y.QU16, cap * Y.maxQU * 2))) return rc;
            if ((rc = dalloc(p, &Y.LAT16, cap * Y.maxL * 2))) return rc;
        }
        if (Y.maxTop > 0) {
            Y.max_tiles = (int)((cap * slots + 63) / 64) + Y.maxExperts;
            if ((rc = dalloc(p, &Y.YS, cap * slots * E * 4))) return rc;
            if ((rc = dalloc(p, &Y.ZR, (size_t)Y.maxExperts * 4))) return rc;
            if ((rc = dalloc(p, &Y.moe_ids, cap * slots * 4))) return rc;
            if ((rc = dalloc(p, &Y.moe_wts, cap * slots * 4))) return rc;
            if ((rc = dalloc(p, &Y.moe_perm, cap * slots * 4))) return rc;
            if ((rc = dalloc(p, &Y.tile_group, (size_t)Y.max_tiles * 4))) return rc;
            if ((rc = dalloc(p, &Y.tile_row0, (size_t)Y.max_tiles * 4))) return rc;
            if ((rc = dalloc(p, &Y.tile_rows, (size_t)Y.max_tiles * 4))) return rc;
            if (!Y.f32 && Y.cap > 1 && E % 128 == 0) { // expert projections of the BF16 prefill on the tcgen05 GEMM
                Y.max_tiles128 = (int)((cap * slots + 127) / 128) + Y.maxExperts;
                const size_t rowsP = (size_t)Y.max_tiles128 * 128;
                if ((rc = dalloc(p, &Y.AS16, rowsP * E * 2))) return rc;
                if ((rc = dalloc(p, &Y.HS16, rowsP * maxF * 2))) return rc;
                if ((rc = dalloc(p, &Y.YSP, rowsP * E * 4))) return rc;
                if ((rc = dalloc(p, &Y.row_scale, rowsP * 4))) return rc;
                if ((rc = dalloc(p, &Y.srt, rowsP * 4))) return rc;
                if ((rc = dalloc(p, &Y.slot_row, cap * slots * 4))) return rc;
                if ((rc = dalloc(p, &Y.tile_group128, (size_t)Y.max_tiles128 * 4))) return rc;
            }
            CK(cudaMemset(Y.moe_ids, 0, cap * slots * 4));
            CK(cudaMemset(Y.moe_wts, 0, cap * slots * 4));
        }
    }
    if ((rc = dalloc(p, &Y.LOG, (size_t)(Y.f32 ? Y.logit_rows : 256) * c.vocab_size * 4))) return rc;
    if ((rc = dalloc(p, &Y.tok, cap * 4))) return rc;
    if ((rc = dalloc(p, &Y.rows, cap * 4))) return rc;
    {
        const char *e = getenv("B200_LAYERED_SPLITS");
        if (e && atoi(e) >= 1) Y.max_splits = atoi(e) > 8 ? 8 : atoi(e);
        int maxH = 1, maxdv = Y.max_att_dv;
        for (const LyLayer &L : Y.layers) if (L.s.heads > maxH) maxH = L.s.heads;
        if (Y.max_att_heads > maxH) maxH = Y.max_att_heads;
        if (Y.max_splits > 1) {
            if ((rc = dalloc(p, &Y.split.o, (size_t)maxH * Y.max_splits * maxdv * 4))) return rc;
            if ((rc = dalloc(p, &Y.split.ml, (size_t)maxH * Y.max_splits * 2 * 4))) return rc;
            if ((rc = dalloc(p, &Y.split.count, (size_t)maxH * 4))) return rc;
            CK(cudaMemset(Y.split.count, 0, (size_t)maxH * 4));
        }
    }
    if ((rc = dalloc(p, &Y.st_pf, sizeof(StepState)))) return rc;
    CK(cudaMemset(Y.st_pf, 0, sizeof(StepState)));
    // what the shared single-token entry points use
    if ((rc = dalloc(p, &p->logits, (size_t)sampler_padded(c.vocab_size) * 4))) return rc;
    CK(cudaMemset(p->logits, 0, (size_t)sampler_padded(c.vocab_size) * 4));
    if ((rc = dalloc(p, &p->smp_indices, (size_t)c.vocab_size * 4))) return rc;
    if ((rc = dalloc(p, &p->smp_out, 8 * 4))) return rc;
    p->seq_cap = (c.context_length > Y.cap ? c.context_length : Y.cap) + 8;
    if ((rc = dalloc(p, &p->st, sizeof(StepState)))) return rc;
    if ((rc = dalloc(p, &p->seq_tokens, (size_t)p->seq_cap * 4))) return rc;
    if ((rc = dalloc(p, &p->out_ids, (size_t)p->seq_cap * 4))) return rc;
    CK(cudaMemset(p->st, 0, sizeof(StepState)));
    CK(cudaMemset(p->seq_tokens, 0, (size_t)p->seq_cap * 4));
    CK(cudaMallocHost(&p->h_st, sizeof(StepState)));
    CK(cudaMallocHost(&p->h_ids, (size_t)p->seq_cap * 4));
    p->x = Y.X;
    if (!Y.f32 && (rc = ly_tc_init(p))) return rc;
    if ((rc = ly_capture(p, true, &p->g_decode, &p->launches_decode))) return rc;
    if ((rc = ly_capture(p, false, &p->g_prefill, nullptr))) return rc;
    CK(cudaStreamSynchronize(p->stream));
    return B200_OK;
}

// One chunk of n <= cap tokens at positions start_pos..: fills the rings; optionally returns the logits of selected rows and
// the residual stream after every run ([runs][n][width]).
static int ly_batch(b200_plan *p, const int32_t *tokens, int n, int start_pos, const int32_t *rows, int n_rows, float *logits_out, float *trace_out) {
    Layered &Y = *p->ly;
    const int E = Y.c.width, V = Y.c.vocab_size;
    if (n > Y.cap) return fail(p, B200_ERR_BAD_ARG, "chunk of %d tokens exceeds prefill_batch_size %d", n, Y.cap);
    if (start_pos < 0 || start_pos + n > Y.c.context_length) return fail(p, B200_ERR_BAD_ARG, "positions %d..%d outside the context (%d)", start_pos, start_pos + n - 1, Y.c.context_length);
    for (int i = 0; i < n; i++)
        if (tokens[i] < 0 || tokens[i] >= V) return fail(p, B200_ERR_BAD_ARG, "token %d out of range", tokens[i]);
    for (int i = 0; i < n_rows; i++)
        if (rows[i] < 0 || rows[i] >= n) return fail(p, B200_ERR_BAD_ARG, "row %d outside the chunk of %d tokens", rows[i], n);
    if (n_rows > 0 && (!rows || !logits_out)) return fail(p, B200_ERR_BAD_ARG, "rows without an output buffer");
    int rc;
    if (trace_out && !Y.trace)
        if ((rc = dalloc(p, &Y.trace, Y.runs.size() * (size_t)Y.cap * E * 4))) return rc;
    memcpy(p->h_ids, tokens, (size_t)n * 4);
    CK(cudaMemcpyAsync(Y.tok, p->h_ids, (size_t)n * 4, cudaMemcpyHostToDevice, p->stream));
    StepState *h = p->h_st;
    memset(h, 0, sizeof(StepState));
    h->token = tokens[0]; h->pos = start_pos;
    CK(cudaMemcpyAsync(Y.st_pf, h, sizeof(StepState), cudaMemcpyHostToDevice, p->stream));
    CK(cudaEventRecord(p->ev0, p->stream));
    Y.pf_pos = start_pos;
    if ((rc = ly_enqueue(p, false, n, Y.st_pf, Y.tok, false, trace_out ? Y.trace : nullptr, &p->launches_prefill))) return rc;
    CK(cudaEventRecord(p->ev1, p->stream));
    CK(cudaStreamSynchronize(p->stream)); // h_ids / h_st are reused below
    CK(cudaEventElapsedTime(&p->prefill_ms, p->ev0, p->ev1));
    for (int r0 = 0; r0 < n_rows; r0 += Y.logit_rows) {
        const int m = n_rows - r0 < Y.logit_rows ? n_rows - r0 : Y.logit_rows;
        memcpy(p->h_ids, rows + r0, (size_t)m * 4);
        CK(cudaMemcpyAsync(Y.rows, p->h_ids, (size_t)m * 4, cudaMemcpyHostToDevice, p->stream));
        if (Y.outnorm) {
            ly::OutNormArgs a = ly_outnorm_args(Y, m);
            a.w_out = Y.final_norm; a.gather = Y.rows; a.st = Y.st_pf;
            a.out32 = Y.f32 ? Y.A32 : nullptr; a.out16 = Y.f32 ? nullptr : Y.A16;
            if ((rc = launch_k(p, false, ly::k_outnorm_rows<LY_NORM_THREADS>, dim3(m), dim3(LY_NORM_THREADS), (size_t)2 * E * 4, a))) return rc;
        } else if (Y.c.block == B200_BLOCK_PARALLEL) {
            ly::BlockNormArgs a = ly_block_norm_args(Y);
            a.w1 = Y.final_norm; a.b1 = Y.final_norm_b; a.gather = Y.rows;
            a.out1_32 = Y.f32 ? Y.A32 : nullptr; a.out1_16 = Y.f32 ? nullptr : Y.A16;
            if ((rc = launch_k(p, false, ly::k_block_norm_rows, dim3(m), dim3(LY_NORM_THREADS), (size_t)E * 4, a))) return rc;
        } else {
            ly::NormArgs a{};
            a.x = Y.X; a.w_pre = Y.final_norm; a.gather = Y.rows; a.eps = Y.c.norm_eps; a.E = E; a.w_off = Y.w_off;
            a.out32 = Y.f32 ? Y.A32 : nullptr; a.out16 = Y.f32 ? nullptr : Y.A16;
            if ((rc = launch_k(p, false, ly::k_norm_rows, dim3(m), dim3(LY_NORM_THREADS), (size_t)E * 4, a))) return rc;
        }
        LyTc t_head;
        if (Y.tc_head) { t_head.a = &Y.m_a; t_head.b = &Y.m_head; t_head.c = &Y.m_log_c; }
        if ((rc = ly_project<ly::EPI_STORE>(p, false, m, Y.A32, Y.A16, Y.head, nullptr, V, E, Y.LOG, nullptr, V, 0, &t_head))) return rc;
        if (Y.c.logit_softcap > 0.0f &&
            (rc = launch_k(p, false, ly::k_softcap, dim3((unsigned)(((size_t)m * V + 255) / 256)), dim3(256), (size_t)0, Y.LOG, (long long)m * V, Y.c.logit_softcap))) return rc;
        CK(cudaMemcpyAsync(logits_out + (size_t)r0 * V, Y.LOG, (size_t)m * V * 4, cudaMemcpyDeviceToHost, p->stream));
        CK(cudaStreamSynchronize(p->stream));
    }
    if (trace_out)
        for (size_t r = 0; r < Y.runs.size(); r++)
            CK(cudaMemcpy(trace_out + r * (size_t)n * E, Y.trace + r * (size_t)Y.cap * E, (size_t)n * E * 4, cudaMemcpyDeviceToHost));
    return B200_OK;
}

static int ly_kv_reset(b200_plan *p) {
    Layered &Y = *p->ly;
    for (LyRun &R : Y.runs) {
        if (R.S) {
            CK(cudaMemsetAsync(R.S, 0, R.s_floats * 4, p->stream));
            CK(cudaMemsetAsync(R.cstate, 0, R.c_floats * 4, p->stream));
        }
        if (R.prev) CK(cudaMemsetAsync(R.prev, 0, (size_t)Y.c.width * 4, p->stream));
        if (!R.own || !R.kc) continue;
        CK(cudaMemsetAsync(R.kc, 0, (size_t)Y.ring * R.kw * 4, p->stream));
        if (R.vc) CK(cudaMemsetAsync(R.vc, 0, (size_t)Y.ring * R.vw * 4, p->stream));
    }
    CK(cudaStreamSynchronize(p->stream));
    return B200_OK;
}

// "x" (row 0 of the residual stream), "logits", "key_cache" / "value_cache" of RUN `layer` ([ring][kv width])
static int ly_read_buffer(b200_plan *p, const char *name, int layer, void *dst, size_t bytes) {
    Layered &Y = *p->ly;
    const std::string s = name;
    const void *src = nullptr;
    size_t sz = 0;
    if (s == "x") { src = Y.X; sz = (size_t)Y.c.width * 4; }
    else if (s == "logits") { src = p->logits; sz = (size_t)Y.c.vocab_size * 4; }
    else if (s == "key_cache" || s == "value_cache") {
        if (layer < 0 || layer >= (int)Y.runs.size()) return fail(p, B200_ERR_BAD_ARG, "run out of range");
        // latent attention keeps ONE cache per layer: "key_cache" = [latent | rotated shared key part] rows, no "value_cache"
        src = s == "key_cache" ? Y.runs[layer].kc : Y.runs[layer].vc;
        sz = (size_t)Y.ring * (s == "key_cache" ? Y.runs[layer].kw : Y.runs[layer].vw) * 4;
        if (!src) return fail(p, B200_ERR_BAD_ARG, "run %d has no %s", layer, name);
    } else if (s == "delta_state" || s == "conv_state") {
        if (layer < 0 || layer >= (int)Y.runs.size() || !Y.runs[layer].S) return fail(p, B200_ERR_BAD_ARG, "run %d has no %s", layer, name);
        src = s == "delta_state" ? Y.runs[layer].S : Y.runs[layer].cstate;
        sz = (s == "delta_state" ? Y.runs[layer].s_floats : Y.runs[layer].c_floats) * 4;
    } else return fail(p, B200_ERR_BAD_ARG, "unknown buffer %s", name);
    if (bytes < sz) sz = bytes;
    CK(cudaSetDevice(p->device));
    CK(cudaStreamSynchronize(p->stream));
    CK(cudaMemcpy(dst, src, sz, cudaMemcpyDeviceToHost));
    return B200_OK;
}

// Stand-alone timing of one projection of the decode step, cycling over the layers so the weights are not L2-resident:
// which 0 = gated feed-forward projection, 1 = down projection, 2 = fused q|k|v|gate projection, 3 = output projection, 4 = classifier.
static int ly_time_kernel(b200_plan *p, int which, int reps, float *avg_ms, int64_t *algorithmic_bytes) {
    Layered &Y = *p->ly;
    const int E = Y.c.width;
    CK(cudaSetDevice(p->device));
    CK(cudaStreamSynchronize(p->stream));
    int launches = 0, rc;
    int64_t bytes = 0, sum_bytes = 0; // layers may differ: the answer is the mean over the timed launches
    auto one = [&](const LyLayer *L) -> int {
        switch (which) {
        case 0: if (!L->w_gu) return B200_OK; bytes = (int64_t)2 * L->s.ff_dim * E * 2; launches++;
                if (L->s.ff_kind == B200_FF_DENSE_PLAIN) { // one matrix, activation in the epilogue
                    bytes /= 2;
                    return ly_project<ly::EPI_ACT>(p, true, 1, Y.A32, nullptr, L->w_gu, nullptr, L->s.ff_dim, E, Y.H32, nullptr, L->s.ff_dim, L->s.ff_act);
                }
                return ly_project<ly::EPI_GATED>(p, true, 1, Y.A32, nullptr, L->w_gu, nullptr, L->s.ff_dim, E, Y.H32, nullptr, L->s.ff_dim, L->s.ff_act);
        case 1: if (!L->w_down) return B200_OK; bytes = (int64_t)L->s.ff_dim * E * 2; launches++;
                return ly_project<ly::EPI_STORE>(p, true, 1, Y.H32, nullptr, L->w_down, nullptr, E, L->s.ff_dim, Y.Y, nullptr, E, 0);
        case 2: bytes = (int64_t)L->Pn * E * 2; launches++;
                return ly_project<ly::EPI_STORE>(p, true, 1, Y.A32, nullptr, L->w_proj, L->b_proj, L->Pn, E, Y.PROJ, nullptr, Y.maxP, 0);
        case 3: bytes = (int64_t)L->gd * E * 2; launches++;
                return ly_project<ly::EPI_STORE>(p, true, 1, Y.ATT32, nullptr, L->w_o, nullptr, E, L->gd, Y.Y, nullptr, E, 0);
        default: bytes = (int64_t)Y.c.vocab_size * E * 2; launches++;
                return ly_project<ly::EPI_STORE>(p, true, 1, Y.A32, nullptr, Y.head, nullptr, Y.c.vocab_size, E, p->logits, nullptr, Y.c.vocab_size, 0);
        }
    };
    if (which < 0 || which > 4) return fail(p, B200_ERR_BAD_ARG, "which must be 0..4");
    for (const LyLayer &L : Y.layers) if ((rc = one(&L))) return rc; // warm-up pass
    launches = 0;
    CK(cudaEventRecord(p->ev0, p->stream));
    for (int r = 0; r < reps; r++)
        for (const LyLayer &L : Y.layers) {
            const int before = launches;
            if ((rc = one(&L))) return rc;
            if (launches > before) sum_bytes += bytes;
            if (which == 4) break;
        }
    CK(cudaEventRecord(p->ev1, p->stream));
    CK(cudaStreamSynchronize(p->stream));
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, p->ev0, p->ev1));
    if (launches == 0) return fail(p, B200_ERR_UNSUPPORTED, "the plan has no such projection");
    *avg_ms = ms / launches;
    if (algorithmic_bytes) *algorithmic_bytes = sum_bytes / launches;
    return B200_OK;
}
