// latent_plan.cuh -- host side of the PARALLEL block of layered plans (included by layered_plan.cuh): layers whose mixer is
// latent attention and whose feed-forward is a mixture of experts, both reading a norm of the same residual row.
//
// Kernel sequence of one layer (decode: one row in the CUDA graph; prefill: n rows per launch):
//   block norm (x += mult * (previous mixer + previous experts), LN1 and LN2 of x)
//   -> fused q | [latent' | shared key part] | gate projection            (streaming matvec / tcgen05 or mma.sync GEMM)
//   -> latent prep (latent RMS norm, rotations, cache write)
//   -> W_uk folded into the query, one product per head                    (batched matvec / GEMM over blockIdx.y / z)
//   -> attention over the cached rows [latent | shared key part]            (k_window_attention, one key/value head for all query heads)
//   -> W_uv per head on the attention's latent-space output, times the sigmoid gate
//      (BF16 prefill of layers whose (key, value) size is (64, 64), (128, 128) or (192, 128) instead: keys and values expanded per head for the chunk,
//       tensor-core attention kernel with the gate in its epilogue)
//   -> output projection
//   -> router -> (prefill: slots grouped by expert) -> gated expert projection -> expert down projection, one result row per slot.
// The next block norm (or the final one) adds both branches to the residual.
//
// Cache: per layer with a W_dkv of its own one FP32 buffer [context][kv_rank + rot_dim]; a layer that reads another layer's
// cache holds a pointer to that buffer and writes nothing.  Slots are positions; a new request overwrites from position 0 and
// never reads beyond its own last position, so nothing is cleared between requests.
#pragma once

// (cos, sin) of every position and rotated pair, evaluated in double: f_i = base^(-2i / dims); with frequency blending
// f_i <- f_i / factor * ramp_i + f_i * (1 - ramp_i), ramp from pair floor(d(fast)) to ceil(d(slow)) where
// d(t) = dims * ln(original / (2 pi t)) / (2 ln base), and both cos and sin times 0.1 ln(factor) + 1.
static int ly_rope_table(b200_plan *p, const b200_layer_spec &s, int positions, const float **out) {
    Layered &Y = *p->ly;
    const std::vector<float> key = {(float)s.rope_dims, s.rope_base, s.yarn_factor, s.yarn_original, s.yarn_fast, s.yarn_slow};
    for (auto &t : Y.rope_tables)
        if (t.first == key) { *out = t.second; return B200_OK; }
    const int dims = s.rope_dims, half = dims / 2;
    std::vector<double> f((size_t)half);
    double mag = 1.0;
    for (int i = 0; i < half; i++) f[i] = pow((double)s.rope_base, -2.0 * i / dims);
    if (s.yarn_factor > 0.0f) {
        const double factor = s.yarn_factor, two_pi = 6.283185307179586476925286766559;
        auto turn_dim = [&](double t) { return dims * log((double)s.yarn_original / (two_pi * t)) / (2.0 * log((double)s.rope_base)); };
        double lo = floor(turn_dim(s.yarn_fast)), hi = ceil(turn_dim(s.yarn_slow));
        if (lo < 0) lo = 0;
        if (hi > dims - 1) hi = dims - 1;
        const double span = hi - lo > 0.001 ? hi - lo : 0.001;
        for (int i = 0; i < half; i++) {
            double ramp = (i - lo) / span;
            ramp = ramp < 0 ? 0 : (ramp > 1 ? 1 : ramp);
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp);
        }
        mag = 0.1 * log(factor) + 1.0;
    }
    std::vector<float> h((size_t)positions * half * 2);
    for (int pos = 0; pos < positions; pos++)
        for (int i = 0; i < half; i++) {
            const double a = (double)pos * f[i];
            h[((size_t)pos * half + i) * 2] = (float)(cos(a) * mag);
            h[((size_t)pos * half + i) * 2 + 1] = (float)(sin(a) * mag);
        }
    float *d = nullptr;
    int rc;
    if ((rc = dalloc(p, &d, h.size() * 4 + 16))) return rc;
    CK(cudaMemcpy(d, h.data(), h.size() * 4, cudaMemcpyHostToDevice));
    Y.rope_tables.push_back({key, d});
    *out = d;
    return B200_OK;
}

// Validation of one latent-attention layer and the sizes derived from it.
static int ly_latent_sizes(b200_plan *p, int l, LyLayer &L, int n_layers, const b200_layer_spec *specs) {
    b200_layer_spec &s = L.s;
    if (s.heads <= 0 || s.key_dim <= 0 || s.value_dim <= 0 || s.rot_dim < 0 || s.kv_rank <= 0)
        return fail(p, B200_ERR_BAD_ARG, "layer %d: heads %d / key %d / rotated %d / value %d / latent %d", l, s.heads, s.key_dim, s.rot_dim, s.value_dim, s.kv_rank);
    if (s.rope_dims < 0 || s.rope_dims > s.rot_dim || (s.rope_dims & 1) || (s.rope_dims > 0 && !(s.rope_base > 0.0f)))
        return fail(p, B200_ERR_BAD_ARG, "layer %d: %d rotated dimensions of %d, base %g", l, s.rope_dims, s.rot_dim, (double)s.rope_base);
    if (s.rope_layout != B200_ROPE_HALF && s.rope_layout != B200_ROPE_INTERLEAVED) return fail(p, B200_ERR_BAD_ARG, "layer %d: rotation layout %d", l, s.rope_layout);
    if (s.yarn_factor > 0.0f && !(s.yarn_original > 0.0f && s.yarn_fast > 0.0f && s.yarn_slow > 0.0f))
        return fail(p, B200_ERR_BAD_ARG, "layer %d: frequency blending needs original length, fast and slow turn counts", l);
    if (s.kv_from >= 0) {
        if (s.kv_from >= l) return fail(p, B200_ERR_BAD_ARG, "layer %d reads the cache of layer %d, which does not run before it", l, s.kv_from);
        const b200_layer_spec &o = specs[s.kv_from];
        if (o.mixer != B200_MIXER_LATENT_ATTENTION || o.kv_from >= 0) return fail(p, B200_ERR_BAD_ARG, "layer %d reads the cache of layer %d, which has none of its own", l, s.kv_from);
        if (o.kv_rank != s.kv_rank || o.rot_dim != s.rot_dim) return fail(p, B200_ERR_BAD_ARG, "layer %d and layer %d differ in latent or rotated size", l, s.kv_from);
    }
    (void)n_layers;
    s.kv_heads = 1;
    L.kw = s.kv_rank + s.rot_dim;
    L.qw = s.heads * L.kw;
    L.lw = s.heads * s.kv_rank;
    L.qd = s.heads * (s.key_dim + s.rot_dim);
    L.kd = L.vd = 0;
    L.gd = s.heads * s.value_dim;
    L.q_off = 0;
    L.kv_off = s.kv_from >= 0 ? -1 : L.qd;
    L.g_off = s.gate ? L.qd + (s.kv_from >= 0 ? 0 : L.kw) : -1;
    L.Pn = L.qd + (s.kv_from >= 0 ? 0 : L.kw) + (s.gate ? L.gd : 0);
    // zero rows up to whole 128-row tiles, so that the prefill takes the tcgen05 GEMM whatever the latent size; the decode step streams Pn rows
    L.P = p->ly->c.width % 64 == 0 ? (L.Pn + 127) / 128 * 128 : L.Pn;
    return B200_OK;
}

// Weights of a parallel-block layer: norms with bias, the fused projection, per-head W_uk^T and W_uv, output, router, experts.
static int ly_latent_upload(b200_plan *p, int l, LyLayer &L, const b200_tensor *tensors, int nt) {
    Layered &Y = *p->ly;
    const b200_layer_spec &s = L.s;
    const int E = Y.c.width;
    const std::string pre = "l" + std::to_string(l) + ".", mx = pre + "mix.", ff = pre + "mlp.";
    int rc;
    if ((rc = ly_vec_f32(p, tensors, nt, pre + "norm1", E, &L.norm1))) return rc;
    if ((rc = ly_vec_f32(p, tensors, nt, pre + "norm1.b", E, &L.ln1_b))) return rc;
    if ((rc = dalloc(p, &L.w_proj, (size_t)L.P * E * 2))) return rc;
    if (L.P > L.Pn) CK(cudaMemset(L.w_proj + (size_t)L.Pn * E, 0, (size_t)(L.P - L.Pn) * E * 2));
    if ((rc = ly_mat(p, tensors, nt, mx + "q", L.qd, E, L.w_proj, 0))) return rc;
    if (s.kv_from < 0) {
        if ((rc = ly_mat(p, tensors, nt, mx + "dkv", L.kw, E, L.w_proj, L.kv_off))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "dkv.norm", s.kv_rank, &L.cnorm))) return rc;
    }
    if (s.gate && (rc = ly_mat(p, tensors, nt, mx + "g", L.gd, E, L.w_proj, L.g_off))) return rc;
    if (s.rope_dims > 0) { if ((rc = ly_rope_table(p, s, Y.c.context_length, &L.rope))) return rc; }
    else if ((rc = dalloc(p, (float **)&L.rope, 16))) return rc;
    { // W_uk [heads * key_dim][kv_rank] -> per head [kv_rank][key_dim], so the folded query is a row-dot product like every other
        const b200_tensor *t = find(tensors, nt, mx + "uk");
        if (!t) return fail(p, B200_ERR_BAD_ARG, "missing tensor %suk", mx.c_str());
        if (t->ggml_type != B200_GGML_BF16 || t->n_dims != 2 || t->dims[0] != s.kv_rank || t->dims[1] != (int64_t)s.heads * s.key_dim)
            return fail(p, B200_ERR_BAD_ARG, "tensor %suk is not BF16 [%d][%d]", mx.c_str(), s.heads * s.key_dim, s.kv_rank);
        const uint16_t *src = (const uint16_t *)t->data;
        std::vector<uint16_t> tr((size_t)s.heads * s.key_dim * s.kv_rank);
        for (int h = 0; h < s.heads; h++)
            for (int d = 0; d < s.key_dim; d++)
                for (int j = 0; j < s.kv_rank; j++)
                    tr[((size_t)h * s.kv_rank + j) * s.key_dim + d] = src[((size_t)h * s.key_dim + d) * s.kv_rank + j];
        if (L.expand) {
            if ((rc = dalloc(p, &L.w_uk, tr.size() * 2))) return rc;
            if ((rc = ly_mat(p, tensors, nt, mx + "uk", s.heads * s.key_dim, s.kv_rank, L.w_uk, 0))) return rc;
        }
        if ((rc = dalloc(p, &L.w_ukT, tr.size() * 2))) return rc;
        if (p->up.on) { if ((rc = up_h2d(p, L.w_ukT, tr.data(), tr.size() * 2))) return rc; }
        else { CK(cudaMemcpy(L.w_ukT, tr.data(), tr.size() * 2, cudaMemcpyHostToDevice)); p->up.h2d_bytes += (int64_t)tr.size() * 2; }
    }
    if ((rc = dalloc(p, &L.w_uv, (size_t)L.gd * s.kv_rank * 2))) return rc;
    if ((rc = ly_mat(p, tensors, nt, mx + "uv", L.gd, s.kv_rank, L.w_uv, 0))) return rc;
    if ((rc = dalloc(p, &L.w_o, (size_t)E * L.gd * 2))) return rc;
    if ((rc = ly_mat(p, tensors, nt, mx + "o", E, L.gd, L.w_o, 0))) return rc;
    if (s.ff_kind == B200_FF_MOE) {
        const int F = s.ff_dim, X = s.ff_experts;
        if ((rc = ly_vec_f32(p, tensors, nt, pre + "norm2", E, &L.norm2))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, pre + "norm2.b", E, &L.ln2_b))) return rc;
        if ((rc = dalloc(p, &L.w_router, (size_t)X * E * 2))) return rc;
        if ((rc = ly_mat(p, tensors, nt, ff + "router", X, E, L.w_router, 0))) return rc;
        if ((rc = dalloc(p, &L.w_gu, (size_t)X * 2 * F * E * 2))) return rc;
        if ((rc = dalloc(p, &L.w_down, (size_t)X * E * F * 2))) return rc;
        for (int e = 0; e < X; e++) {
            const std::string ex = ff + "e" + std::to_string(e) + ".";
            if ((rc = ly_mat(p, tensors, nt, ex + "gate", F, E, L.w_gu, e * 2 * F))) return rc;
            if ((rc = ly_mat(p, tensors, nt, ex + "up", F, E, L.w_gu, e * 2 * F + F))) return rc;
            if ((rc = ly_mat(p, tensors, nt, ex + "down", E, F, L.w_down, e * E))) return rc;
        }
    }
    return B200_OK;
}

// A projection with operand views: decode = the streaming matvec over (rows, yb) CTAs, prefill = the any-shape GEMM of the
// plan's compute mode over (columns, row tiles, zb) CTAs.  tiles > 0: grouped rows (gv.tile_*), else ceil(n / 64) row tiles.
template <int EPI>
static int ly_project_view(b200_plan *p, bool decode, int n, const float *a32, const ly::bf16 *a16, const ly::bf16 *W, int N, int K, float *c32, ly::bf16 *c16,
                           int ldc, int act, const ly::GemmView &gv, const ly::MvView &mv, int yb, int zb, int tiles) {
    Layered &Y = *p->ly;
    if (decode) {
        const int warps = LY_MV_THREADS / 32;
        return launch_k(p, false, ly::k_matvec_bf16<EPI>, dim3((N + warps - 1) / warps, yb), dim3(LY_MV_THREADS), (size_t)K * 4, W, (const float *)nullptr, a32, c32, N, K, act, mv);
    }
    dim3 grid((N + 63) / 64, tiles > 0 ? tiles : (n + 63) / 64, zb);
    const float *nb = nullptr;
    if (Y.f32) {
        if (c16) return fail(p, B200_ERR_STATE, "FP32 plans keep FP32 activations");
        return launch_k(p, false, ly::k_gemm_f32<EPI, float>, grid, dim3(256), (size_t)0, a32, W, nb, c32, n, N, K, ldc, act, gv);
    }
    if (c16) return launch_k(p, false, ly::k_gemm_bf16<EPI, ly::bf16>, grid, dim3(128), (size_t)0, a16, W, nb, c16, n, N, K, ldc, act, gv);
    return launch_k(p, false, ly::k_gemm_bf16<EPI, float>, grid, dim3(128), (size_t)0, a16, W, nb, c32, n, N, K, ldc, act, gv);
}

static ly::BlockNormArgs ly_block_norm_args(const Layered &Y) {
    ly::BlockNormArgs a{};
    a.x = Y.X; a.emb_scale = Y.c.embedding_scale; a.add_mult = Y.c.residual_mult; a.eps = Y.c.norm_eps; a.E = Y.c.width; a.rms = 0;
    return a;
}

static int ly_enqueue_parallel(b200_plan *p, bool decode, int n, const StepState *st, const int *tokens, bool with_head, float *trace, int *launches) {
    Layered &Y = *p->ly;
    const int E = Y.c.width;
    const bool h16 = !decode && !Y.f32; // prefill in BF16 mode rounds GEMM operands to BF16
    int nl = 0, rc;
    const float *pend_a = nullptr, *pend_b = nullptr;
    int pend_terms = 0;
    const int *pend_map = nullptr;
    float *pend_trace = nullptr;
    auto bnorm = [&](bool embed, const float *w1, const float *b1, const float *w2, const float *b2) {
        ly::BlockNormArgs a = ly_block_norm_args(Y);
        a.emb = embed ? Y.emb : nullptr; a.tokens = tokens; a.st = st;
        a.add_a = pend_a; a.add_b = pend_b; a.add_b_terms = pend_terms; a.add_b_map = pend_map; a.trace = pend_trace;
        a.w1 = w1; a.b1 = b1; a.w2 = w2; a.b2 = b2;
        if (w1) { a.out1_32 = h16 ? nullptr : Y.A32; a.out1_16 = h16 ? Y.A16 : nullptr; }
        if (w2) { a.out2_32 = h16 ? nullptr : Y.A2_32; a.out2_16 = h16 ? Y.A2_16 : nullptr; }
        pend_a = pend_b = nullptr; pend_terms = 0; pend_map = nullptr; pend_trace = nullptr;
        nl++;
        return launch_k(p, false, ly::k_block_norm_rows, dim3(n), dim3(LY_NORM_THREADS), (size_t)E * 4, a);
    };
    for (size_t r = 0; r < Y.runs.size(); r++) {
        const LyRun &R = Y.runs[r];
        const LyLayer &L = Y.layers[R.layer];
        const b200_layer_spec &s = L.s;
        const bool moe = s.ff_kind == B200_FF_MOE;
        if ((rc = bnorm(r == 0, L.norm1, L.ln1_b, moe ? L.norm2 : nullptr, L.ln2_b))) return rc;
        LyTc t_proj, t_o;
        if (Y.tc && !decode) {
            if (L.tc_proj) { t_proj.a = &Y.m_a; t_proj.b = &L.m_proj; t_proj.c = &Y.m_proj_c; }
            if (L.tc_o) { t_o.a = &L.m_att; t_o.b = &L.m_o; t_o.c = &Y.m_y_c; }
        }
        if ((rc = ly_project<ly::EPI_STORE>(p, decode, n, Y.A32, Y.A16, L.w_proj, nullptr, decode ? L.Pn : L.P, E, Y.PROJ, nullptr, Y.maxP, 0, &t_proj))) return rc;
        nl++;
        ly::LatentArgs la{};
        la.heads = s.heads; la.dk = s.key_dim; la.dr = s.rot_dim; la.rank = s.kv_rank; la.q_off = L.q_off; la.kv_off = L.kv_off;
        la.cnorm = L.cnorm; la.cs = L.rope; la.rope_dims = s.rope_dims; la.rope_layout = s.rope_layout; la.eps = Y.c.norm_eps;
        if ((rc = launch_k(p, false, ly::k_latent_prep, dim3(n), dim3(256), (size_t)0, Y.PROJ, Y.maxP, la, R.kc, R.own ? R.kc16 : (ly::bf16 *)nullptr, Y.ring, Y.Q, h16 ? Y.QU16 : nullptr, st))) return rc;
        nl++;
        if (h16 && L.expand && R.kc16) {
            // BF16 prefill, (key, value) size an instance of the tensor-core attention: keys and values of every cached position up to the chunk's end are
            // expanded per head (two GEMMs over the BF16 twin of the cache), the rotated shared part is copied behind each head's
            // key, and the tensor-core attention kernel reads [q_u | rot q_r] from the projection rows; gate in its epilogue
            const int DK = s.key_dim + s.rot_dim, M = Y.pf_pos + n;
            const LyRun &O = s.kv_from >= 0 ? Y.runs[s.kv_from] : R;
            if (Y.tc && L.tc_expand && O.tc_lat) {
                // both expansions on the tcgen05 GEMM (FP32 results), then one pass that rounds them to BF16 and appends the rotated shared part
                const int mt = (M + 127) / 128;
                int gr = pg::gemm_launch<pg::GEMM_F32, pg::GEMM_STAGES>(O.m_lat, L.m_xk_b, L.m_xk_b, L.m_xk_c, Y.KXF, s.heads * s.key_dim, M, mt, s.heads * s.key_dim / pg::BN, s.kv_rank, p->stream, pg::FLAVOR_BF16);
                if (!gr) gr = pg::gemm_launch<pg::GEMM_F32, pg::GEMM_STAGES>(O.m_lat, L.m_xv_b, L.m_xv_b, L.m_xv_c, Y.VXF, L.gd, M, mt, L.gd / pg::BN, s.kv_rank, p->stream, pg::FLAVOR_BF16);
                if (gr) return fail(p, B200_ERR_CUDA, "tensor-core expansion GEMM launch failed (%d)", gr);
                if ((rc = launch_k(p, false, ly::k_latent_pack, dim3(M), dim3(256), (size_t)0, (const float *)Y.KXF, (const float *)Y.VXF, (const ly::bf16 *)R.kc16, L.kw, s.kv_rank, s.rot_dim, s.heads,
                                   s.key_dim, s.value_dim, Y.KX16, Y.VX16))) return rc;
            } else {
                ly::GemmView gv{};
                gv.lda = L.kw; gv.w_bs = (long long)s.key_dim * s.kv_rank; gv.c_bs = DK;
                if ((rc = ly_project_view<ly::EPI_STORE>(p, false, M, nullptr, R.kc16, L.w_uk, s.key_dim, s.kv_rank, nullptr, Y.KX16, s.heads * DK, 0, gv, ly::MvView{}, 1, s.heads, 0))) return rc;
                ly::GemmView gv2{};
                gv2.lda = L.kw;
                if ((rc = ly_project_view<ly::EPI_STORE>(p, false, M, nullptr, R.kc16, L.w_uv, L.gd, s.kv_rank, nullptr, Y.VX16, L.gd, 0, gv2, ly::MvView{}, 1, 1, 0))) return rc;
                const long long cells = (long long)M * s.heads * s.rot_dim;
                if (cells > 0 && (rc = launch_k(p, false, ly::k_latent_spread, dim3((unsigned)((cells + 255) / 256)), dim3(256), (size_t)0, (const ly::bf16 *)R.kc16, L.kw, s.kv_rank, s.rot_dim,
                                                s.heads, s.key_dim, Y.KX16, M))) return rc;
            }
            ly::WindowAttn wa{};
            wa.heads = wa.kv_heads = s.heads; wa.dk = DK; wa.dv = s.value_dim; wa.window = s.window; wa.ring = Y.ring; wa.ldk = s.heads * DK; wa.ldv = L.gd;
            wa.scale = s.score_scale; wa.gate = s.gate; wa.gate_off = L.g_off - L.q_off; wa.eps = Y.c.norm_eps;
            rc = ly_launch_mma(p, ly_mma_kind(DK, s.value_dim), n, s.heads, s.window, (const float *)(Y.PROJ + L.q_off), Y.maxP, wa, (const ly::bf16 *)Y.KX16, (const ly::bf16 *)Y.VX16, st,
                               Y.ATT16, L.gd);
            if (rc) return rc;
            nl += 4;
        } else {
            { // folded query: Q[h][0 .. rank) = W_uk[h]^T q_u[h]
                ly::GemmView gv{};
                ly::MvView mv{};
                mv.w_bs = gv.w_bs = (long long)s.kv_rank * s.key_dim;
                mv.x_bs = s.key_dim + s.rot_dim; mv.y_bs = L.kw;
                gv.lda = h16 ? s.heads * s.key_dim : Y.maxP; gv.a_bs = h16 ? s.key_dim : s.key_dim + s.rot_dim; gv.c_bs = L.kw;
                if ((rc = ly_project_view<ly::EPI_STORE>(p, decode, n, Y.PROJ + L.q_off, Y.QU16, L.w_ukT, s.kv_rank, s.key_dim, Y.Q, nullptr, L.qw, 0, gv, mv, s.heads, s.heads, 0))) return rc;
                nl++;
            }
            ly::WindowAttn wa{};
            wa.heads = s.heads; wa.kv_heads = 1; wa.dk = L.kw; wa.dv = s.kv_rank; wa.window = s.window; wa.ring = Y.ring; wa.ldk = wa.ldv = L.kw;
            wa.scale = s.score_scale; wa.softcap = 0.0f; wa.eps = Y.c.norm_eps;
            const size_t asm_ = ly_att_smem(wa.dk, wa.window);
            if (h16) rc = launch_k(p, false, ly::k_window_attention<ly::bf16>, dim3(n, s.heads), dim3(LY_ATT_THREADS), asm_, (const float *)Y.Q, L.qw, wa,
                                   (const float *)R.kc, (const float *)R.kc, st, Y.LAT16, L.lw, ly::KeySplit{nullptr, nullptr, nullptr});
            else {
                int sp = 1;
                if (decode && Y.split.o && s.window >= 64) { sp = p->n_sms / s.heads; if (sp > Y.max_splits) sp = Y.max_splits; if (sp < 1) sp = 1; }
                rc = launch_k(p, false, ly::k_window_attention<float>, dim3(n, s.heads, sp), dim3(LY_ATT_THREADS), asm_, (const float *)Y.Q, L.qw, wa,
                              (const float *)R.kc, (const float *)R.kc, st, Y.LAT32, L.lw, sp > 1 ? Y.split : ly::KeySplit{nullptr, nullptr, nullptr});
            }
            if (rc) return rc;
            nl++;
            { // per head: W_uv on the latent-space output, times sigmoid(gate)
                ly::GemmView gv{};
                ly::MvView mv{};
                mv.w_bs = gv.w_bs = (long long)s.value_dim * s.kv_rank;
                mv.x_bs = s.kv_rank; mv.y_bs = s.value_dim; mv.mul = s.gate ? Y.PROJ + L.g_off : nullptr;
                gv.lda = L.lw; gv.a_bs = s.kv_rank; gv.c_bs = s.value_dim; gv.mul = mv.mul; gv.ldmul = Y.maxP;
                if ((rc = ly_project_view<ly::EPI_STORE>(p, decode, n, Y.LAT32, Y.LAT16, L.w_uv, s.value_dim, s.kv_rank, Y.ATT32, h16 ? Y.ATT16 : nullptr, L.gd, 0, gv, mv,
                                                         s.heads, s.heads, 0))) return rc;
                nl++;
            }
        }
        if ((rc = ly_project<ly::EPI_STORE>(p, decode, n, Y.ATT32, Y.ATT16, L.w_o, nullptr, E, L.gd, Y.Y, nullptr, E, 0, &t_o))) return rc;
        nl++;
        pend_a = Y.Y;
        if (moe) {
            const int F = s.ff_dim, X = s.ff_experts, top = s.ff_top;
            if (decode) { // one row: the router's rows stream through the multi-CTA matvec, one warp selects
                if ((rc = ly_project<ly::EPI_STORE>(p, true, 1, Y.A2_32, nullptr, L.w_router, nullptr, X, E, Y.ZR, nullptr, X, 0))) return rc;
                if ((rc = launch_k(p, false, ly::k_moe_topk, dim3(1), dim3(32), (size_t)2 * X * 4, (const float *)Y.ZR, X, top, Y.moe_ids, Y.moe_wts, ly::RouteMode{0, nullptr, X, 1.0f}))) return rc;
                nl += 2;
            } else {
                const int rpc = 1; // a CTA per row: four warps share the row's experts
                const size_t rsm = (size_t)rpc * (E + 2 * X) * 4;
                const ly::RouteMode rm{0, nullptr, X, 1.0f};
                if (h16) rc = launch_k(p, false, ly::k_moe_route<ly::bf16>, dim3((n + rpc - 1) / rpc), dim3(128), rsm, (const ly::bf16 *)Y.A2_16, (const ly::bf16 *)L.w_router, n, E, X, top, rpc, Y.moe_ids, Y.moe_wts, rm, 0, (float *)nullptr);
                else rc = launch_k(p, false, ly::k_moe_route<float>, dim3((n + rpc - 1) / rpc), dim3(128), rsm, (const float *)Y.A2_32, (const ly::bf16 *)L.w_router, n, E, X, top, rpc, Y.moe_ids, Y.moe_wts, rm, 0, (float *)nullptr);
                if (rc) return rc;
                nl++;
            }
            if (h16 && Y.tc && L.tc_moe) {
                // tcgen05 route: slots sorted by expert, every expert padded to whole 128-row tiles; the rows of LN2(x) are gathered
                // into that order, the gate/up GEMM reads expert tile_group[m tile]'s rows of the stacked matrices and applies the
                // routing weight and the activation in its epilogue, the down GEMM leaves its results in sorted order and the next
                // block norm finds a slot's row through slot_row
                int t128 = (n * top + 127) / 128 + X;
                if (t128 > Y.max_tiles128) t128 = Y.max_tiles128;
                if ((rc = launch_k(p, false, ly::k_moe_group_padded, dim3(1), dim3(1024), (size_t)3 * X * 4, (const int *)Y.moe_ids, (const float *)Y.moe_wts, n * top, X, t128, Y.srt, Y.slot_row,
                                   Y.row_scale, Y.tile_group128, X, 0))) return rc;
                if ((rc = launch_k(p, false, ly::k_moe_gather, dim3(t128 * 128), dim3(128), (size_t)0, (const ly::bf16 *)Y.A2_16, E, top, (const int *)Y.srt, (const int *)Y.tile_group128, Y.AS16))) return rc;
                const uint32_t fl = pg::FLAVOR_BF16 | (s.ff_act == B200_ACT_SILU ? pg::FLAVOR_SILU_BF16 : pg::FLAVOR_GELU_BF16);
                int gr = pg::gemm_launch<pg::GEMM_GATEUP, pg::GEMM_STAGES>(Y.m_as, L.m_moe_gate, L.m_moe_up, Y.m_ysp, Y.HS16, F, t128 * 128, t128, F / (pg::BN / 2), E, p->stream, fl,
                                                                         pg::Grouped{Y.tile_group128, 2 * F, Y.row_scale});
                if (!gr) gr = pg::gemm_launch<pg::GEMM_F32, pg::GEMM_STAGES>(L.m_moe_h, L.m_moe_down, L.m_moe_down, Y.m_ysp, Y.YSP, E, t128 * 128, t128, E / pg::BN, F, p->stream, pg::FLAVOR_BF16,
                                                                            pg::Grouped{Y.tile_group128, E, nullptr});
                if (gr) return fail(p, B200_ERR_CUDA, "tensor-core expert GEMM launch failed (%d)", gr);
                nl += 4;
                pend_b = Y.YSP; pend_map = Y.slot_row; pend_terms = top;
                pend_trace = trace ? trace + r * (size_t)Y.cap * E : nullptr;
                continue;
            }
            int tiles = 0;
            if (!decode) {
                tiles = (n * top + 63) / 64 + X;
                if (tiles > Y.max_tiles) tiles = Y.max_tiles;
                if ((rc = launch_k(p, false, ly::k_moe_group, dim3(1), dim3(1024), (size_t)3 * X * 4, (const int *)Y.moe_ids, n * top, X, tiles, Y.moe_perm, Y.tile_group, Y.tile_row0, Y.tile_rows, X))) return rc;
                nl++;
            }
            ly::GemmView gv{};
            ly::MvView mv{};
            gv.tile_group = Y.tile_group; gv.tile_row0 = Y.tile_row0; gv.tile_rows = Y.tile_rows; gv.perm = Y.moe_perm;
            gv.a_div = top; gv.w_gs = mv.w_gs = (long long)2 * F * E; gv.in_scale = mv.in_scale = Y.moe_wts;
            mv.group = Y.moe_ids; mv.y_bs = F;
            if ((rc = ly_project_view<ly::EPI_GATED>(p, decode, n, Y.A2_32, Y.A2_16, L.w_gu, F, E, Y.H32, h16 ? Y.H16 : nullptr, F, s.ff_act, gv, mv, top, 1, tiles))) return rc;
            nl++;
            gv.a_div = 1; gv.w_gs = mv.w_gs = (long long)E * F; gv.in_scale = mv.in_scale = nullptr;
            mv.x_bs = F; mv.y_bs = E;
            if ((rc = ly_project_view<ly::EPI_STORE>(p, decode, n, Y.H32, Y.H16, L.w_down, E, F, Y.YS, nullptr, E, 0, gv, mv, top, 1, tiles))) return rc;
            nl++;
            pend_b = Y.YS; pend_terms = top;
        }
        pend_trace = trace ? trace + r * (size_t)Y.cap * E : nullptr;
    }
    if (decode) {
        if (with_head) {
            if ((rc = bnorm(false, Y.final_norm, Y.final_norm_b, nullptr, nullptr))) return rc;
            if ((rc = ly_project<ly::EPI_STORE>(p, true, 1, Y.A32, nullptr, Y.head, nullptr, Y.c.vocab_size, E, p->logits, nullptr, Y.c.vocab_size, 0))) return rc;
            nl++;
            if (Y.c.logit_softcap > 0.0f) {
                if ((rc = launch_k(p, false, ly::k_softcap, dim3((Y.c.vocab_size + 255) / 256), dim3(256), (size_t)0, p->logits, (long long)Y.c.vocab_size, Y.c.logit_softcap))) return rc;
                nl++;
            }
        } else if ((rc = bnorm(false, nullptr, nullptr, nullptr, nullptr))) return rc;
        if ((rc = launch_k(p, false, k_argmax_advance, dim3(1), dim3(1024), (size_t)0, (const float *)p->logits, Y.c.vocab_size, p->st, (const int *)p->seq_tokens,
                           p->out_ids, with_head ? 1 : 0, (const float *)nullptr, (const int *)nullptr, 0, TraceBuf{nullptr, 0, 0}, p->tp, -1))) return rc;
        nl++;
    } else if ((rc = bnorm(false, nullptr, nullptr, nullptr, nullptr))) return rc;
    if (launches) *launches = nl;
    return B200_OK;
}
