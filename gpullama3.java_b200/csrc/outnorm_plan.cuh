// outnorm_plan.cuh -- host side of the OUTNORM block of layered plans (included by layered_plan.cuh): layers whose sublayers read
// the residual row itself and are normalised on their OUTPUT, x += ls * GN(sublayer(x); w) with GN an RMS norm in groups, with a
// token shift in front of every mixer and the depth average over all earlier layers' results behind every layer.  Per layer the
// mixer is a real-gated linear recurrent unit, a state-space recurrence or a differential attention (which may read another
// layer's key / value rings); the feed-forward a plain activation layer or a softmax-routed mixture of experts with identity
// experts and a gated shared expert.
//
// Kernel sequence of one layer (decode: one row in the CUDA graph; prefill: n rows per launch):
//   row kernel (finishes the previous sublayer: norm, layer scale, residual add; depth average; for one row also the token shift)
//   [-> token shift of the chunk]
//   -> fused projection                                                   (streaming matvec / tcgen05 or mma.sync GEMM)
//   -> attention:   slice norm + rotation + ring write -> attention over (head, map) pairs -> map difference + head norm
//      recurrent unit: convolution over the input ring -> block-diagonal gate products -> two-level scan
//      state space: convolution + SiLU -> recurrence (state columns in registers) -> gated grouped norm
//   -> output projection -> row kernel (x += ls1 * GN(.; norm1); keeps the row the next call's token shift needs)
//   -> plain feed-forward (up + activation, down) or: router -> shared expert -> (prefill: slots grouped by expert) -> experts.
// The next row kernel assembles the mixture (weights on the experts' results, identity experts, gated shared expert).
//
// State per layer RUN: attention rings (position j in slot j % ring; a layer that reads another layer's rings holds pointers),
// the recurrent state (FP32), the ring of convolution inputs, and the last row every mixer read before its shift.  Position 0
// starts from zeros whatever the buffers hold, so requests follow one another without clearing.
#pragma once

static int ly_bf16_host(b200_plan *p, const b200_tensor *tensors, int nt, const std::string &name, int64_t n, std::vector<float> &out) {
    const b200_tensor *t = find(tensors, nt, name);
    if (!t) return fail(p, B200_ERR_BAD_ARG, "missing tensor %s", name.c_str());
    if (n_elems(t) != n) return fail(p, B200_ERR_BAD_ARG, "tensor %s has %lld elements, expected %lld", name.c_str(), (long long)n_elems(t), (long long)n);
    out.resize((size_t)n);
    if (t->ggml_type == B200_GGML_BF16) {
        const uint16_t *s = (const uint16_t *)t->data;
        for (int64_t i = 0; i < n; i++) { uint32_t u = (uint32_t)s[i] << 16; memcpy(&out[i], &u, 4); }
    } else if (t->ggml_type == B200_GGML_F32) memcpy(out.data(), t->data, (size_t)n * 4);
    else return fail(p, B200_ERR_UNSUPPORTED, "tensor %s: type %d (BF16 or F32 expected)", name.c_str(), t->ggml_type);
    return B200_OK;
}

// Validation of one OUTNORM layer and the sizes derived from it.
static int ly_outnorm_sizes(b200_plan *p, int l, LyLayer &L, const b200_layer_spec *specs) {
    Layered &Y = *p->ly;
    b200_layer_spec &s = L.s;
    const int E = Y.c.width;
    const bool pad = !Y.f32 && E % 64 == 0;
    if (s.heads <= 0 || s.kv_heads <= 0 || s.heads % s.kv_heads || s.key_dim <= 0 || s.value_dim <= 0)
        return fail(p, B200_ERR_BAD_ARG, "layer %d: heads %d / groups %d / key %d / value %d", l, s.heads, s.kv_heads, s.key_dim, s.value_dim);
    if (s.mixer == B200_MIXER_WINDOW_ATTENTION) {
        const int maps = s.score_maps > 1 ? s.score_maps : 1;
        if (maps > 2) return fail(p, B200_ERR_UNSUPPORTED, "layer %d: %d score maps", l, maps);
        if (s.sink || s.gate || s.qkv_bias || s.qk_norm || s.bias_rows || s.value_from_key || s.head_temp || s.head_mix)
            return fail(p, B200_ERR_UNSUPPORTED, "layer %d: sink, gate, biases, whole-projection norm, distance bias, key-values, head temperature and head mixing are not combined with this block", l);
        if (s.rope_dims < 0 || s.rope_dims % 2 || s.rope_dims > s.key_dim || (s.rope_dims > 0 && !(s.rope_base > 0.0f)))
            return fail(p, B200_ERR_BAD_ARG, "layer %d: rotation of %d of %d entries, base %g", l, s.rope_dims, s.key_dim, (double)s.rope_base);
        if (s.rope_layout != B200_ROPE_HALF && s.rope_layout != B200_ROPE_INTERLEAVED) return fail(p, B200_ERR_BAD_ARG, "layer %d: rotation layout %d", l, s.rope_layout);
        if (s.yarn_factor > 0.0f && !(s.yarn_original > 0.0f && s.yarn_fast > 0.0f && s.yarn_slow > 0.0f))
            return fail(p, B200_ERR_BAD_ARG, "layer %d: frequency blending needs original length, fast and slow turn counts", l);
        if (s.kv_from >= 0) {
            if (s.kv_from >= l) return fail(p, B200_ERR_BAD_ARG, "layer %d reads the keys of layer %d, which does not run before it", l, s.kv_from);
            const b200_layer_spec &o = specs[s.kv_from];
            if (o.mixer != B200_MIXER_WINDOW_ATTENTION || o.kv_from >= 0) return fail(p, B200_ERR_BAD_ARG, "layer %d reads the keys of layer %d, which has none of its own", l, s.kv_from);
            if (o.kv_heads != s.kv_heads || o.key_dim != s.key_dim || o.value_dim != s.value_dim || (o.score_maps > 1 ? o.score_maps : 1) != maps)
                return fail(p, B200_ERR_BAD_ARG, "layer %d and layer %d differ in key / value heads or sizes", l, s.kv_from);
        }
        s.window = Y.c.context_length; // causal over the whole sequence
        L.qd = s.heads * maps * s.key_dim; L.kd = s.kv_heads * maps * s.key_dim; L.vd = s.kv_heads * s.value_dim; L.gd = s.heads * s.value_dim;
        L.pv = L.vd;
        L.Pn = L.qd + (s.kv_from >= 0 ? 0 : L.kd + L.vd);
        if (s.heads * maps * s.value_dim > Y.maxDO) Y.maxDO = s.heads * maps * s.value_dim;
        if (s.value_dim > Y.max_att_dv) Y.max_att_dv = s.value_dim;
        if (s.heads * maps > Y.max_att_heads) Y.max_att_heads = s.heads * maps;
        if (s.window > Y.max_window) Y.max_window = s.window;
    } else if (s.mixer == B200_MIXER_RGLRU) {
        const int W = s.heads * s.value_dim; // blocks x channels per block
        if (s.conv_taps < 1 || s.conv_taps > 64) return fail(p, B200_ERR_BAD_ARG, "layer %d: %d convolution taps", l, s.conv_taps);
        s.window = 1;
        L.qd = L.gd = W; L.dC = W;
        L.Pn = 2 * W;
        if (W > Y.maxD) Y.maxD = W;
        if (2 * W > Y.maxQ) Y.maxQ = 2 * W;
        if (s.conv_taps > Y.max_taps) Y.max_taps = s.conv_taps;
    } else if (s.mixer == B200_MIXER_SSD) {
        const int inner = s.heads * s.value_dim, gn = s.kv_heads * s.key_dim;
        if (s.conv_taps < 1 || s.conv_taps > 64) return fail(p, B200_ERR_BAD_ARG, "layer %d: %d convolution taps", l, s.conv_taps);
        if (!ly::ssd_reg_rows(s.key_dim)) return fail(p, B200_ERR_UNSUPPORTED, "layer %d: a state of %d rows per column exceeds the 256 the recurrence keeps in registers", l, s.key_dim);
        if (s.mixer_norm_groups < 1 || inner % s.mixer_norm_groups || s.mixer_norm_groups > LY_OUTNORM_MAX_GROUPS)
            return fail(p, B200_ERR_BAD_ARG, "layer %d: %d values in %d norm groups", l, inner, s.mixer_norm_groups);
        s.window = 1;
        L.gd = inner; L.dC = inner + 2 * gn;
        L.Pn = 2 * inner + 2 * gn + s.heads;
        if (L.dC > Y.maxD) Y.maxD = L.dC;
        if (inner > Y.maxDO) Y.maxDO = inner;
        if (s.conv_taps > Y.max_taps) Y.max_taps = s.conv_taps;
    } else return fail(p, B200_ERR_UNSUPPORTED, "layer %d: mixer %d in a block with the norm on the sublayer's output", l, s.mixer);
    L.P = pad ? (L.Pn + 127) / 128 * 128 : L.Pn;
    if (L.gd > Y.maxO) Y.maxO = L.gd;
    int scratch = L.P; // the projection buffer also takes the FP32 result of a plain feed-forward's first product on the tcgen05 route
    if (s.ff_kind == B200_FF_DENSE_PLAIN) {
        if (s.ff_dim <= 0 || s.ff_act < 0 || s.ff_act > B200_ACT_GELU_ERF) return fail(p, B200_ERR_BAD_ARG, "layer %d: feed-forward width %d / activation %d", l, s.ff_dim, s.ff_act);
        if (s.ff_dim > Y.maxF) Y.maxF = s.ff_dim;
        if (s.ff_dim > scratch) scratch = s.ff_dim;
    } else if (s.ff_kind == B200_FF_MOE) {
        const int XI = s.ff_experts + s.moe_identity;
        if (s.moe_router != B200_MOE_SOFTMAX_OUTPUT) return fail(p, B200_ERR_UNSUPPORTED, "layer %d: router kind %d in this block", l, s.moe_router);
        if (s.ff_dim <= 0 || s.ff_experts < 0 || s.moe_identity < 0 || XI <= 0 || s.ff_top <= 0 || s.ff_top > XI || s.ff_act != B200_ACT_SILU || s.moe_shared_ff < 0 ||
            (size_t)(E + 2 * (XI + 1)) * 4 > (size_t)Y.smem_max)
            return fail(p, B200_ERR_BAD_ARG, "layer %d: %d experts + %d identity experts of width %d, %d chosen, activation %d", l, s.ff_experts, s.moe_identity, s.ff_dim, s.ff_top, s.ff_act);
        if (s.ff_dim > Y.maxF) Y.maxF = s.ff_dim;
        if (s.moe_shared_ff > Y.maxF) Y.maxF = s.moe_shared_ff;
        if (s.ff_top > Y.maxTop) Y.maxTop = s.ff_top;
        if (XI + 1 > Y.maxExperts) Y.maxExperts = XI + 1;
    } else if (s.ff_kind != B200_FF_NONE) return fail(p, B200_ERR_UNSUPPORTED, "layer %d: feed-forward kind %d in this block", l, s.ff_kind);
    if (scratch > Y.maxP) Y.maxP = scratch;
    return B200_OK;
}

// Weights of one OUTNORM layer.
static int ly_outnorm_upload(b200_plan *p, int l, LyLayer &L, const b200_tensor *tensors, int nt) {
    Layered &Y = *p->ly;
    const b200_layer_spec &s = L.s;
    const int E = Y.c.width;
    const std::string pre = "l" + std::to_string(l) + ".", mx = pre + "mix.", ff = pre + "mlp.";
    int rc;
    if ((rc = ly_vec_f32(p, tensors, nt, pre + "norm1", E, &L.norm1))) return rc;
    if ((rc = ly_vec_f32(p, tensors, nt, pre + "ls1", E, &L.ls1))) return rc;
    if (Y.c.token_shift && (rc = ly_vec_f32(p, tensors, nt, pre + "shift", E, &L.shift))) return rc;
    if (Y.c.depth_average && (rc = ly_vec_f32(p, tensors, nt, pre + "dwa", l + 2, &L.dwa))) return rc;
    if ((rc = dalloc(p, &L.w_proj, (size_t)L.P * E * 2))) return rc;
    if (L.P > L.Pn) CK(cudaMemset(L.w_proj + (size_t)L.Pn * E, 0, (size_t)(L.P - L.Pn) * E * 2));
    if (s.mixer == B200_MIXER_WINDOW_ATTENTION) {
        if ((rc = ly_mat(p, tensors, nt, mx + "q", L.qd, E, L.w_proj, 0))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "q.norm", s.key_dim, &L.qnorm, s.qk_head_norm != 0))) return rc;
        if (s.kv_from < 0) {
            if ((rc = ly_mat(p, tensors, nt, mx + "k", L.kd, E, L.w_proj, L.qd))) return rc;
            if ((rc = ly_mat(p, tensors, nt, mx + "v", L.vd, E, L.w_proj, L.qd + L.kd))) return rc;
            if ((rc = ly_vec_f32(p, tensors, nt, mx + "k.norm", s.key_dim, &L.knorm, s.qk_head_norm != 0))) return rc;
        }
        if (!s.qk_head_norm) { // no norm: unit weights keep one kernel
            std::vector<float> one((size_t)s.key_dim, 1.0f);
            if ((rc = dalloc(p, &L.qnorm, one.size() * 4)) || (rc = dalloc(p, &L.knorm, one.size() * 4))) return rc;
            CK(cudaMemcpy(L.qnorm, one.data(), one.size() * 4, cudaMemcpyHostToDevice));
            CK(cudaMemcpy(L.knorm, one.data(), one.size() * 4, cudaMemcpyHostToDevice));
        }
        if (s.rope_dims > 0) { if ((rc = ly_rope_table(p, s, Y.c.context_length, &L.rope))) return rc; }
        else if ((rc = dalloc(p, (float **)&L.rope, 16))) return rc;
        if (s.score_maps > 1) { // lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff_init, one number for the layer (evaluated in double)
            std::vector<float> a, b, c, d;
            if ((rc = ly_bf16_host(p, tensors, nt, mx + "lq1", s.key_dim, a)) || (rc = ly_bf16_host(p, tensors, nt, mx + "lk1", s.key_dim, b)) ||
                (rc = ly_bf16_host(p, tensors, nt, mx + "lq2", s.key_dim, c)) || (rc = ly_bf16_host(p, tensors, nt, mx + "lk2", s.key_dim, d))) return rc;
            double s1 = 0.0, s2 = 0.0;
            for (int i = 0; i < s.key_dim; i++) { s1 += (double)a[i] * b[i]; s2 += (double)c[i] * d[i]; }
            L.diff_lambda = (float)(exp(s1) - exp(s2) + (double)s.diff_init);
        }
    } else if (s.mixer == B200_MIXER_RGLRU) {
        const int W = L.qd, nb = s.heads, bs = s.value_dim;
        if ((rc = ly_mat(p, tensors, nt, mx + "x", W, E, L.w_proj, 0))) return rc;
        if ((rc = ly_mat(p, tensors, nt, mx + "y", W, E, L.w_proj, W))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "x.b", W, &L.x_bias))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "y.b", W, &L.y_bias))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "conv", (int64_t)W * s.conv_taps, &L.conv_w))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "conv.b", W, &L.conv_b))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "lam", W, &L.lam))) return rc;
        // gate matrices of block b stacked as [r rows (bs) | i rows (bs)] x bs, their biases in the same order
        const b200_tensor *ta = find(tensors, nt, mx + "ra"), *ti = find(tensors, nt, mx + "ri");
        if (!ta || !ti || ta->ggml_type != B200_GGML_BF16 || ti->ggml_type != B200_GGML_BF16 || n_elems(ta) != (int64_t)nb * bs * bs || n_elems(ti) != (int64_t)nb * bs * bs)
            return fail(p, B200_ERR_BAD_ARG, "tensors %sra / %sri: BF16 [%d][%d][%d] expected", mx.c_str(), mx.c_str(), nb, bs, bs);
        std::vector<uint16_t> g((size_t)nb * 2 * bs * bs);
        for (int b = 0; b < nb; b++) {
            memcpy(&g[(size_t)b * 2 * bs * bs], (const uint16_t *)ta->data + (size_t)b * bs * bs, (size_t)bs * bs * 2);
            memcpy(&g[(size_t)b * 2 * bs * bs + (size_t)bs * bs], (const uint16_t *)ti->data + (size_t)b * bs * bs, (size_t)bs * bs * 2);
        }
        if ((rc = dalloc(p, &L.w_gates, g.size() * 2))) return rc;
        CK(cudaMemcpy(L.w_gates, g.data(), g.size() * 2, cudaMemcpyHostToDevice));
        p->up.h2d_bytes += (int64_t)g.size() * 2;
        std::vector<float> ba, bi, gb((size_t)2 * W);
        if ((rc = ly_bf16_host(p, tensors, nt, mx + "ra.b", W, ba)) || (rc = ly_bf16_host(p, tensors, nt, mx + "ri.b", W, bi))) return rc;
        for (int b = 0; b < nb; b++)
            for (int j = 0; j < bs; j++) { gb[(size_t)b * 2 * bs + j] = ba[(size_t)b * bs + j]; gb[(size_t)b * 2 * bs + bs + j] = bi[(size_t)b * bs + j]; }
        if ((rc = dalloc(p, &L.gate_bias, gb.size() * 4))) return rc;
        CK(cudaMemcpy(L.gate_bias, gb.data(), gb.size() * 4, cudaMemcpyHostToDevice));
    } else { // B200_MIXER_SSD
        if ((rc = ly_mat(p, tensors, nt, mx + "in", L.Pn, E, L.w_proj, 0))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "conv", (int64_t)L.dC * s.conv_taps, &L.conv_w))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "conv.b", L.dC, &L.conv_b))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "A_log", s.heads, &L.a_log))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "dt_bias", s.heads, &L.dt_bias))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "D", s.heads, &L.ssd_d))) return rc;
        if ((rc = ly_vec_f32(p, tensors, nt, mx + "norm", L.gd, &L.onorm))) return rc;
    }
    if ((rc = dalloc(p, &L.w_o, (size_t)E * L.gd * 2))) return rc;
    if ((rc = ly_mat(p, tensors, nt, mx + "o", E, L.gd, L.w_o, 0))) return rc;
    if (s.ff_kind == B200_FF_NONE) return B200_OK;
    if ((rc = ly_vec_f32(p, tensors, nt, pre + "norm2", E, &L.norm2))) return rc;
    if ((rc = ly_vec_f32(p, tensors, nt, pre + "ls2", E, &L.ls2))) return rc;
    if (s.ff_kind == B200_FF_DENSE_PLAIN) {
        const int F = s.ff_dim;
        if ((rc = dalloc(p, &L.w_gu, (size_t)F * E * 2))) return rc;
        if ((rc = ly_mat(p, tensors, nt, ff + "up", F, E, L.w_gu, 0))) return rc;
        if ((rc = dalloc(p, &L.w_down, (size_t)E * F * 2))) return rc;
        return ly_mat(p, tensors, nt, ff + "down", E, F, L.w_down, 0);
    }
    // mixture of experts: router rows [experts | identity experts | gate of the shared expert], stacked expert matrices
    const int F = s.ff_dim, X = s.ff_experts, XI = X + s.moe_identity, SF = s.moe_shared_ff;
    if ((rc = dalloc(p, &L.w_router, (size_t)(XI + 1) * E * 2))) return rc;
    CK(cudaMemset(L.w_router + (size_t)XI * E, 0, (size_t)E * 2));
    if ((rc = ly_mat(p, tensors, nt, ff + "router", XI, E, L.w_router, 0))) return rc;
    if ((rc = ly_vec_f32(p, tensors, nt, ff + "correction", XI, &L.correction))) return rc;
    if (X > 0) {
        if ((rc = dalloc(p, &L.w_gu, (size_t)X * 2 * F * E * 2))) return rc;
        if ((rc = dalloc(p, &L.w_down, (size_t)X * E * F * 2))) return rc;
    }
    for (int e = 0; e < X; e++) {
        const std::string ex = ff + "e" + std::to_string(e) + ".";
        if ((rc = ly_mat(p, tensors, nt, ex + "gate", F, E, L.w_gu, e * 2 * F))) return rc;
        if ((rc = ly_mat(p, tensors, nt, ex + "up", F, E, L.w_gu, e * 2 * F + F))) return rc;
        if ((rc = ly_mat(p, tensors, nt, ex + "down", E, F, L.w_down, e * E))) return rc;
    }
    if (SF > 0) {
        if ((rc = ly_mat(p, tensors, nt, ff + "shared.sg", 1, E, L.w_router, XI))) return rc;
        if ((rc = dalloc(p, &L.w_sgu, (size_t)2 * SF * E * 2))) return rc;
        if ((rc = ly_mat(p, tensors, nt, ff + "shared.gate", SF, E, L.w_sgu, 0))) return rc;
        if ((rc = ly_mat(p, tensors, nt, ff + "shared.up", SF, E, L.w_sgu, SF))) return rc;
        if ((rc = dalloc(p, &L.w_sdown, (size_t)E * SF * 2))) return rc;
        if ((rc = ly_mat(p, tensors, nt, ff + "shared.down", E, SF, L.w_sdown, 0))) return rc;
    }
    return B200_OK;
}

// State of one OUTNORM run: rings of an attention layer (or pointers to the rings it reads), recurrent state and convolution
// ring of a recurrent layer, and the row in front of the next call's token shift.
static int ly_outnorm_run(b200_plan *p, LyRun &R, const LyLayer &L) {
    Layered &Y = *p->ly;
    const b200_layer_spec &s = L.s;
    int rc;
    if (Y.c.token_shift) {
        if ((rc = dalloc(p, &R.prev, (size_t)Y.c.width * 4))) return rc;
        CK(cudaMemset(R.prev, 0, (size_t)Y.c.width * 4));
    }
    if (s.mixer == B200_MIXER_WINDOW_ATTENTION) {
        R.kw = L.kd; R.vw = L.vd;
        if (s.kv_from >= 0) { // runs = layers in this block
            const LyRun &O = Y.runs[s.kv_from];
            R.own = false; R.kc = O.kc; R.vc = O.vc; R.kc16 = O.kc16; R.vc16 = O.vc16;
            return B200_OK;
        }
        if ((rc = dalloc(p, &R.kc, (size_t)Y.ring * L.kd * 4)) || (rc = dalloc(p, &R.vc, (size_t)Y.ring * L.vd * 4))) return rc;
        CK(cudaMemset(R.kc, 0, (size_t)Y.ring * L.kd * 4));
        CK(cudaMemset(R.vc, 0, (size_t)Y.ring * L.vd * 4));
        const int kind = ly_mma_kind(s.key_dim, s.value_dim);
        if (!Y.f32 && Y.att_mma && Y.cap > 1 && kind && ly_mma_smem(kind, s.window) <= (size_t)Y.smem_max && Y.maxP % 4 == 0) {
            if ((rc = dalloc(p, &R.kc16, (size_t)Y.ring * L.kd * 2)) || (rc = dalloc(p, &R.vc16, (size_t)Y.ring * L.vd * 2))) return rc;
            CK(cudaMemset(R.kc16, 0, (size_t)Y.ring * L.kd * 2));
            CK(cudaMemset(R.vc16, 0, (size_t)Y.ring * L.vd * 2));
        }
        return B200_OK;
    }
    R.s_floats = s.mixer == B200_MIXER_RGLRU ? (size_t)L.qd : ly::ssd_state_floats(s.heads, s.key_dim, s.value_dim);
    R.c_floats = (size_t)Y.cring * L.dC;
    if ((rc = dalloc(p, &R.S, R.s_floats * 4)) || (rc = dalloc(p, &R.cstate, R.c_floats * 4))) return rc;
    CK(cudaMemset(R.S, 0, R.s_floats * 4));
    CK(cudaMemset(R.cstate, 0, R.c_floats * 4));
    return B200_OK;
}

// TMA descriptors of the OUTNORM feed-forwards for the tcgen05 GEMMs (the mixers' projections use the common ones).
static void ly_outnorm_tc_init(b200_plan *p) {
    Layered &Y = *p->ly;
    const int E = Y.c.width;
    const uint64_t rows = (uint64_t)Y.cap_pad;
    auto fits = [](int N, int K) { return N % 128 == 0 && K % 64 == 0; };
    const bool sh_c = Y.SH && pg::make_map_c(&Y.m_sh_c, Y.SH, rows, E) == 0;
    for (LyLayer &L : Y.layers) {
        const int F = L.s.ff_dim, SF = L.s.moe_shared_ff;
        if (L.s.ff_kind == B200_FF_DENSE_PLAIN) {
            L.tc_gu = fits(F, E) && Y.maxP % 4 == 0 && pg::make_map(&L.m_up, L.w_gu, F, E, 128) == 0;
            L.tc_down = fits(E, F) && pg::make_map(&L.m_down, L.w_down, E, F, 128) == 0 && pg::make_map(&L.m_h, Y.H16, rows, F, pg::BM) == 0;
        }
        if (L.s.ff_kind == B200_FF_MOE && SF > 0) {
            L.tc_sgu = fits(SF, E) && pg::make_map(&L.m_sgate, L.w_sgu, SF, E, 128) == 0 && pg::make_map(&L.m_sup, L.w_sgu + (size_t)SF * E, SF, E, 128) == 0;
            L.tc_sdown = sh_c && fits(E, SF) && pg::make_map(&L.m_sdown, L.w_sdown, E, SF, 128) == 0 && pg::make_map(&L.m_sh, Y.H16, rows, SF, pg::BM) == 0;
        }
    }
}

static ly::OutNormArgs ly_outnorm_args(const Layered &Y, int n) {
    ly::OutNormArgs a{};
    a.x = Y.X; a.groups = Y.c.norm_groups > 0 ? Y.c.norm_groups : 1; a.eps = Y.c.norm_eps; a.E = Y.c.width; a.n = n;
    a.stash = Y.STASH; a.stash_stride = (long long)Y.cap * Y.c.width; a.stash_idx = -1;
    return a;
}

static int ly_enqueue_outnorm(b200_plan *p, bool decode, int n, const StepState *st, const int *tokens, bool with_head, float *trace, int *launches) {
    Layered &Y = *p->ly;
    const int E = Y.c.width;
    const bool h16 = !decode && !Y.f32; // prefill in BF16 mode rounds GEMM operands to BF16
    int nl = 0, rc;
    ly::OutNormArgs pend = ly_outnorm_args(Y, n); // what the next row kernel finishes
    pend.emb = Y.emb; pend.tokens = tokens; pend.st = st;
    if (Y.c.depth_average) pend.stash_idx = 0;
    auto post = [&](const float *shift, const float *prev, const float *w_out, bool out) {
        ly::OutNormArgs a = pend;
        a.st = st; a.shift = shift; a.prev = prev; a.w_out = w_out;
        if (out) { a.out32 = h16 ? nullptr : Y.A32; a.out16 = h16 ? Y.A16 : nullptr; }
        pend = ly_outnorm_args(Y, n);
        nl++;
        // a single row is one CTA: more threads keep more of its loads in flight
        if (n == 1 && E >= 2048) return launch_k(p, false, ly::k_outnorm_rows<1024>, dim3(1), dim3(1024), (size_t)2 * E * 4, a);
        return launch_k(p, false, ly::k_outnorm_rows<LY_NORM_THREADS>, dim3(n), dim3(LY_NORM_THREADS), (size_t)2 * E * 4, a);
    };
    for (size_t r = 0; r < Y.runs.size(); r++) {
        const LyRun &R = Y.runs[r];
        const LyLayer &L = Y.layers[R.layer];
        const b200_layer_spec &s = L.s;
        // the mixer's input: the (shifted) residual row.  One row: the row kernel shifts it; a chunk: a kernel of its own, because
        // a row needs its neighbour's finished x
        const bool inline_shift = n == 1 || !L.shift;
        if ((rc = post(n == 1 ? L.shift : nullptr, R.prev, nullptr, inline_shift))) return rc;
        if (!inline_shift) {
            if ((rc = launch_k(p, false, ly::k_shift_rows, dim3(n), dim3(256), (size_t)0, (const float *)Y.X, E, (const float *)L.shift, (const float *)R.prev, st,
                               h16 ? (float *)nullptr : Y.A32, h16 ? Y.A16 : (ly::bf16 *)nullptr))) return rc;
            nl++;
        }
        LyTc t_proj, t_o;
        if (Y.tc && !decode) {
            if (L.tc_proj) { t_proj.a = &Y.m_a; t_proj.b = &L.m_proj; t_proj.c = &Y.m_proj_c; }
            if (L.tc_o) { t_o.a = &L.m_att; t_o.b = &L.m_o; t_o.c = &Y.m_y_c; }
        }
        if ((rc = ly_project<ly::EPI_STORE>(p, decode, n, Y.A32, Y.A16, L.w_proj, nullptr, decode ? L.Pn : L.P, E, Y.PROJ, nullptr, Y.maxP, 0, &t_proj))) return rc;
        nl++;
        float *att32 = h16 ? nullptr : Y.ATT32;
        ly::bf16 *att16 = h16 ? Y.ATT16 : nullptr;
        if (s.mixer == B200_MIXER_WINDOW_ATTENTION) {
            const int maps = s.score_maps > 1 ? s.score_maps : 1, pairs = s.heads * maps;
            ly::SliceNormRopeArgs sa{};
            sa.q_slices = pairs; sa.k_slices = s.kv_heads * maps; sa.dk = s.key_dim; sa.v_width = L.vd; sa.has_kv = R.own ? 1 : 0;
            sa.qnorm = L.qnorm; sa.knorm = L.knorm; sa.cs = L.rope; sa.rope_dims = s.rope_dims; sa.rope_layout = s.rope_layout; sa.eps = Y.c.norm_eps; sa.ring = Y.ring;
            if ((rc = launch_k(p, false, ly::k_slice_norm_rope, dim3(n), dim3(256), (size_t)0, Y.PROJ, Y.maxP, sa, R.kc, R.vc, R.own ? R.kc16 : (ly::bf16 *)nullptr,
                               R.own ? R.vc16 : (ly::bf16 *)nullptr, st))) return rc;
            ly::WindowAttn wa{};
            wa.heads = pairs; wa.kv_heads = s.kv_heads; wa.dk = s.key_dim; wa.dv = s.value_dim; wa.window = s.window; wa.ring = Y.ring;
            wa.ldk = L.kd; wa.ldv = L.vd; wa.scale = s.score_scale; wa.softcap = s.softcap; wa.eps = Y.c.norm_eps; wa.maps = maps;
            // with one map the attention writes the mixer's output itself; with two it leaves both maps' rows for the difference
            float *o32 = maps > 1 ? Y.DO : att32;
            const int ldo = maps > 1 ? pairs * s.value_dim : L.gd;
            const int kind = ly_mma_kind(s.key_dim, s.value_dim);
            if (h16 && R.kc16 && kind)
                rc = ly_launch_mma(p, kind, n, pairs, s.window, Y.PROJ, Y.maxP, wa, (const ly::bf16 *)R.kc16, (const ly::bf16 *)R.vc16, st, Y.ATT16, ldo, maps > 1 ? Y.DO : (float *)nullptr);
            else if (h16 && maps == 1)
                rc = launch_k(p, false, ly::k_window_attention<ly::bf16>, dim3(n, pairs), dim3(LY_ATT_THREADS), ly_att_smem(s.key_dim, s.window), (const float *)Y.PROJ, Y.maxP, wa,
                              (const float *)R.kc, (const float *)R.vc, st, Y.ATT16, ldo, ly::KeySplit{nullptr, nullptr, nullptr});
            else {
                int sp = 1;
                if (decode && Y.split.o && s.window >= 64) { sp = p->n_sms / pairs; if (sp > Y.max_splits) sp = Y.max_splits; if (sp < 1) sp = 1; }
                rc = launch_k(p, false, ly::k_window_attention<float>, dim3(n, pairs, sp), dim3(LY_ATT_THREADS), ly_att_smem(s.key_dim, s.window), (const float *)Y.PROJ, Y.maxP, wa,
                              (const float *)R.kc, (const float *)R.vc, st, o32, ldo, sp > 1 ? Y.split : ly::KeySplit{nullptr, nullptr, nullptr});
            }
            if (rc) return rc;
            nl += 2;
            if (maps > 1) {
                if ((rc = launch_k(p, false, ly::k_diff_combine, dim3(n), dim3(256), (size_t)0, (const float *)Y.DO, ldo, s.heads, s.value_dim, L.diff_lambda, 1.0f - s.diff_init, Y.c.norm_eps,
                                   att32, att16, L.gd))) return rc;
                nl++;
            }
        } else if (s.mixer == B200_MIXER_RGLRU) {
            const int W = L.qd, nb = s.heads, bs = s.value_dim;
            ly::ConvArgs ca{};
            ca.C = W; ca.taps = s.conv_taps; ca.cring = Y.cring; ca.w = L.conv_w; ca.bias_in = L.x_bias; ca.bias_out = L.conv_b; ca.silu = 0;
            if ((rc = launch_k(p, false, ly::k_conv_rows, dim3((n + LY_CONV_ROWS - 1) / LY_CONV_ROWS, (W + 255) / 256), dim3(256), (size_t)0, (const float *)Y.PROJ, Y.maxP, 0, ca, R.cstate, Y.DLT, Y.maxD,
                               h16 ? Y.U16 : (ly::bf16 *)nullptr, Y.maxD, st, n))) return rc;
            { // gate logits of every block: [r | i] rows of the block's stacked matrix times the block's channels
                ly::GemmView gv{};
                ly::MvView mv{};
                mv.w_bs = gv.w_bs = (long long)2 * bs * bs; mv.x_bs = bs; mv.y_bs = 2 * bs;
                gv.lda = Y.maxD; gv.a_bs = bs; gv.c_bs = 2 * bs;
                if ((rc = ly_project_view<ly::EPI_STORE>(p, decode, n, Y.DLT, Y.U16, L.w_gates, 2 * bs, bs, Y.Q, nullptr, Y.maxQ, 0, gv, mv, nb, nb, 0))) return rc;
            }
            ly::RglruArgs ra{};
            ra.W = W; ra.blocks = nb; ra.gate_bias = L.gate_bias; ra.lam = L.lam; ra.y_bias = L.y_bias;
            // a chunk: 16 channels x up to 32 row groups per CTA (the last group may be short, never empty rows in between); few rows: 32 channels, one group
            if (n >= 64) rc = launch_k(p, false, ly::k_rglru_scan<16, RGLRU_MAX_GROUPS>, dim3((W + 15) / 16), dim3(16 * RGLRU_MAX_GROUPS), (size_t)0, (const float *)Y.DLT, Y.maxD, (const float *)Y.Q, Y.maxQ,
                                       (const float *)(Y.PROJ + W), Y.maxP, ra, R.S, n, st, att32, att16, L.gd);
            else rc = launch_k(p, false, ly::k_rglru_scan<32, 1>, dim3((W + 31) / 32), dim3(32), (size_t)0, (const float *)Y.DLT, Y.maxD, (const float *)Y.Q, Y.maxQ,
                               (const float *)(Y.PROJ + W), Y.maxP, ra, R.S, n, st, att32, att16, L.gd);
            if (rc) return rc;
            nl += 3;
        } else { // B200_MIXER_SSD
            const int inner = L.gd, gn = s.kv_heads * s.key_dim;
            ly::ConvArgs ca{};
            ca.C = L.dC; ca.taps = s.conv_taps; ca.cring = Y.cring; ca.w = L.conv_w; ca.bias_in = nullptr; ca.bias_out = L.conv_b; ca.silu = 1;
            if ((rc = launch_k(p, false, ly::k_conv_rows, dim3((n + LY_CONV_ROWS - 1) / LY_CONV_ROWS, (L.dC + 255) / 256), dim3(256), (size_t)0, (const float *)Y.PROJ, Y.maxP, inner, ca, R.cstate, Y.DLT, Y.maxD,
                               (ly::bf16 *)nullptr, 0, st, n))) return rc;
            ly::SsdArgs sa{};
            sa.heads = s.heads; sa.groups = s.kv_heads; sa.N = s.key_dim; sa.P = s.value_dim; sa.a_log = L.a_log; sa.dt_bias = L.dt_bias; sa.D = L.ssd_d;
            const dim3 grid(s.heads, (s.value_dim + SSD_COLS - 1) / SSD_COLS), block(SSD_THREADS);
            const float *dt = Y.PROJ + 2 * inner + 2 * gn;
            switch (ly::ssd_reg_rows(s.key_dim)) {
            case 1: rc = launch_k(p, false, ly::k_ssd_scan<1>, grid, block, (size_t)0, (const float *)Y.DLT, Y.maxD, dt, Y.maxP, sa, R.S, n, st, Y.DO, Y.maxDO); break;
            case 2: rc = launch_k(p, false, ly::k_ssd_scan<2>, grid, block, (size_t)0, (const float *)Y.DLT, Y.maxD, dt, Y.maxP, sa, R.S, n, st, Y.DO, Y.maxDO); break;
            case 4: rc = launch_k(p, false, ly::k_ssd_scan<4>, grid, block, (size_t)0, (const float *)Y.DLT, Y.maxD, dt, Y.maxP, sa, R.S, n, st, Y.DO, Y.maxDO); break;
            case 8: rc = launch_k(p, false, ly::k_ssd_scan<8>, grid, block, (size_t)0, (const float *)Y.DLT, Y.maxD, dt, Y.maxP, sa, R.S, n, st, Y.DO, Y.maxDO); break;
            default: rc = launch_k(p, false, ly::k_ssd_scan<16>, grid, block, (size_t)0, (const float *)Y.DLT, Y.maxD, dt, Y.maxP, sa, R.S, n, st, Y.DO, Y.maxDO);
            }
            if (rc) return rc;
            if ((rc = launch_k(p, false, ly::k_gated_group_norm, dim3(n), dim3(n == 1 && inner >= 2048 ? 1024 : 256), (size_t)inner * 4, (const float *)Y.DO, Y.maxDO, (const float *)Y.PROJ, Y.maxP, (const float *)L.onorm, inner,
                               s.mixer_norm_groups, Y.c.norm_eps, att32, att16, L.gd))) return rc;
            nl += 3;
        }
        if ((rc = ly_project<ly::EPI_STORE>(p, decode, n, Y.ATT32, Y.ATT16, L.w_o, nullptr, E, L.gd, Y.Y, nullptr, E, 0, &t_o))) return rc;
        nl++;
        pend.y = Y.Y; pend.w = L.norm1; pend.ls = L.ls1; pend.save_prev = R.prev;
        if (s.ff_kind != B200_FF_NONE) {
            // the feed-forward reads x itself: FP32 from the residual buffer, or its BF16 rounding written by the row kernel
            if ((rc = post(nullptr, nullptr, nullptr, h16))) return rc;
            const float *x32 = Y.X;
            if (s.ff_kind == B200_FF_DENSE_PLAIN) {
                const int F = s.ff_dim;
                LyTc t_down;
                if (Y.tc && !decode && L.tc_down) { t_down.a = &L.m_h; t_down.b = &L.m_down; t_down.c = &Y.m_y_c; }
                if (Y.tc && h16 && L.tc_gu) { // tcgen05 product into the FP32 projection buffer, then the activation into the next operand
                    LyTc t_up; t_up.a = &Y.m_a; t_up.b = &L.m_up; t_up.c = &Y.m_proj_c;
                    if ((rc = ly_project<ly::EPI_STORE>(p, false, n, nullptr, Y.A16, L.w_gu, nullptr, F, E, Y.PROJ, nullptr, Y.maxP, 0, &t_up))) return rc;
                    if ((rc = launch_k(p, false, ly::k_act_rows, dim3(n), dim3(256), (size_t)0, (const float *)Y.PROJ, Y.maxP, F, s.ff_act, Y.H16, F))) return rc;
                    nl += 2;
                } else {
                    if ((rc = ly_project<ly::EPI_ACT>(p, decode, n, x32, Y.A16, L.w_gu, nullptr, F, E, Y.H32, h16 ? Y.H16 : nullptr, F, s.ff_act))) return rc;
                    nl++;
                }
                if ((rc = ly_project<ly::EPI_STORE>(p, decode, n, Y.H32, Y.H16, L.w_down, nullptr, E, F, Y.Y, nullptr, E, 0, &t_down))) return rc;
                nl++;
                pend.y = Y.Y;
            } else {
                const int F = s.ff_dim, X = s.ff_experts, XI = X + s.moe_identity, top = s.ff_top, SF = s.moe_shared_ff;
                const int groups = XI > X ? X + 1 : X; // the identity experts share one id behind the real ones
                const ly::RouteMode rm{1, L.correction, X, s.moe_scale};
                const int extra = SF > 0 ? 1 : 0;
                if (decode) { // one row: the router's rows stream through the multi-CTA matvec, one warp selects
                    if ((rc = ly_project<ly::EPI_STORE>(p, true, 1, x32, nullptr, L.w_router, nullptr, XI + extra, E, Y.ZR, nullptr, XI + extra, 0))) return rc;
                    if ((rc = launch_k(p, false, ly::k_moe_topk, dim3(1), dim3(32), (size_t)2 * XI * 4, (const float *)Y.ZR, XI, top, Y.moe_ids, Y.moe_wts, rm))) return rc;
                    nl += 2;
                } else {
                    const size_t rsm = (size_t)(E + 2 * (XI + extra)) * 4;
                    if (h16) rc = launch_k(p, false, ly::k_moe_route<ly::bf16>, dim3(n), dim3(128), rsm, (const ly::bf16 *)Y.A16, (const ly::bf16 *)L.w_router, n, E, XI, top, 1, Y.moe_ids, Y.moe_wts, rm, extra, Y.SGL);
                    else rc = launch_k(p, false, ly::k_moe_route<float>, dim3(n), dim3(128), rsm, x32, (const ly::bf16 *)L.w_router, n, E, XI, top, 1, Y.moe_ids, Y.moe_wts, rm, extra, Y.SGL);
                    if (rc) return rc;
                    nl++;
                }
                if (SF > 0) { // the shared expert runs for every row; its hidden rows leave the buffer before the experts use it
                    LyTc t_sgu, t_sdown;
                    if (Y.tc && !decode) {
                        if (L.tc_sgu) { t_sgu.a = &Y.m_a; t_sgu.b = &L.m_sgate; t_sgu.b2 = &L.m_sup; t_sgu.c = &Y.m_y_c; }
                        if (L.tc_sdown) { t_sdown.a = &L.m_sh; t_sdown.b = &L.m_sdown; t_sdown.c = &Y.m_sh_c; }
                    }
                    if ((rc = ly_project<ly::EPI_GATED>(p, decode, n, x32, Y.A16, L.w_sgu, nullptr, SF, E, Y.H32, h16 ? Y.H16 : nullptr, SF, s.ff_act, &t_sgu))) return rc;
                    if ((rc = ly_project<ly::EPI_STORE>(p, decode, n, Y.H32, Y.H16, L.w_sdown, nullptr, E, SF, Y.SH, nullptr, E, 0, &t_sdown))) return rc;
                    nl += 2;
                    pend.shared = Y.SH; pend.sg = decode ? Y.ZR + XI : Y.SGL; pend.sg_ld = 1;
                }
                pend.ids = Y.moe_ids; pend.wts = Y.moe_wts; pend.top = top; pend.n_real = X;
                pend.ys = Y.YS; // never read when every chosen expert is an identity
                if (X > 0 && h16 && Y.tc && L.tc_moe) {
                    // tcgen05 route: slots sorted by expert, every expert padded to whole 128-row tiles (identity slots get no row); the
                    // routing weight multiplies the experts' results in the row kernel
                    int t128 = (n * top + 127) / 128 + X;
                    if (t128 > Y.max_tiles128) t128 = Y.max_tiles128;
                    if ((rc = launch_k(p, false, ly::k_moe_group_padded, dim3(1), dim3(1024), (size_t)3 * groups * 4, (const int *)Y.moe_ids, (const float *)Y.moe_wts, n * top, groups, t128, Y.srt,
                                       Y.slot_row, Y.row_scale, Y.tile_group128, X, 1))) return rc;
                    if ((rc = launch_k(p, false, ly::k_moe_gather, dim3(t128 * 128), dim3(128), (size_t)0, (const ly::bf16 *)Y.A16, E, top, (const int *)Y.srt, (const int *)Y.tile_group128, Y.AS16))) return rc;
                    const uint32_t fl = pg::FLAVOR_BF16 | pg::FLAVOR_SILU_BF16;
                    int gr = pg::gemm_launch<pg::GEMM_GATEUP, pg::GEMM_STAGES>(Y.m_as, L.m_moe_gate, L.m_moe_up, Y.m_ysp, Y.HS16, F, t128 * 128, t128, F / (pg::BN / 2), E, p->stream, fl,
                                                                             pg::Grouped{Y.tile_group128, 2 * F, nullptr});
                    if (!gr) gr = pg::gemm_launch<pg::GEMM_F32, pg::GEMM_STAGES>(L.m_moe_h, L.m_moe_down, L.m_moe_down, Y.m_ysp, Y.YSP, E, t128 * 128, t128, E / pg::BN, F, p->stream, pg::FLAVOR_BF16,
                                                                                pg::Grouped{Y.tile_group128, E, nullptr});
                    if (gr) return fail(p, B200_ERR_CUDA, "tensor-core expert GEMM launch failed (%d)", gr);
                    nl += 4;
                    pend.ys = Y.YSP; pend.ys_map = Y.slot_row;
                } else if (X > 0) {
                    int tiles = 0;
                    if (!decode) {
                        tiles = (n * top + 63) / 64 + groups;
                        if (tiles > Y.max_tiles) tiles = Y.max_tiles;
                        if ((rc = launch_k(p, false, ly::k_moe_group, dim3(1), dim3(1024), (size_t)3 * groups * 4, (const int *)Y.moe_ids, n * top, groups, tiles, Y.moe_perm, Y.tile_group, Y.tile_row0,
                                           Y.tile_rows, X))) return rc;
                        nl++;
                    }
                    ly::GemmView gv{};
                    ly::MvView mv{};
                    gv.tile_group = Y.tile_group; gv.tile_row0 = Y.tile_row0; gv.tile_rows = Y.tile_rows; gv.perm = Y.moe_perm;
                    gv.a_div = top; gv.w_gs = mv.w_gs = (long long)2 * F * E;
                    mv.group = Y.moe_ids; mv.y_bs = F; mv.n_groups = X;
                    if ((rc = ly_project_view<ly::EPI_GATED>(p, decode, n, x32, Y.A16, L.w_gu, F, E, Y.H32, h16 ? Y.H16 : nullptr, F, s.ff_act, gv, mv, top, 1, tiles))) return rc;
                    gv.a_div = 1; gv.w_gs = mv.w_gs = (long long)E * F;
                    mv.x_bs = F; mv.y_bs = E;
                    if ((rc = ly_project_view<ly::EPI_STORE>(p, decode, n, Y.H32, Y.H16, L.w_down, E, F, Y.YS, nullptr, E, 0, gv, mv, top, 1, tiles))) return rc;
                    nl += 2;
                }
            }
            pend.w = L.norm2; pend.ls = L.ls2;
        }
        if (Y.c.depth_average) { pend.stash_idx = R.layer + 1; pend.dwa = L.dwa; }
        pend.trace = trace ? trace + r * (size_t)Y.cap * E : nullptr;
    }
    if (decode) {
        if (with_head) {
            if ((rc = post(nullptr, nullptr, Y.final_norm, true))) return rc;
            if ((rc = ly_project<ly::EPI_STORE>(p, true, 1, Y.A32, nullptr, Y.head, nullptr, Y.c.vocab_size, E, p->logits, nullptr, Y.c.vocab_size, 0))) return rc;
            nl++;
        } else if ((rc = post(nullptr, nullptr, nullptr, false))) return rc;
        if ((rc = launch_k(p, false, k_argmax_advance, dim3(1), dim3(1024), (size_t)0, (const float *)p->logits, Y.c.vocab_size, p->st, (const int *)p->seq_tokens,
                           p->out_ids, with_head ? 1 : 0, (const float *)nullptr, (const int *)nullptr, 0, TraceBuf{nullptr, 0, 0}, p->tp, -1))) return rc;
        nl++;
    } else if ((rc = post(nullptr, nullptr, nullptr, false))) return rc;
    if (launches) *launches = nl;
    return B200_OK;
}
