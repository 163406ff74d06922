"""CPU tests of the Dinuzen support code: config.json registry and the C-ABI structures, synthetic model directories, and
properties of the float64 oracle the GPU tests compare against, one mechanism at a time."""
import ctypes
import math

import numpy as np
import pytest

from dinuzen_util import configs, decisive_routing, min_margin, needle_attention, needle_rglru, needle_ssd, oracle, rel_rms, w64


def test_config_registry_and_abi_structs(pkg, tmp_path):
    S = pkg.synth
    cfg = configs(S)["shared_keys"]
    w = S.dinuzen_weights(cfg, 0)
    d = str(tmp_path / "m")
    S.write_model_dir(d, cfg, w)
    m = pkg.load_model(d, 77)
    c = m.configuration
    assert m.model_type == "DINUZEN" and c.arch == pkg.loader.ARCH_DINUZEN and c.context_length == 77
    assert (c.width, c.vocab_size, c.n_layers, c.block, c.loop, c.norm_eps, c.norm_groups, c.token_shift, c.depth_average) == (48, 80, 5, "outnorm", None, 1e-6, 3, True, True)
    l0, l1, l2, l3 = c.layers[:4]
    assert (l0.mixer, l0.heads, l0.kv_heads, l0.key_dim, l0.value_dim, l0.window, l0.score_maps, l0.qk_head_norm, l0.kv_from, l0.ff_dim) == ("window_attention", 3, 3, 10, 14, 77, 2, True, -1, 0)
    assert (l0.rope_dims, l0.rope_layout, l0.yarn, l0.score_scale, l0.softcap, l0.diff_init) == (10, "interleaved", (4.0, 32.0, 8.0, 1.0), pytest.approx(0.3), 30.0, pytest.approx(0.3))
    assert (l1.mixer, l1.heads, l1.kv_heads, l1.key_dim, l1.value_dim, l1.conv_taps, l1.mixer_norm_groups, l1.ff_kind, l1.ff_act, l1.ff_dim) == ("ssd", 2, 1, 20, 12, 3, 3, "dense_plain", "gelu_erf", 40)
    assert (l2.kv_from, l2.ff_kind, l2.ff_experts, l2.ff_top, l2.moe_identity, l2.moe_scale, l2.moe_shared_ff, l2.moe_router, l2.softcap) == (0, "moe", 5, 3, 2, 2.0, 12, "softmax_output", 5.0)
    assert (l3.mixer, l3.heads, l3.value_dim, l3.conv_taps, l3.ff_dim) == ("rglru", 3, 8, 2, 0)
    assert "l2.mix.k" not in m.tensors and m.tensors["l2.mlp.router"][1] == (48, 7) and m.tensors["l3.mix.ra"][1] == (8, 8, 3) and m.tensors["l4.dwa"][1] == (6,)
    lc, specs = pkg.plan.make_layered_config(m, "float32")
    assert (lc.arch, lc.block, lc.compute, lc.norm_groups, lc.token_shift, lc.depth_average, lc.loop_times) == (6, 3, 1, 3, 1, 1, -1)
    assert (specs[0].mixer, specs[0].score_maps, specs[0].qk_head_norm, specs[0].rope_layout, specs[0].ff_kind) == (1, 2, 1, 1, 0)
    assert (specs[1].mixer, specs[1].mixer_norm_groups, specs[1].ff_kind, specs[1].ff_act) == (5, 3, 3, 3)
    assert (specs[2].moe_router, specs[2].moe_identity, specs[2].moe_shared_ff, specs[2].kv_from, specs[3].mixer) == (1, 2, 12, 0, 4)
    assert ctypes.sizeof(pkg.native.LayerSpec) == 41 * 4 and ctypes.sizeof(pkg.native.LayeredConfig) == 17 * 4
    # in-memory model = on-disk model
    mm = S.dinuzen_model(cfg, w, 77)
    assert mm.configuration == c and all(np.array_equal(mm.tensors[k][2], m.tensors[k][2]) for k in m.tensors)
    # absent optional keys: no scaling, no cap, no identity experts, no shared expert, no feed-forward
    bare = S.dinuzen_config(32, 40, [S.dinuzen_attention(2, 1, 8, 8, S.dinuzen_moe(3, 1, 8))])
    del bare["layers"][0]["mixer"]["softcap"], bare["layers"][0]["mlp"]["router"]["identity"], bare["layers"][0]["mlp"]["shared"]
    b = pkg.loader.dinuzen_configuration(bare, {}, 8).layers[0]
    assert (b.softcap, b.yarn, b.moe_identity, b.moe_shared_ff, b.kv_from) == (0.0, (0.0, 0.0, 0.0, 0.0), 0, 0, -1)
    # unknown mixer / feed-forward kinds are refused; so is a reader of another layer's keys with projections of its own
    with pytest.raises(pkg.loader.UnsupportedModel):
        pkg.loader.dinuzen_configuration(dict(cfg, layers=[dict(cfg["layers"][0], type="delta")]), {}, 8)
    with pytest.raises(pkg.loader.UnsupportedModel):
        pkg.loader.dinuzen_configuration(dict(cfg, layers=[dict(cfg["layers"][0], mlp={"kind": "gated"})]), {}, 8)
    with pytest.raises(pkg.loader.UnsupportedModel):
        pkg.loader.dinuzen_configuration(cfg, {"l2.mix.k": (60, 48)}, 8)
    # the earlier designs keep their defaults
    p = pkg.loader.pibidra_configuration(S.pibidra_config(32, 40, [S.pibidra_layer(2, 1, 8, 8, 4, 16)]), {"l0.mix.rel": (8, 2)}, 8)
    assert (p.layers[0].score_maps, p.layers[0].moe_router, p.norm_groups, p.token_shift, p.depth_average) == (1, "sigmoid_input", 1, False, False)


def test_grouped_norm_shift_and_depth_average():
    O = oracle()
    rng = np.random.default_rng(1)
    v = rng.standard_normal((3, 12)) + 2.0
    y = O.group_rms_norm(v, None, 3, 0.0)
    assert np.allclose((y.reshape(3, 3, 4) ** 2).mean(-1), 1.0)                     # every part has unit mean square of its own
    assert not np.allclose(y, O.group_rms_norm(v, None, 1, 0.0))
    assert np.all(np.abs(O.group_rms_norm(v * 1e-6, None, 3, 1e-2)) < 1e-4)         # eps sits inside the root
    wv = rng.standard_normal(12)
    assert np.allclose(O.group_rms_norm(v, wv, 2, 1e-5), O.group_rms_norm(v, None, 2, 1e-5) * wv)
    x = rng.standard_normal((5, 4))
    s = np.array([0.0, 1.0, 0.25, -1.0])
    h = O.token_shift(x, s)
    assert np.array_equal(h[:, 0], x[:, 0]) and np.allclose(h[1:, 1], x[:-1, 1], rtol=0, atol=1e-15) and h[0, 1] == 0.0   # shift 1: the previous row, zeros first
    assert np.allclose(h[2, 2], 0.75 * x[2, 2] + 0.25 * x[1, 2]) and np.allclose(h[0], x[0] * (1 - s))
    X = [rng.standard_normal((2, 3)) for _ in range(3)]
    assert np.allclose(O.depth_average(X, np.array([0.5, 0.0, 2.0])), 0.5 * X[0] + 2.0 * X[2])


def test_rotation_pairs_frequencies_and_blending():
    O = oracle()
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 12)), rng.standard_normal((1, 12))
    for rot in ({"dims": 8, "base": 50.0}, {"dims": 12, "base": 3.0, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}, {"dims": 0, "base": 10.0}):
        mag = O.rope_frequencies(rot)[1] if rot["dims"] else 1.0
        s = [(O.rotate_interleaved(q, [i], rot) @ O.rotate_interleaved(k, [j], rot).T).item() for i, j in ((7, 3), (104, 100), (4, 0))]
        assert s[0] == pytest.approx(s[1]) == pytest.approx(s[2])                     # a score depends on the distance only
        r = O.rotate_interleaved(q, [9], rot)
        assert np.array_equal(r[:, rot["dims"]:], q[:, rot["dims"]:])                 # entries from `dims` on pass unchanged
        assert np.allclose(O.rotate_interleaved(q, [0], rot)[:, :rot["dims"]], q[:, :rot["dims"]] * mag)
    e0 = np.zeros((1, 8)); e0[0, 0] = 1.0
    r = O.rotate_interleaved(e0, [1], {"dims": 8, "base": 10.0})
    assert r[0, 0] == pytest.approx(math.cos(1.0)) and r[0, 1] == pytest.approx(math.sin(1.0)) and not r[0, 2:].any()   # entry 0 turns with entry 1
    f, mag = O.rope_frequencies({"dims": 8, "base": 100.0})
    assert np.allclose(f, 100.0 ** (-np.arange(4) / 4)) and mag == 1.0
    rot = {"dims": 16, "base": 10000.0, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0}}
    f2, mag2 = O.rope_frequencies(rot)
    f0 = 10000.0 ** (-np.arange(8) / 8)
    assert mag2 == pytest.approx(0.1 * math.log(8.0) + 1.0)
    assert f2[0] == pytest.approx(f0[0]) and f2[-1] == pytest.approx(f0[-1] / 8.0) and np.all(np.diff(f2 / f0) <= 1e-12)   # fast pairs keep, slow pairs stretch


def test_differential_attention_pieces():
    O = oracle()
    rng = np.random.default_rng(2)
    E, H, G, d, dv, T = 24, 4, 2, 6, 5, 9
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "rot": {"dims": 4, "base": 20.0}, "scale": 0.4, "softcap": 3.0, "diff": 0.25}
    w = {"q": rng.standard_normal((H * 2 * d, E)), "k": rng.standard_normal((G * 2 * d, E)), "v": rng.standard_normal((G * dv, E)), "o": np.eye(H * dv),
         "q.norm": rng.standard_normal(d), "k.norm": rng.standard_normal(d), "lq1": rng.standard_normal(d) * 0.3, "lk1": rng.standard_normal(d) * 0.3,
         "lq2": rng.standard_normal(d) * 0.3, "lk2": rng.standard_normal(d) * 0.3}
    h = rng.standard_normal((T, E))
    kv = O.attention_keys_values(h, w, "", m, 1e-5)
    out = O.mixer_attention(h, w, "", m, 1e-5, kv).reshape(T, H, dv)
    assert np.allclose((out ** 2).mean(-1), (1 - 0.25) ** 2, rtol=1e-3)               # head norm without weight, times (1 - diff)
    lam = O.diff_lambda(w, "", 0.25)
    assert lam == pytest.approx(math.exp(w["lq1"] @ w["lk1"]) - math.exp(w["lq2"] @ w["lk2"]) + 0.25)
    # causal: a later token changes nothing earlier; the first token attends to itself alone, so both maps return its value
    h2 = h.copy(); h2[-1] += 1.0
    out2 = O.mixer_attention(h2, w, "", m, 1e-5, O.attention_keys_values(h2, w, "", m, 1e-5)).reshape(T, H, dv)
    assert np.allclose(out[:-1], out2[:-1]) and not np.allclose(out[-1], out2[-1])
    v0 = kv[1][0]
    for hd in range(H):
        o = v0[hd // 2] * (1 - lam)
        assert np.allclose(out[0, hd], o / np.sqrt((o * o).mean() + 1e-5) * 0.75)
    # the cap bounds every score; the norm is per slice with ONE weight for all heads and maps
    assert np.all(np.abs(O.softcap(np.array([-1e3, 0.5, 1e3]), 3.0)) <= 3.0) and O.softcap(np.array([0.01]), 3.0)[0] == pytest.approx(0.01, rel=1e-4)
    k_raw = (h @ w["k"].T).reshape(T, G, 2, d)
    kn = O.group_rms_norm(k_raw, w["k.norm"], 1, 1e-5)
    assert np.allclose(kn[3, 1, 0], k_raw[3, 1, 0] / np.sqrt((k_raw[3, 1, 0] ** 2).mean() + 1e-5) * w["k.norm"])


def test_recurrent_unit_pieces():
    O = oracle()
    rng = np.random.default_rng(3)
    T, W = 7, 6
    u = rng.standard_normal((T, W))
    # convolution: last column = current token, zeros before the start
    wc = np.zeros((W, 3)); wc[:, 2] = 1.0
    assert np.allclose(O.causal_conv(u, wc, np.zeros(W)), u)
    wc = np.zeros((W, 3)); wc[:, 0] = 1.0
    c = O.causal_conv(u, wc, np.ones(W))
    assert np.allclose(c[:2], 1.0) and np.allclose(c[2:], u[:-2] + 1.0)
    # gates are block diagonal: a change in block 1's input leaves block 0's gates alone
    w = {"ra": rng.standard_normal((2, 3, 3)), "ra.b": rng.standard_normal((2, 3)), "ri": rng.standard_normal((2, 3, 3)), "ri.b": rng.standard_normal((2, 3))}
    r, i = O.rglru_gates(u, w, "", 2)
    u2 = u.copy(); u2[:, 3:] += 1.0
    r2, i2 = O.rglru_gates(u2, w, "", 2)
    assert np.allclose(r[:, :3], r2[:, :3]) and not np.allclose(r[:, 3:], r2[:, 3:]) and np.allclose(i[:, :3], i2[:, :3])
    assert np.allclose(r[2, :3], O.sigmoid(w["ra"][0] @ u[2, :3] + w["ra.b"][0]))
    # the scan: decay 1 keeps nothing new (sqrt(1 - a^2) = 0), decay ~0 passes i * u; the first token is no special case
    lam = np.full(W, -40.0)
    assert np.allclose(O.rglru_scan(u, r, i, lam), 0.0, atol=1e-6)
    lam = np.full(W, 40.0)
    big_r = np.ones((T, W))
    assert np.allclose(O.rglru_scan(u, big_r, i, lam), i * u)
    lam = rng.standard_normal(W)
    S = O.rglru_scan(u, r, i, lam)
    a0 = np.exp(-8.0 * r[0] * O.softplus(lam))
    assert np.allclose(S[0], np.sqrt(1 - a0 ** 2) * i[0] * u[0])
    a1 = np.exp(-8.0 * r[1] * O.softplus(lam))
    assert np.allclose(S[1], a1 * S[0] + np.sqrt(1 - a1 ** 2) * i[1] * u[1])


def test_state_space_pieces():
    O = oracle()
    rng = np.random.default_rng(4)
    T, H, P, N, G = 6, 4, 3, 5, 2
    x, B, C = rng.standard_normal((T, H, P)), rng.standard_normal((T, G, N)), rng.standard_normal((T, G, N))
    dt = O.softplus(rng.standard_normal((T, H)))
    A_log, D = rng.standard_normal(H), rng.standard_normal(H)
    y = O.ssd_scan(x, B, C, dt, A_log, D, G)
    # equal to the explicit sum over earlier tokens: y_t = sum_s exp(-exp(A) sum_{s<r<=t} dt_r) dt_s <C_t, B_s> x_s + D x_t
    for hd in (0, 3):
        g = hd // 2
        for t in range(T):
            acc = D[hd] * x[t, hd]
            for s in range(t + 1):
                acc = acc + math.exp(-math.exp(A_log[hd]) * dt[s + 1:t + 1, hd].sum()) * dt[s, hd] * (C[t, g] @ B[s, g]) * x[s, hd]
            assert np.allclose(y[t, hd], acc)
    # heads 0, 1 read group 0 and heads 2, 3 group 1
    B2 = B.copy(); B2[:, 1] += 1.0
    y2 = O.ssd_scan(x, B2, C, dt, A_log, D, G)
    assert np.allclose(y[:, :2], y2[:, :2]) and not np.allclose(y[:, 2:], y2[:, 2:])
    assert O.softplus(np.array([-800.0, 0.0, 800.0])) == pytest.approx([0.0, math.log(2.0), 800.0])


def test_router_and_experts():
    O = oracle()
    rng = np.random.default_rng(5)
    E, X, I = 10, 4, 2
    w = {"router": rng.standard_normal((X + I, E)), "correction": np.zeros(X + I)}
    x = rng.standard_normal((8, E))
    r = {"experts": X, "identity": I, "top": 3, "scale": 1.75}
    ids, wts = O.moe_route(x, w, "", r)
    z = x @ w["router"].T
    assert np.array_equal(ids, np.argsort(-z, axis=-1, kind="stable")[:, :3]) and np.allclose(wts.sum(-1), 1.75)   # renormalised over the chosen, times scale
    # the correction moves the CHOICE, the weights still come from the plain scores
    w2 = dict(w, correction=np.array([0, 0, 0, 0, 0, 5.0]))
    ids2, wts2 = O.moe_route(x, w2, "", r)
    assert np.all(ids2[:, 0] == 5)
    s = np.exp(z - z.max(-1, keepdims=True)); s /= s.sum(-1, keepdims=True)
    assert np.allclose(wts2, np.take_along_axis(s, ids2, -1) / np.take_along_axis(s, ids2, -1).sum(-1, keepdims=True) * 1.75)
    # identity experts return their input; with only identity experts chosen the mixture is scale * x
    for e in range(X):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = rng.standard_normal((6, E)), rng.standard_normal((6, E)), rng.standard_normal((E, 6))
    w3 = dict(w, correction=np.array([0, 0, 0, 0, 9.0, 9.0]))
    out = O.ff_moe(x, w3, "", {"router": dict(r, top=2), "expert": {"ff": 6}, "shared": None})
    assert np.allclose(out, 1.75 * x)
    # a shared expert is added for every token, times ONE sigmoid gate per token
    w3.update({"shared.gate": rng.standard_normal((5, E)), "shared.up": rng.standard_normal((5, E)), "shared.down": rng.standard_normal((E, 5)), "shared.sg": rng.standard_normal((1, E))})
    out2 = O.ff_moe(x, w3, "", {"router": dict(r, top=2), "expert": {"ff": 6}, "shared": {"ff": 5}})
    assert np.allclose(out2 - out, O.sigmoid(x @ w3["shared.sg"].T) * O.gated_expert(x, w3, "shared."))
    assert O.gelu_erf(np.array([0.0, 10.0, -10.0])) == pytest.approx([0.0, 10.0, 0.0], abs=1e-9) and O.gelu_erf(np.array([1.0]))[0] == pytest.approx(0.8413447460685429)
    assert abs(O.gelu_tanh(np.array([1.0]))[0] - 0.8413447460685429) > 1e-5          # the two GELUs differ


def test_whole_model_properties(pkg):
    """Causality of the whole stack, the depth average's reach, shared keys, and decisive routing for reduced precision."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["shared_keys"]
    w = w64(S.dinuzen_weights(cfg, 3))
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], 14).tolist()
    lg, tr = O.forward(cfg, w, toks, return_layers=True)
    lg2 = O.forward(cfg, w, toks[:9] + [(toks[9] + 1) % cfg["vocab"]] + toks[10:])
    assert np.allclose(lg[:9], lg2[:9]) and not np.allclose(lg[9], lg2[9])
    assert tr.shape == (5, 14, 48)
    # the last layer's depth average reads the embedding output: changing dwa[0] there moves the logits
    w2 = dict(w); w2["l4.dwa"] = w["l4.dwa"].copy(); w2["l4.dwa"][0] += 0.5
    assert rel_rms(O.forward(cfg, w2, toks)[-1], lg[-1]) > 1e-3
    # layer 2 reads layer 0's keys: changing layer 0's key projection moves layer 2's output even when layer 0's own output is muted
    w3 = dict(w); w3["l0.ls1"] = np.zeros_like(w["l0.ls1"]); w4 = dict(w3); w4["l0.mix.k"] = w["l0.mix.k"] * 1.5 + 0.1
    assert rel_rms(O.forward(cfg, w4, toks)[-1], O.forward(cfg, w3, toks)[-1]) > 1e-3
    wd = decisive_routing(cfg, S.dinuzen_weights(cfg, 3))
    assert min_margin(O, cfg, w64(wd), toks) > 0.01


@pytest.mark.parametrize("which", ["attention", "rglru", "ssd"])
def test_planted_models_have_teeth(pkg, which):
    """Removing the planted token changes the row it decides by far more than any tolerance of the GPU tests."""
    S, O = pkg.synth, oracle()
    cfg, w, A, B, fill = {"attention": needle_attention, "rglru": needle_rglru, "ssd": needle_ssd}[which](S)
    rng = np.random.default_rng(2)
    f = [int(fill[i]) for i in rng.integers(0, len(fill), 300)]
    for back in (1, 7, 299):
        seq = f[:300 - back] + [B] + f[300 - back:299] + [A]
        without = f[:300 - back] + [f[0]] + f[300 - back:299] + [A]
        assert len(seq) == 301
        a, b = O.forward(cfg, w64(w), seq)[-1], O.forward(cfg, w64(w), without)[-1]
        assert rel_rms(a, b) > 0.2, (which, back)
