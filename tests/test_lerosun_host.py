"""CPU tests of the Lerosun support code: config.json registry and the C-ABI structures, synthetic model directories, and
properties of the float64 oracle the GPU tests compare against (each mechanism on its own, and the identity the product path
rests on: mixing the scores over the heads equals attending with a query into which the mixing was folded)."""
import math

import numpy as np
import pytest

from lerosun_util import configs, needle_attention, needle_delta, oracle, rel_rms, w64


def test_config_registry_and_abi_structs(pkg, tmp_path):
    S = pkg.synth
    cfg = configs(S)["loop_mid"]
    w = S.lerosun_weights(cfg, 0)
    d = str(tmp_path / "m")
    S.write_model_dir(d, cfg, w)
    m = pkg.load_model(d, 77)
    c = m.configuration
    assert m.model_type == "LEROSUN" and c.arch == pkg.loader.ARCH_LEROSUN and c.context_length == 77
    assert (c.width, c.vocab_size, c.n_layers, c.block, c.loop, c.norm_eps, c.embedding_scale) == (48, 80, 5, "prenorm", (1, 4, 3), 1e-6, 1.0)
    assert c.layer_runs() == 11
    l0, l1, l2, l4 = c.layers[0], c.layers[1], c.layers[2], c.layers[4]
    assert (l0.mixer, l0.heads, l0.kv_heads, l0.key_dim, l0.value_dim, l0.conv_taps, l0.ff_dim, l0.ff_act) == ("gated_delta", 2, 1, 8, 24, 4, 40, "relu")
    assert (l1.mixer, l1.heads, l1.kv_heads, l1.key_dim, l1.value_dim, l1.window, l1.rope_dims, l1.ff_dim) == ("window_attention", 3, 3, 10, 10, 9, 10, 0)
    assert (l1.sink, l1.sink_learned, l1.gate, l1.gate_per_head, l1.value_from_key, l1.head_temp, l1.head_mix, l1.qkv_bias, l1.qk_norm) == (True,) * 8 + (False,)
    assert (l2.rope_dims, l2.rope_base, l2.rope_layout, l2.score_scale) == (4, 50.0, "half", pytest.approx(12 ** -0.5))
    assert l4.rope_dims == 0
    tt, dims, raw = m.tensors["l0.norm1"]
    assert tt == pkg.loader.GGML_BF16 and dims == () and raw.nbytes == 2   # a norm weight is ONE number
    assert m.tensors["l0.mix.q.conv"][1] == (4, 8) and m.tensors["l1.mix.talk"][1] == (3, 3) and m.tensors["l1.mix.g"][1] == (48, 3)
    lc, specs = pkg.plan.make_layered_config(m, "float32")
    assert (lc.arch, lc.block, lc.compute, lc.loop_start, lc.loop_stop, lc.loop_times) == (5, 2, 1, 1, 4, 3)
    assert (specs[0].mixer, specs[0].conv_taps, specs[0].ff_kind, specs[0].ff_act) == (3, 4, 1, 2)
    assert (specs[1].mixer, specs[1].sink, specs[1].gate, specs[1].value_from_key, specs[1].head_temp, specs[1].head_mix, specs[1].rope_dims, specs[1].ff_kind) == (1, 2, 2, 1, 1, 1, 10, 0)
    # in-memory model = on-disk model
    mm = S.lerosun_model(cfg, w, 77)
    assert mm.configuration == c and all(np.array_equal(mm.tensors[k][2], m.tensors[k][2]) for k in m.tensors)
    # no loop; unknown mixer / feed-forward kinds are refused
    c2 = dict(cfg)
    del c2["loop"]
    assert pkg.loader.lerosun_configuration(c2, {}, 8).loop is None
    with pytest.raises(pkg.loader.UnsupportedModel):
        pkg.loader.lerosun_configuration(dict(cfg, layers=[dict(cfg["layers"][0], type="latent_attention")]), {}, 8)
    with pytest.raises(pkg.loader.UnsupportedModel):
        pkg.loader.lerosun_configuration(dict(cfg, layers=[dict(cfg["layers"][0], mlp={"kind": "moe"})]), {}, 8)
    # the earlier designs keep their own flags
    p = pkg.loader.pibidra_configuration(S.pibidra_config(32, 40, [S.pibidra_layer(2, 1, 8, 8, 4, 16)]), {"l0.mix.rel": (8, 2)}, 8)
    assert not (p.layers[0].sink_learned or p.layers[0].gate_per_head or p.layers[0].value_from_key or p.layers[0].head_mix) and p.block == "sandwich"


def test_scalar_norm_and_activations():
    O = oracle()
    rng = np.random.default_rng(1)
    v = rng.standard_normal((3, 10)) + 2.0
    y = O.scalar_rms_norm(v, 1.0, 0.0)
    assert np.allclose((y * y).mean(-1), 1.0) and np.allclose(O.scalar_rms_norm(v, -2.5, 0.0), -2.5 * y)
    assert np.all(np.abs(O.scalar_rms_norm(v * 1e-6, 1.0, 1e-2)) < 1e-4)       # eps sits inside the root
    assert O.softplus(np.array([-800.0, 0.0, 800.0])) == pytest.approx([0.0, math.log(2.0), 800.0])
    assert O.silu(np.array([0.0, 30.0, -30.0])) == pytest.approx([0.0, 30.0, 0.0], abs=1e-10)


def test_partial_rotation():
    O = oracle()
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 2 * 12)), rng.standard_normal((1, 2 * 12))
    # a score between two rotated heads depends on the distance only; entries from `dims` on pass unchanged; position 0 is the identity
    for dims, base in ((8, 50.0), (12, 3.0), (2, 1e4), (0, 10.0)):
        s = [(O.rotate_half_partial(q, 2, 12, dims, base, i) @ O.rotate_half_partial(k, 2, 12, dims, base, j).T).item() for i, j in ((7, 3), (104, 100), (4, 0))]
        assert s[0] == pytest.approx(s[1]) == pytest.approx(s[2])
        r = O.rotate_half_partial(q, 2, 12, dims, base, 9).reshape(2, 12)
        assert np.array_equal(r[:, dims:], q.reshape(2, 12)[:, dims:])
        assert np.array_equal(O.rotate_half_partial(q, 2, 12, dims, base, 0), q)
    # entry i turns with entry i + dims/2 (not with i + 1): a vector with only entry 0 set moves into entry dims/2
    e0 = np.zeros((1, 12)); e0[0, 0] = 1.0
    r = O.rotate_half_partial(e0, 1, 12, 8, 1.0, 1)[0]    # base 1: every pair turns by one radian per position
    assert r[0] == pytest.approx(math.cos(1.0)) and r[4] == pytest.approx(math.sin(1.0)) and abs(r[1]) < 1e-15
    # frequencies fall with the pair index: base^(-2i / dims)
    e1 = np.zeros((1, 12)); e1[0, 1] = 1.0
    r = O.rotate_half_partial(e1, 1, 12, 8, 16.0, 1)[0]
    assert r[1] == pytest.approx(math.cos(16.0 ** -0.25)) and r[5] == pytest.approx(math.sin(16.0 ** -0.25))


def test_mixed_scores_equal_a_folded_query():
    """score'_h = sum_m T[h, m] t_m c <q^m, k^g(m)> = <q'^h, [k^0 | k^1 | ...]> with q'^h = [sum_{m in group g} T[h, m] t_m c q^m]_g: the
    form the attention kernels run (one query of key heads x key size entries per head, one key row for all heads)."""
    O = oracle()
    rng = np.random.default_rng(2)
    H, G, d, n = 6, 3, 5, 9
    q, k = rng.standard_normal(H * d), rng.standard_normal((n, G * d))
    temp, talk, c = rng.standard_normal(H), rng.standard_normal((H, H)), 0.37
    e = O.mixed_head_scores(q, k, H, G, d, c, temp, talk)
    group = H // G
    for h in range(H):
        folded = np.concatenate([sum(talk[h, m] * temp[m] * c * q[m * d:(m + 1) * d] for m in range(g * group, (g + 1) * group)) for g in range(G)])
        assert np.allclose(k @ folded, e[h])
    # the identity matrix and unit temperatures leave plain grouped attention scores
    e1 = O.mixed_head_scores(q, k, H, G, d, c, np.ones(H), np.eye(H))
    assert np.allclose(e1[4], k[:, 2 * d:3 * d] @ q[4 * d:5 * d] * c)


def test_sink_softmax_and_window():
    O = oracle()
    e = np.array([0.3, -1.0, 2.0])
    p = O.sink_softmax(e, 0.5)
    assert p.sum() == pytest.approx(1.0 - math.exp(0.5) / (math.exp(0.5) + np.exp(e).sum()))
    assert O.sink_softmax(e, -800.0).sum() == pytest.approx(1.0) and O.sink_softmax(e, 800.0).sum() == pytest.approx(0.0)
    assert O.sink_softmax(e + 700.0, 700.5) == pytest.approx(p)               # stable for large logits
    # a row sees itself and window - 1 rows before it; values ride with their key/value head
    rng = np.random.default_rng(3)
    T, H, G, d = 12, 4, 2, 3
    q, k, v = rng.standard_normal((T, H * d)), rng.standard_normal((T, G * d)), rng.standard_normal((T, G * d))
    kw = dict(heads=H, kv_heads=G, d=d, dv=d, scale=0.5, temp=np.ones(H), talk=np.eye(H), sink=np.full(H, -800.0))
    o = O.window_attention(q, k, v, window=4, **kw)
    k2, v2 = k.copy(), v.copy()
    k2[:6], v2[:6] = rng.standard_normal((6, G * d)), rng.standard_normal((6, G * d))  # rows 0..5 are outside the window of rows 9..
    o2 = O.window_attention(q, k2, v2, window=4, **kw)
    assert np.allclose(o[9:], o2[9:]) and not np.allclose(o[8], o2[8])
    assert np.allclose(O.window_attention(q, k, v, window=1, **kw), np.repeat(v.reshape(T, G, d), 2, axis=1).reshape(T, H * d))


def test_causal_convolution_and_unit_heads():
    O = oracle()
    u = np.arange(1.0, 11.0).reshape(5, 2)
    w = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = O.causal_conv(u, w)
    assert np.array_equal(y[:, 1], u[:, 1])                                   # the last column is the current token's tap
    assert y[0, 0] == 100.0 * u[0, 0] and y[1, 0] == 10.0 * u[0, 0] + 100.0 * u[1, 0] and y[4, 0] == u[2, 0] + 10.0 * u[3, 0] + 100.0 * u[4, 0]
    x = np.array([[3.0, 4.0, 0.0, 0.0]])
    n = O.unit_heads(x, 2, 2)
    assert n[0, :2] == pytest.approx([0.6, 0.8], rel=1e-6) and np.all(n[0, 2:] == 0.0)  # a zero head stays zero: the constant sits inside the root


def test_gated_delta_rule_properties():
    O = oracle()
    rng = np.random.default_rng(4)
    T, H, G, d, dv = 7, 2, 1, 4, 3
    q, k = O.unit_heads(rng.standard_normal((T, G * d)), G, d), O.unit_heads(rng.standard_normal((T, G * d)), G, d)
    v = rng.standard_normal((T, H * dv))
    one, zero = np.ones((T, H)), np.zeros((T, H))
    kw = dict(heads=H, kv_heads=G, d=d, dv=dv)
    # beta = 1, no decay, read with the key just written: the value comes back (the write replaces what the key held)
    assert np.allclose(O.gated_delta_rule(k, k, v, one, one, **kw), v, atol=1e-5)
    # beta = 0: nothing is ever written
    assert np.all(O.gated_delta_rule(q, k, v, zero, one, **kw) == 0.0)
    # decay 0: only the current token's write is read
    o = O.gated_delta_rule(q, k, v, 0.7 * one, zero, **kw)
    assert np.allclose(o[:, :dv], 0.7 * (q * k).sum(-1, keepdims=True) * v[:, :dv])
    # without decay and with orthogonal keys the state is a plain sum of outer products
    kk = np.eye(4)[[0, 1, 2, 3, 0, 1, 2]]
    o = O.gated_delta_rule(kk, kk, v, one, one, **kw)
    assert np.allclose(o[4], v[4]) and np.allclose(o[3], v[3])
    # causality: a later token changes nothing earlier
    v2 = v.copy(); v2[5] += 1.0
    g = 0.9 * one
    assert np.allclose(O.gated_delta_rule(q, k, v, 0.5 * one, g, **kw)[:5], O.gated_delta_rule(q, k, v2, 0.5 * one, g, **kw)[:5])


def test_loop_order_and_planted_models():
    O = oracle()
    assert O.layer_runs({"layers": [0] * 5, "loop": {"start": 1, "stop": 4, "times": 2}}) == [0, 1, 2, 3, 1, 2, 3, 4]
    assert O.layer_runs({"layers": [0] * 3}) == [0, 1, 2] and O.layer_runs({"layers": [0] * 2, "loop": {"start": 0, "stop": 2, "times": 3}}) == [0, 1] * 3

    import __graft_entry__ as ge
    S = ge.import_package().synth
    cfg, w, A, B, fill = needle_attention(S, 12, kv_heads=2)

    def row(dist):
        toks = [fill[(5 * t + 1) % len(fill)] for t in range(41)]
        toks[40], toks[40 - dist] = A, B
        return O.forward(cfg, w64(w), toks)[40]
    assert rel_rms(row(11), row(12)) > 0.1 and rel_rms(row(12), row(13)) < 1e-9
    cfg, w, A, B, fill = needle_delta(S)
    toks = [fill[(7 * t + 3) % len(fill)] for t in range(200)]
    toks[-1] = A
    t2 = list(toks); t2[1] = B
    assert rel_rms(O.forward(cfg, w64(w), t2)[-1], O.forward(cfg, w64(w), toks)[-1]) > 0.1
