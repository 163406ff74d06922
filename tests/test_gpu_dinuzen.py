"""GPU tests of the output-normed layered plans (csrc/recurrent.cuh, csrc/outnorm_plan.cuh and the kernels they share with the other
layered designs) on small random Dinuzen models, against the float64 oracle (oracle/dinuzen_oracle.py, which shares no code with
the product).

Tolerances.  FP32 compute mode and the decode step (FP32 activations in either mode): relative RMS error of a logits row
<= 5e-5 (only the summation order differs): this is the sharp comparison, and every case runs in it.  BF16 compute mode, batched
prefill: GEMM operands are rounded to BF16 and the untrained random layers pass the rounding of every layer on to the next, so the
bound grows with depth: 1.2 % per layer (+ 1 for the classifier).  In BF16 mode the routers never face a close call (see
dinuzen_util.decisive_routing): a flipped expert is a different function, not a rounding error.  Where a test plants a key or a
write that decides the output, the model has one layer (bound 2.4 %) and a slip of the cache or the state moves the row by more
than 10 %."""
import numpy as np
import pytest

from dinuzen_util import bf16_values, configs, decisive_routing, min_margin, needle_attention, needle_rglru, needle_ssd, oracle, rel_rms, w64

pytestmark = pytest.mark.gpu

TOL_DECODE = 5e-5
ALL = ["trio", "shared_keys", "odd", "recurrent_only", "attention_only", "tiles_a", "tiles_b"]


class _Tol:
    """TOL[compute] for one-layer models; TOL(compute, cfg) scales the BF16 bound with the number of layers."""

    def __getitem__(self, compute):
        return {"float32": 5e-5, "bfloat16": 2.4e-2}[compute]

    def __call__(self, compute, cfg):
        return 5e-5 if compute == "float32" else 1.2e-2 * (len(cfg["layers"]) + 1)


TOL = _Tol()


def weights_for(S, O, cfg, seed, compute, toks):
    """Random weights; in BF16 mode with decisive routers.  In FP32 mode the seed must not produce a near-tie of two experts."""
    w = S.dinuzen_weights(cfg, seed)
    if compute == "bfloat16":
        w = decisive_routing(cfg, w, seed)
        assert min_margin(O, cfg, w64(w), toks) > 1e-3  # several times what BF16 rounding moves a choice score
    else:
        assert min_margin(O, cfg, w64(w), toks) > 2e-5, "near-tie of two experts in the oracle: pick another seed"
    return w


def make_plan(pkg, cfg, weights, ctx=256, batch=16, compute="float32"):
    model = pkg.synth.dinuzen_model(cfg, weights, ctx)
    return pkg.B200MasterPlan.initialize_plan(model, prefill_batch_size=batch, compute=compute)


def prefill_all(plan, toks, batch, start=0):
    rows = []
    for c0 in range(0, len(toks), batch):
        part = toks[c0:c0 + batch]
        lg, _ = plan.forward_batch_logits(part, start + c0, list(range(len(part))))
        rows.append(lg)
    return np.concatenate(rows)


def assert_rows(got, ref, tol, what=""):
    errs = [rel_rms(got[i], ref[i]) for i in range(len(ref))]
    worst = int(np.argmax(errs))
    assert errs[worst] <= tol, f"{what}: relative RMS error {errs[worst]:.3g} > {tol} at row {worst}"


def portions(plan, toks, sizes, batch):
    """The prompt in portions of the given sizes (each cut again at the chunk capacity; a portion of one token is a decode step),
    the rest decoded one by one."""
    got, p = [], 0
    for m in sizes:
        if m == 1:
            got.append(plan.forward_decode(toks[p], p)[0][None])
        else:
            got.append(prefill_all(plan, toks[p:p + m], batch, start=p))
        p += m
    while p < len(toks):
        got.append(plan.forward_decode(toks[p], p)[0][None])
        p += 1
    return np.concatenate(got)


@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ALL)
def test_every_layer_matches_oracle(pkg, name, compute):
    """Residual stream after every layer (as the next layer reads it) and the logits: each mixer alone (recurrent_only,
    attention_only) and in every order, with and without feed-forwards, shared keys, identity and shared experts."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    toks = np.random.default_rng(5).integers(0, cfg["vocab"], 23).tolist()
    w = weights_for(S, O, cfg, 11, compute, toks)
    ref_lg, ref_tr = O.forward(cfg, w64(w), toks, return_layers=True)
    plan = make_plan(pkg, cfg, w, batch=32, compute=compute)
    try:
        assert plan.layered_info()[0] == len(ref_tr)
        lg, tr = plan.forward_batch_logits(toks, 0, list(range(len(toks))), want_trace=True)
        for r in range(len(ref_tr)):
            assert rel_rms(tr[r], ref_tr[r]) <= TOL(compute, cfg), f"layer {r}"
        assert_rows(lg, ref_lg, TOL(compute, cfg), "logits")
    finally:
        plan.free()


@pytest.mark.parametrize("name", ALL)
def test_prefill_equals_token_by_token_decode(pkg, name):
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    toks = np.random.default_rng(6).integers(0, cfg["vocab"], 40).tolist()
    for compute in ("float32", "bfloat16"):
        w = weights_for(S, O, cfg, 12, compute, toks)
        ref = O.forward(cfg, w64(w), toks)
        plan = make_plan(pkg, cfg, w, batch=64, compute=compute)
        try:
            whole = prefill_all(plan, toks, 64)
            step = np.stack([plan.forward_decode(t, p)[0] for p, t in enumerate(toks)])  # position 0 starts from an empty state without a reset
            assert_rows(step, ref, TOL_DECODE, "decode")
            assert_rows(whole, ref, TOL(compute, cfg), "prefill")
        finally:
            plan.free()


@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["trio", "shared_keys", "odd", "recurrent_only"])
def test_portions_of_every_size(pkg, name, compute):
    """The same prompt cut into portions of 1 .. 13 tokens (edges inside the convolutions' taps, the shifted row across every edge),
    then decoded one by one; the chunk capacity (7) is below the portion sizes, so portions are cut again."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    toks = np.random.default_rng(7).integers(0, cfg["vocab"], 70).tolist()
    w = weights_for(S, O, cfg, 13, compute, toks)
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, ctx=70, batch=7, compute=compute)  # the last token fills the context
    try:
        for sizes in ([2, 3, 2, 13, 5, 2, 11, 2, 7], [9, 2, 1, 2, 2, 12, 1, 1, 3], [50], [2] * 20, [1, 2, 1, 60]):
            assert_rows(portions(plan, toks, sizes, 7), ref, TOL(compute, cfg), f"portions {sizes}")
    finally:
        plan.free()


@pytest.mark.parametrize("name", ["tiles_a", "tiles_b"])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_tensor_core_prefill_shapes(pkg, name, compute):
    """Shapes that take the tcgen05 GEMMs and the tensor-core attention in BF16 mode: a prompt longer than several key tiles and
    several scan groups, whole and in ragged portions (one of them a single row), then decoded."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    toks = np.random.default_rng(12).integers(0, cfg["vocab"], 230).tolist()
    w = weights_for(S, O, cfg, 21, compute, toks)
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, ctx=256, batch=100, compute=compute)
    try:
        assert_rows(prefill_all(plan, toks, 100), ref, TOL(compute, cfg), "whole")
        assert_rows(portions(plan, toks, (65, 2, 100, 1, 37), 100), ref, TOL(compute, cfg), "portions")
    finally:
        plan.free()


def test_state_and_slots_are_reused_across_requests(pkg):
    """Request after request on one plan without clearing anything: a request starts from empty recurrent states, empty
    convolution rings, an empty shifted row and empty key rings whatever the previous one left; kv_reset in between changes nothing."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["trio"]
    rng = np.random.default_rng(8)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (30, 3, 41, 1, 17, 2)]
    w = weights_for(S, O, cfg, 14, "float32", sum(seqs, []))
    plan = make_plan(pkg, cfg, w, ctx=48, batch=4, compute="float32")
    try:
        for k, toks in enumerate(seqs):
            n = len(toks)
            ref = O.forward(cfg, w64(w), toks)
            cut = n // 2
            got = [prefill_all(plan, toks[:cut], 4)] if cut else []
            got += [plan.forward_decode(toks[p], p)[0][None] for p in range(cut, n)]
            assert_rows(np.concatenate(got), ref, TOL["float32"], f"request of {n}")
            assert np.abs(plan.read_buffer("delta_state", 32, layer=1)).max() > 0
            if k == 2:
                plan.kv_reset()
                assert np.abs(plan.read_buffer("delta_state", 32, layer=1)).max() == 0
    finally:
        plan.free()


@pytest.mark.parametrize("kv_heads", [1, 2])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_a_far_key_and_the_first_tokens(pkg, compute, kv_heads):
    """One key decides the output.  It sits at the first positions of the sequence, right before the query, at the query itself,
    hundreds of tokens back (several key tiles; the decode step splits the keys over CTAs), on both sides of a chunk edge and in
    the last slot of the context -- in a prompt, with the query decoded after a prefill, and with everything decoded."""
    S, O = pkg.synth, oracle()
    cfg, w, A, B, fill = needle_attention(S, kv_heads=kv_heads)
    wd = w64(w)
    ctx, batch = 400, 128
    plan = make_plan(pkg, cfg, w, ctx=ctx, batch=batch, compute=compute)
    try:
        for i, at in [(399, 0), (399, 1), (399, 127), (399, 128), (399, 398), (399, 399), (330, 40), (129, 2), (128, 127), (5, 0), (1, 0), (0, 0)]:
            toks = [fill[(7 * t + 3) % len(fill)] for t in range(i + 1)]
            toks[i] = A
            if at != i:
                toks[at] = B
            ref = O.forward(cfg, wd, toks)[i]
            without = list(toks)
            if at != i:
                without[at] = fill[0]
                assert rel_rms(O.forward(cfg, wd, without)[i], ref) > 0.1, "the planted key has teeth"
            assert rel_rms(prefill_all(plan, toks, batch)[i], ref) <= TOL[compute], f"prompt, query {i}, key at {at}"
            if i:
                prefill_all(plan, toks[:i], batch)
            assert rel_rms(plan.forward_decode(toks[i], i)[0], ref) <= TOL[compute], f"decoded query {i}, key at {at}"  # the keys came from the prefill kernels
            if i <= 330:
                ids, _ = plan.decode_sequence(toks, i + 1, 0, feedback=False)
                assert rel_rms(plan.read_buffer("logits", cfg["vocab"]), ref) <= TOL_DECODE, f"all decoded, query {i}, key at {at}"
    finally:
        plan.free()


@pytest.mark.parametrize("which", ["rglru", "ssd"])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_the_state_keeps_a_far_write(pkg, compute, which):
    """Recurrent layers with decays near one: what token B wrote up to 419 tokens back decides the read-out at token A -- whole,
    across chunk edges and scan groups, with the last tokens decoded, and all decoded; without B the row is a different one."""
    S, O = pkg.synth, oracle()
    cfg, w, A, B, fill = (needle_rglru if which == "rglru" else needle_ssd)(S)
    wd = w64(w)
    plan = make_plan(pkg, cfg, w, ctx=512, batch=64, compute=compute)
    try:
        n = 420
        toks = [fill[(7 * t + 3) % len(fill)] for t in range(n)]
        toks[n - 1] = A
        without = O.forward(cfg, wd, toks)[n - 1]
        for at in (0, 1, 19, 63, 64, n - 2):
            t2 = list(toks)
            t2[at] = B
            ref = O.forward(cfg, wd, t2)[n - 1]
            assert rel_rms(ref, without) > 0.1, "the planted write has teeth"
            assert rel_rms(prefill_all(plan, t2, 64)[n - 1], ref) <= TOL[compute], f"prompt, write at {at}"
            assert rel_rms(portions(plan, t2, [3, 64, 2, 300], 64)[n - 1], ref) <= TOL[compute], f"portions, write at {at}"
        ids, _ = plan.decode_sequence(t2, n, 0, feedback=False)
        assert rel_rms(plan.read_buffer("logits", cfg["vocab"]), ref) <= 4 * TOL_DECODE  # 420 steps of a state that forgets nothing
    finally:
        plan.free()


def _check_f32(pkg, cfg, w, toks, what, sizes=(1, 2, 3, 2)):
    S, O = pkg.synth, oracle()
    ref_lg, ref_tr = O.forward(cfg, w64(w), toks, return_layers=True)
    plan = make_plan(pkg, cfg, w, batch=64, compute="float32")
    try:
        lg, tr = plan.forward_batch_logits(toks, 0, list(range(len(toks))), want_trace=True)
        assert rel_rms(tr[0][:5], ref_tr[0][:5]) <= TOL["float32"], what + ": first tokens"
        for r in range(len(ref_tr)):
            assert rel_rms(tr[r], ref_tr[r]) <= TOL["float32"], f"{what}: layer {r}"
        assert_rows(lg, ref_lg, TOL["float32"], what)
        assert_rows(portions(plan, toks, list(sizes), 64), ref_lg, TOL["float32"], what + " (portions, decode)")
    finally:
        plan.free()
    return ref_lg, ref_tr


def test_each_block_mechanism_alone(pkg):
    """Weights that isolate one mechanism of the block each (FP32, prefill and decode): a shift of exactly one (the mixer reads the
    previous token only) and of zero; a depth average that returns the embedding output, or mixes all earlier results with weights
    far from (0, .., 0, 1); layer scales that mute one sublayer; norm groups of four entries each."""
    S, O = pkg.synth, oracle()
    rng = np.random.default_rng(9)
    toks = rng.integers(0, 60, 33).tolist()
    A, R, M, D = S.dinuzen_attention, S.dinuzen_rglru, S.dinuzen_mamba2, S.dinuzen_dense
    for case in ("shift_one", "shift_zero", "dwa_first", "dwa_wide", "mute_mixer", "mute_ff", "groups_many"):
        cfg = S.dinuzen_config(40, 60, [A(4, 2, 8, 6, D(24), rot_dims=4), R(16, 2, 3, D(20)), M(2, 8, 6, 1, 2, D(16))], groups=10 if case == "groups_many" else 5)
        w = S.dinuzen_weights(cfg, 15)
        for i in range(3):
            if case == "shift_one":
                w[f"l{i}.shift"][:] = 1.0
            if case == "shift_zero":
                w[f"l{i}.shift"][:] = 0.0
            if case == "dwa_wide":
                w[f"l{i}.dwa"] = rng.standard_normal(i + 2).astype(np.float32)
            if case == "mute_mixer":
                w[f"l{i}.ls1"][:] = 0.0
            if case == "mute_ff":
                w[f"l{i}.ls2"][:] = 0.0
        if case == "dwa_first":
            w["l2.dwa"] = np.array([1.0, 0.0, 0.0, 0.0], dtype=np.float32)
        w = bf16_values(w)
        ref_lg, ref_tr = _check_f32(pkg, cfg, w, toks, case)
        if case == "dwa_first":
            assert rel_rms(ref_tr[2], w64(w)["embed"][np.asarray(toks)]) < 1e-12


def test_wide_rows(pkg):
    """A residual row and a state-space read-out of 2048 entries: the single-row launches of the decode step run with more threads
    per row than the chunk's."""
    S = pkg.synth
    mlp = S.dinuzen_moe(2, 1, 16, identity=1, scale=1.5, shared=16)
    cfg = S.dinuzen_config(2048, 64, [S.dinuzen_mamba2(4, 512, 4, 1, 2, mlp, norm_groups=4), S.dinuzen_rglru(32, 2, 2, None)], groups=8)
    toks = np.random.default_rng(3).integers(0, 64, 12).tolist()
    w = S.dinuzen_weights(cfg, 31)
    assert min_margin(oracle(), cfg, w64(w), toks) > 2e-5
    _check_f32(pkg, cfg, w, toks, "wide", sizes=(3, 1, 2))


def test_each_attention_mechanism_alone(pkg):
    """The same for the differential attention: a lambda far from its start value (large lq / lk), diff near one and zero, a cap
    that binds (scores far above it) and no cap, q / k norm weights of both signs, rotation over the whole slice with a small base,
    over two entries, none; frequency blending whose ramp starts and ends inside the slice; one key/value head for all query heads."""
    S, O = pkg.synth, oracle()
    rng = np.random.default_rng(10)
    toks = rng.integers(0, 60, 50).tolist()
    A = S.dinuzen_attention
    cases = {
        "lambda": A(4, 2, 8, 6, None, rot_dims=4), "diff_high": A(4, 2, 8, 6, None, rot_dims=4, diff=0.95), "diff_zero": A(4, 2, 8, 6, None, rot_dims=4, diff=0.0),
        "cap_binds": A(4, 2, 8, 6, None, rot_dims=4, scale=4.0, softcap=2.0), "no_cap": A(4, 2, 8, 6, None, rot_dims=4, scale=1.0, softcap=0.0),
        "norm_signs": A(4, 4, 8, 6, None, rot_dims=8), "rot_full": A(4, 2, 8, 6, None, rot_dims=8, base=3.0), "rot_two": A(4, 2, 9, 6, None, rot_dims=2),
        "rot_none": A(4, 2, 8, 6, None, rot_dims=0), "blend": A(2, 1, 24, 6, None, rot_dims=20, base=100.0, scaling=(8.0, 40, 4.0, 0.5)),
        "blend_all": A(2, 1, 12, 6, None, rot_dims=12, base=100.0, scaling=(3.0, 4, 64.0, 32.0)), "one_kv": A(6, 1, 8, 5, None, rot_dims=6)}
    for case, layer in cases.items():
        cfg = S.dinuzen_config(40, 60, [layer], groups=2)
        w = S.dinuzen_weights(cfg, 16)
        if case == "lambda":
            w["l0.mix.lq1"][:] = 0.5
            w["l0.mix.lk1"][:] = 0.5
        if case == "norm_signs":
            w["l0.mix.q.norm"][::2] *= -3.0
            w["l0.mix.k.norm"][1::3] *= -0.2
        _check_f32(pkg, cfg, bf16_values(w), toks, case)


def test_each_recurrent_mechanism_alone(pkg):
    """The same for the recurrent mixers: decays near zero (the state forgets at once) and near one; gates driven to zero or one
    token by token; a convolution that only looks back (current tap zero), with one tap, with more taps than the first portions have
    tokens; one block and as many blocks as channels; state sizes of 1, 16, 17 and 100 rows; D = 0; norm groups of the read-out."""
    S, O = pkg.synth, oracle()
    rng = np.random.default_rng(12)
    toks = rng.integers(0, 60, 37).tolist()
    R, M = S.dinuzen_rglru, S.dinuzen_mamba2
    cases = {
        "r_forget": R(24, 3, 3), "r_keep": R(24, 3, 3), "r_gates": R(24, 3, 3), "r_look_back": R(24, 2, 4), "r_one_tap": R(24, 2, 1), "r_long_taps": R(20, 1, 7),
        "r_blocks_all": R(12, 12, 2), "m_forget": M(3, 5, 8, 1, 3), "m_keep": M(3, 5, 8, 1, 3), "m_look_back": M(2, 6, 4, 2, 4), "m_state_1": M(2, 6, 1, 1, 2),
        "m_state_17": M(4, 3, 17, 2, 2, norm_groups=3), "m_state_100": M(2, 20, 100, 1, 6, norm_groups=5), "m_no_skip": M(3, 5, 16, 3, 1)}
    for case, layer in cases.items():
        cfg = S.dinuzen_config(40, 60, [layer], groups=4)
        w = S.dinuzen_weights(cfg, 17)
        if case == "r_forget":
            w["l0.mix.lam"][:] = 6.0
        if case == "r_keep":
            w["l0.mix.lam"][:] = -12.0
        if case == "r_gates":
            w["l0.mix.ra"] *= 30.0
            w["l0.mix.ri"] *= 30.0
        if case in ("r_look_back", "m_look_back"):
            w["l0.mix.conv"][:, -1] = 0.0
        if case == "m_forget":
            w["l0.mix.A_log"][:] = 3.0
            w["l0.mix.dt_bias"][:] = 2.0
        if case == "m_keep":
            w["l0.mix.A_log"][:] = -12.0
        if case == "m_no_skip":
            w["l0.mix.D"][:] = 0.0
        _check_f32(pkg, cfg, bf16_values(w), toks, case)


def test_each_expert_mechanism_alone(pkg):
    """The same for the mixture of experts: corrections that decide the choice against the scores (the weights still come from the
    scores); only identity experts; identity experts that are never / always among the chosen; all experts chosen; one expert; a
    scale far from one; a shared expert whose gate is closed, open, or decided by the token; no shared expert."""
    S, O = pkg.synth, oracle()
    rng = np.random.default_rng(14)
    toks = rng.integers(0, 60, 41).tolist()
    X = S.dinuzen_moe
    cases = {
        "correction": X(6, 2, 12, identity=1, scale=1.0, shared=None), "identity_only": X(0, 2, 12, identity=3, scale=1.3, shared=16), "identity_never": X(4, 2, 12, identity=2, shared=None),
        "identity_always": X(4, 3, 12, identity=2, scale=0.5, shared=None), "all_chosen": X(3, 5, 12, identity=2, scale=2.0, shared=8), "one_expert": X(1, 1, 12, identity=0, scale=3.0, shared=None),
        "gate_closed": X(3, 1, 12, identity=0, shared=20), "gate_open": X(3, 1, 12, identity=0, shared=20), "gate_token": X(3, 2, 12, identity=1, shared=20)}
    for case, mlp in cases.items():
        cfg = S.dinuzen_config(40, 60, [S.dinuzen_rglru(16, 2, 2, mlp)], groups=2)
        w = S.dinuzen_weights(cfg, 18)
        n = mlp["router"]["experts"] + mlp["router"]["identity"]
        if case == "correction":
            w["l0.mlp.correction"] = (np.arange(n)[::-1] * 2.0).astype(np.float32)   # experts 0 and 1 always, whatever the scores
        if case == "identity_never":
            w["l0.mlp.correction"][-2:] = -5.0
        if case == "identity_always":
            w["l0.mlp.correction"][-2:] = 5.0
        if case == "gate_closed":
            w["l0.mlp.shared.sg"][:] = 0.0
            w["l0.mlp.shared.sg"][0, 0], w["embed"][:, 0] = -40.0, 1.0
        if case == "gate_open":
            w["l0.mlp.shared.sg"][:] = 0.0
            w["l0.mlp.shared.sg"][0, 0], w["embed"][:, 0] = 40.0, 1.0
            w["l0.ls1"][0] = 0.0
        if case == "gate_token":
            w["l0.mlp.shared.sg"] *= 6.0
        w = bf16_values(w)
        assert min_margin(O, cfg, w64(w), toks) > 2e-5, case
        _check_f32(pkg, cfg, w, toks, case)


def test_long_decoding_through_the_device_loop(pkg):
    """300 single-token steps in one call of the device-resident loop (teacher-forced): the argmax of every step equals the
    oracle's wherever the oracle's best two logits are not a near-tie, and the last logits agree."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["shared_keys"]
    toks = np.random.default_rng(10).integers(0, cfg["vocab"], 300).tolist()
    w = decisive_routing(cfg, S.dinuzen_weights(cfg, 16), 16)
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, ctx=320, batch=1, compute="bfloat16")
    try:
        ids, ms = plan.decode_sequence(toks, len(toks), 0, feedback=False)
        srt = np.sort(ref, axis=1)
        clear = (srt[:, -1] - srt[:, -2]) > 1e-3 * np.abs(ref).max()
        assert clear.sum() > 250 and np.array_equal(ids[clear], ref.argmax(1)[clear])
        assert rel_rms(plan.read_buffer("logits", cfg["vocab"]), ref[-1]) <= 2 * TOL_DECODE
        assert ms > 0
    finally:
        plan.free()


def test_greedy_generation_through_the_engine(pkg):
    """engine.generate_tokens_layered (chunked prefill, then the decode step with the device-side argmax) reproduces the oracle's
    greedy continuation; the device loop with feedback gives the same ids; the device sampler at temperature 0 too."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["trio"]
    w = decisive_routing(cfg, S.dinuzen_weights(cfg, 17), 17)
    wd = w64(w)
    prompt = np.random.default_rng(11).integers(0, cfg["vocab"], 19).tolist()
    seq, want = list(prompt), []
    for _ in range(12):
        lg = O.forward(cfg, wd, seq)[-1]
        top = np.sort(lg)
        assert top[-1] - top[-2] > 1e-4, "near-tie in the oracle: pick another seed"
        want.append(int(lg.argmax()))
        seq.append(want[-1])
    plan = make_plan(pkg, cfg, w, ctx=64, batch=5, compute="float32")
    try:
        got = pkg.engine.generate_tokens_layered(plan, prompt, stop_tokens=[], max_tokens=len(prompt) + 11, context_length=64, batch_size=5)
        assert got == want
        stop = want[4]
        got = pkg.engine.generate_tokens_layered(plan, prompt, stop_tokens=[stop], max_tokens=64, context_length=64, batch_size=5)
        assert got == want[:want.index(stop) + 1]
        for c in range(0, len(prompt) - 1, 5):
            plan.forward_batch_prefill(prompt[c:min(c + 5, len(prompt) - 1)], c)
        ids, _ = plan.decode_sequence([prompt[-1]], 12, len(prompt) - 1, feedback=True)
        assert ids.tolist() == want
        sampler = pkg.sampler.select_sampler(cfg["vocab"], 0.0, 0.9, 1)
        got = pkg.engine.generate_tokens_layered(plan, prompt, stop_tokens=[], max_tokens=len(prompt) + 3, context_length=64, batch_size=5, sampler=sampler)
        assert got == want[:4]
        t = plan.forward_decode_sample(prompt[-1], len(prompt) - 1, 1.3, 0.9, 0.4)
        assert 0 <= t < cfg["vocab"]
    finally:
        plan.free()


def random_layer_list(S, rng):
    """A random list of 1 .. 5 layers with random sizes and constants (key readers only after a layer with keys of the same shape)."""
    layers, key_layers = [], []
    for i in range(int(rng.integers(1, 6))):
        pick = rng.random()
        if rng.random() < 0.25:
            mlp = None
        elif rng.random() < 0.4:
            mlp = S.dinuzen_dense(int(rng.integers(4, 70)))
        else:
            X, I = int(rng.integers(0, 6)), int(rng.integers(0, 3))
            if X + I == 0:
                X = 1
            mlp = S.dinuzen_moe(X, int(rng.integers(1, X + I + 1)), int(rng.integers(3, 40)), identity=I, scale=float(rng.uniform(0.5, 3.0)),
                                shared=None if rng.random() < 0.5 else int(rng.integers(3, 50)))
        if pick < 0.4:
            if key_layers and rng.random() < 0.5:
                j = int(rng.choice(key_layers))
                m = layers[j]["mixer"]
                G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
                layers.append(S.dinuzen_attention(G * int(rng.choice([1, 2, 3])), G, dk, dv, mlp, rot_dims=m["rot"]["dims"], base=m["rot"]["base"],
                                                  scaling=tuple(m["rot"]["scaling"][k] for k in ("factor", "original", "fast", "slow")) if "scaling" in m["rot"] else None,
                                                  scale=float(rng.uniform(0.05, 0.6)), softcap=float(rng.choice([0.0, 5.0, 30.0])), diff=float(rng.uniform(0.0, 0.9)), kv_from=j))
            else:
                G = int(rng.choice([1, 2, 3]))
                dk = int(rng.integers(2, 20))
                layers.append(S.dinuzen_attention(G * int(rng.choice([1, 2, 3])), G, dk, int(rng.integers(1, 40)), mlp, rot_dims=2 * int(rng.integers(0, dk // 2 + 1)),
                                                  base=float(rng.choice([10.0, 1e4, 5e5])), scaling=None if rng.random() < 0.5 else (float(rng.uniform(1.5, 8.0)), int(rng.integers(8, 64)), 32.0, 1.0),
                                                  scale=float(rng.uniform(0.05, 0.6)), softcap=float(rng.choice([0.0, 5.0, 30.0])), diff=float(rng.uniform(0.0, 0.9))))
                key_layers.append(i)
        elif pick < 0.7:
            nb = int(rng.choice([1, 2, 3, 5]))
            layers.append(S.dinuzen_rglru(nb * int(rng.integers(1, 14)), nb, int(rng.integers(1, 6)), mlp))
        else:
            G = int(rng.choice([1, 2, 3]))
            H, P = G * int(rng.choice([1, 2])), int(rng.integers(1, 20))
            ng = [g for g in (1, 2, 3, H) if (H * P) % g == 0]
            layers.append(S.dinuzen_mamba2(H, P, int(rng.integers(1, 40)), G, int(rng.integers(1, 6)), mlp, norm_groups=int(rng.choice(ng))))
    return layers


def test_random_layer_lists(pkg):
    """Twelve random layer lists with random sizes and constants: whole, random portions, decode."""
    S, O = pkg.synth, oracle()
    rng = np.random.default_rng(2025)
    for trial in range(12):
        layers = random_layer_list(S, rng)
        g = int(rng.choice([1, 2, 4]))
        cfg = S.dinuzen_config(int(rng.integers(5, 20)) * 4, int(rng.integers(30, 90)), layers, groups=g, eps=float(rng.choice([1e-6, 1e-5, 1e-3])))
        toks = rng.integers(0, cfg["vocab"], 45).tolist()
        for compute in ("float32", "bfloat16"):
            w = S.dinuzen_weights(cfg, 100 + trial)
            if compute == "bfloat16":
                w = decisive_routing(cfg, w, trial)
            elif min_margin(O, cfg, w64(w), toks) < 2e-5:
                continue
            ref = O.forward(cfg, w64(w), toks)
            plan = make_plan(pkg, cfg, w, ctx=64, batch=9, compute=compute)
            try:
                assert_rows(prefill_all(plan, toks, 9), ref, TOL(compute, cfg), f"trial {trial} whole")
                sizes = [int(x) for x in rng.integers(1, 10, 5)]
                assert_rows(portions(plan, toks, sizes, 9), ref, TOL(compute, cfg), f"trial {trial} portions {sizes}")
            finally:
                plan.free()


def test_bad_arguments_are_refused(pkg):
    S = pkg.synth
    cfg = configs(S)["trio"]
    w = S.dinuzen_weights(cfg, 19)
    for drop in ("l0.mix.q.norm", "l0.mix.lk2", "l1.mix.ra.b", "l1.mlp.correction", "l1.mlp.shared.sg", "l2.mix.dt_bias", "l2.dwa", "l1.shift", "final.norm"):
        w2 = {k: v for k, v in w.items() if k != drop}
        with pytest.raises(pkg.native.B200Error):
            make_plan(pkg, cfg, w2)
    A = S.dinuzen_attention
    for bad in ([A(4, 2, 16, 16), A(4, 1, 16, 16, kv_from=0)],      # other key/value heads than the layer it reads
                [A(4, 2, 16, 16, kv_from=0)],                       # reads itself
                [S.dinuzen_rglru(32, 2, 3), A(4, 2, 16, 16, kv_from=0)]):
        c = S.dinuzen_config(64, 96, bad)
        good = S.dinuzen_config(64, 96, [A(4, 2, 16, 16), A(4, 2, 16, 16)])
        with pytest.raises((pkg.native.B200Error, pkg.loader.UnsupportedModel, KeyError)):
            make_plan(pkg, c, S.dinuzen_weights(good, 1))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_replays_steps(pkg, tmp_path, dtype):
    """bin/trace_run on a model directory: steps longer than --chunk, of two tokens and of one, wanted places out of order, steps
    that want nothing, two requests one after the other on one plan (the second starts from an empty state)."""
    import json
    import os
    import subprocess
    import sys

    S, O = pkg.synth, oracle()
    cfg = configs(S)["tiles_a"]
    w = decisive_routing(cfg, S.dinuzen_weights(cfg, 23), 23)
    mdir = str(tmp_path / "model")
    S.write_model_dir(mdir, cfg, w)
    rng = np.random.default_rng(13)
    reqs = {"a": rng.integers(0, cfg["vocab"], 61).tolist(), "b": rng.integers(0, cfg["vocab"], 9).tolist()}
    ref = {k: O.forward(cfg, w64(w), v) for k, v in reqs.items()}
    plan_steps = [("a", 37, [36, 0, 5]), ("a", 2, []), ("a", 20, [19, 18]), ("a", 1, [0]), ("a", 1, []), ("b", 1, [0]), ("b", 8, [7, 3])]
    lines, expect, at = [], {}, {"a": 0, "b": 0}
    for n, (rid, count, want) in enumerate(plan_steps):
        lo = at[rid]
        at[rid] = lo + count
        end = [rid] if at[rid] == len(reqs[rid]) else []
        lines.append(json.dumps({"step": n, "entries": [{"id": rid, "tokens": reqs[rid][lo:lo + count], "want": want}], "end": end}))
        if want:
            expect[n] = np.stack([ref[rid][lo + k] for k in want])
    out = str(tmp_path / "out")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", mdir, "--dtype", dtype, "--out", out, "--max-tokens", "64",
                        "--chunk", "16"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == ["done %d" % n for n in range(len(plan_steps))]
    for n in range(len(plan_steps)):
        path = os.path.join(out, "%d.f32" % n)
        if n in expect:
            got = np.fromfile(path, dtype="<f4").reshape(expect[n].shape)
            assert_rows(got, expect[n], TOL(dtype, cfg), f"step {n}")
        else:
            assert not os.path.exists(path)
