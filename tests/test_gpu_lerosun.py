"""GPU tests of the pre-norm layered plans (csrc/delta.cuh, csrc/layered.cuh, csrc/layered_plan.cuh) on small random Lerosun
models, against the float64 oracle (oracle/lerosun_oracle.py, which shares no code with the product).

Tolerances.  FP32 compute mode and the decode step (FP32 activations in either mode): relative RMS error of a logits row
<= 3e-5 (only the summation order differs): this is the sharp comparison, and every case runs in it.  BF16 compute mode, batched
prefill: GEMM operands are rounded to BF16 and the untrained random layers pass the rounding of every layer run on to the next, so
the bound grows with depth: 1.2 % per layer run (+ 1 for the classifier); measured 0.3 % .. 1 % per run.  Where a test plants a key
that decides the output, the model has one layer (bound 2.4 %) and a window, state or cache slip moves the row by more than 10 %."""
import numpy as np
import pytest

from lerosun_util import bf16_values, configs, needle_attention, needle_delta, oracle, rel_rms, w64

pytestmark = pytest.mark.gpu

TOL_DECODE = 3e-5


def runs_of(cfg):
    n, loop = len(cfg["layers"]), cfg.get("loop")
    return n + ((loop["times"] - 1) * (loop["stop"] - loop["start"]) if loop else 0)


class _Tol:
    """TOL[compute] for one-layer models; TOL(compute, cfg) scales the BF16 bound with the number of layer runs."""

    def __getitem__(self, compute):
        return {"float32": 3e-5, "bfloat16": 2.4e-2}[compute]

    def __call__(self, compute, cfg):
        return 3e-5 if compute == "float32" else 1.2e-2 * (runs_of(cfg) + 1)


TOL = _Tol()


def make_plan(pkg, cfg, weights, ctx=256, batch=16, compute="float32"):
    model = pkg.synth.lerosun_model(cfg, weights, ctx)
    return pkg.B200MasterPlan.initialize_plan(model, prefill_batch_size=batch, compute=compute)


def prefill_all(plan, toks, batch, start=0):
    rows = []
    for c0 in range(0, len(toks), batch):
        part = toks[c0:c0 + batch]
        lg, _ = plan.forward_batch_logits(part, start + c0, list(range(len(part))))
        rows.append(lg)
    return np.concatenate(rows)


def assert_rows(got, ref, tol, what=""):
    worst = max(rel_rms(got[i], ref[i]) for i in range(len(ref)))
    assert worst <= tol, f"{what}: relative RMS error {worst:.3g} > {tol}"


def portions(plan, toks, sizes, batch):
    """The prompt in portions of the given sizes (each cut again at the chunk capacity), the rest decoded one by one."""
    got, p = [], 0
    for m in sizes:
        got.append(prefill_all(plan, toks[p:p + m], batch, start=p))
        p += m
    while p < len(toks):
        got.append(plan.forward_decode(toks[p], p)[0][None])
        p += 1
    return np.concatenate(got)


@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["pair", "loop_mid", "loop_start_odd", "loop_once_end", "window_one", "delta_only", "attention_only", "big_key", "tiles_a", "tiles_b"])
def test_every_layer_run_matches_oracle(pkg, name, compute):
    """Residual stream after every layer run and the logits: each mixer alone (delta_only, attention_only) and in every order."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    w = S.lerosun_weights(cfg, 11)
    toks = np.random.default_rng(5).integers(0, cfg["vocab"], 23).tolist()
    ref_lg, ref_tr = O.forward(cfg, w64(w), toks, want_layers=True)
    plan = make_plan(pkg, cfg, w, batch=32, compute=compute)
    try:
        assert plan.layered_info()[0] == len(ref_tr)
        lg, tr = plan.forward_batch_logits(toks, 0, list(range(len(toks))), want_trace=True)
        for r in range(len(ref_tr)):
            assert rel_rms(tr[r], ref_tr[r]) <= TOL(compute, cfg), f"layer run {r}"
        assert_rows(lg, ref_lg, TOL(compute, cfg), "logits")
    finally:
        plan.free()


@pytest.mark.parametrize("name", ["loop_mid", "loop_start_odd", "delta_only", "big_key", "tiles_a"])
def test_prefill_equals_token_by_token_decode(pkg, name):
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    w = S.lerosun_weights(cfg, 12)
    toks = np.random.default_rng(6).integers(0, cfg["vocab"], 40).tolist()
    ref = O.forward(cfg, w64(w), toks)
    for compute in ("float32", "bfloat16"):
        plan = make_plan(pkg, cfg, w, batch=64, compute=compute)
        try:
            whole = prefill_all(plan, toks, 64)
            step = np.stack([plan.forward_decode(t, p)[0] for p, t in enumerate(toks)])  # position 0 starts from an empty state without a reset
            assert_rows(step, ref, TOL_DECODE, "decode")
            assert_rows(whole, ref, TOL(compute, cfg), "prefill")
        finally:
            plan.free()


@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["loop_mid", "loop_start_odd", "big_key"])
def test_portions_of_every_size(pkg, name, compute):
    """The same prompt cut into portions of 2 .. 13 tokens (edges inside windows and inside the convolution's taps), then decoded one
    by one; the chunk capacity (7) is below the portion sizes, so portions are cut again, and both rings wrap."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    w = S.lerosun_weights(cfg, 13)
    toks = np.random.default_rng(7).integers(0, cfg["vocab"], 70).tolist()
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, batch=7, compute=compute)
    try:
        for sizes in ([2, 3, 2, 13, 5, 2, 11, 2, 7], [9, 2, 2, 2, 12, 3], [50], [2] * 20):
            assert_rows(portions(plan, toks, sizes, 7), ref, TOL(compute, cfg), f"portions {sizes}")
    finally:
        plan.free()


@pytest.mark.parametrize("name", ["tiles_a", "tiles_b"])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_tensor_core_prefill_shapes(pkg, name, compute):
    """Shapes that take the tcgen05 GEMMs and the tensor-core attention in BF16 mode: a prompt longer than several key tiles, whole
    and in ragged portions (one of them a single row), then decoded."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    w = S.lerosun_weights(cfg, 21)
    toks = np.random.default_rng(12).integers(0, cfg["vocab"], 230).tolist()
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, ctx=256, batch=100, compute=compute)
    try:
        assert_rows(prefill_all(plan, toks, 100), ref, TOL(compute, cfg), "whole")
        assert_rows(portions(plan, toks, (65, 2, 100, 1, 37), 100), ref, TOL(compute, cfg), "portions")
    finally:
        plan.free()


def test_state_and_slots_are_reused_across_requests(pkg):
    """Request after request on one plan without clearing anything, each long enough to wrap the rings several times: a request
    starts from an empty recurrent state and empty windows whatever the previous one left; b200_kv_reset in between changes nothing."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["pair"]
    w = S.lerosun_weights(cfg, 14)
    plan = make_plan(pkg, cfg, w, batch=4, compute="float32")
    rng = np.random.default_rng(8)
    try:
        for k, n in enumerate((30, 3, 41, 1, 17, 2)):
            toks = rng.integers(0, cfg["vocab"], n).tolist()
            ref = O.forward(cfg, w64(w), toks)
            cut = n // 2
            got = [prefill_all(plan, toks[:cut], 4)] if cut else []
            got += [plan.forward_decode(toks[p], p)[0][None] for p in range(cut, n)]
            assert_rows(np.concatenate(got), ref, TOL["float32"], f"request of {n}")
            assert np.abs(plan.read_buffer("delta_state", 4 * 16 * 16, layer=0)).max() > 0
            if k == 2:
                plan.kv_reset()
                assert np.abs(plan.read_buffer("delta_state", 4 * 16 * 16, layer=0)).max() == 0
    finally:
        plan.free()


@pytest.mark.parametrize("kv_heads", [1, 2])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_window_edges_with_a_planted_key(pkg, compute, kv_heads):
    """A key that decides the output, placed just inside (distance window - 1) and just outside (distance window) the window, far
    away, and at the first positions of the sequence -- in a prompt, across a portion edge, and while decoding."""
    S, O = pkg.synth, oracle()
    W = 12
    cfg, w, A, B, fill = needle_attention(S, W, kv_heads=kv_heads)
    wd = w64(w)
    plan = make_plan(pkg, cfg, w, batch=8, compute=compute)
    try:
        for i, dist in [(40, W - 1), (40, W), (40, W - 2), (40, 1), (40, 0), (W - 1, W - 1), (W, W), (3, 3), (0, 0), (57, 37)]:
            toks = [fill[(5 * t + 1) % len(fill)] for t in range(i + 1)]
            toks[i] = A
            if dist:
                toks[i - dist] = B
            ref = O.forward(cfg, wd, toks)
            got = prefill_all(plan, toks, 8)
            assert_rows(got[i:i + 1], ref[i:i + 1], TOL[compute], f"prompt, query {i}, key at distance {dist}")
            if i:
                prefill_all(plan, toks[:i], 8)
            lg = plan.forward_decode(toks[i], i)[0]
            assert rel_rms(lg, ref[i]) <= TOL[compute], f"decoded query {i}, key at distance {dist}"  # the keys came from the prefill kernels
            for p, t in enumerate(toks):
                lg = plan.forward_decode(t, p)[0]
            assert rel_rms(lg, ref[i]) <= TOL_DECODE, f"all decoded, query {i}, key at distance {dist}"

        def row(dist):
            toks = [fill[(5 * t + 1) % len(fill)] for t in range(41)]
            toks[40], toks[40 - dist] = A, B
            return prefill_all(plan, toks, 8)[40]
        assert rel_rms(row(W - 1), row(W)) > 0.1  # the planted key has teeth
    finally:
        plan.free()


@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(pkg, compute):
    """Window 300 (several key tiles, split over CTAs in the decode step): the planted key 290 back is seen, 300 back is not, in a
    prompt cut at a chunk edge and while decoding."""
    S, O = pkg.synth, oracle()
    cfg, w, A, B, fill = needle_attention(S, 300, kv_heads=2)
    wd = w64(w)
    plan = make_plan(pkg, cfg, w, ctx=400, batch=128, compute=compute)
    try:
        rows = {}
        for dist in (290, 299, 300):
            toks = [fill[(7 * t + 3) % len(fill)] for t in range(331)]
            toks[330], toks[330 - dist] = A, B
            ref = O.forward(cfg, wd, toks)[330]
            rows[dist] = prefill_all(plan, toks, 128)[330]
            assert rel_rms(rows[dist], ref) <= TOL[compute], f"prompt, distance {dist}"
            prefill_all(plan, toks[:320], 128)
            for p in range(320, 331):
                lg = plan.forward_decode(toks[p], p)[0]
            assert rel_rms(lg, ref) <= TOL[compute], f"decoded, distance {dist}"
        assert rel_rms(rows[299], rows[300]) > 0.1
    finally:
        plan.free()


@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_the_state_keeps_a_far_write(pkg, compute):
    """Gated delta rule with decays near one: what token B wrote 400 tokens back decides the read-out at token A -- whole, across
    chunk edges, with the last tokens decoded, and all decoded; without B the row is a different one."""
    S, O = pkg.synth, oracle()
    cfg, w, A, B, fill = needle_delta(S)
    wd = w64(w)
    plan = make_plan(pkg, cfg, w, ctx=512, batch=64, compute=compute)
    try:
        n = 420
        toks = [fill[(7 * t + 3) % len(fill)] for t in range(n)]
        toks[n - 1] = A
        without = O.forward(cfg, wd, toks)[n - 1]
        for at in (0, 1, 19, n - 2):
            t2 = list(toks)
            t2[at] = B
            ref = O.forward(cfg, wd, t2)[n - 1]
            assert rel_rms(ref, without) > 0.1, "the planted write has teeth"
            assert rel_rms(prefill_all(plan, t2, 64)[n - 1], ref) <= TOL[compute], f"prompt, write at {at}"
            assert rel_rms(portions(plan, t2, [3, 64, 2, 300], 64)[n - 1], ref) <= TOL[compute], f"portions, write at {at}"
        ids, _ = plan.decode_sequence(t2, n, 0, feedback=False)
        assert rel_rms(plan.read_buffer("logits", cfg["vocab"]), ref) <= TOL_DECODE
    finally:
        plan.free()


def test_each_attention_mechanism_alone(pkg):
    """Weights that isolate one mechanism each, against the oracle in FP32 (prefill and decode): a mixing matrix far from the identity;
    temperatures of both signs; a sink that takes nearly all the mass (the mixer adds next to nothing) and one that takes none; a
    gate that closes one head; rotation over the whole head with a small base (fast turning); no rotation at all."""
    S, O = pkg.synth, oracle()
    rng = np.random.default_rng(9)
    toks = rng.integers(0, 60, 50).tolist()
    for case in ("talk", "temp", "sink_all", "sink_none", "gate", "rot_full", "rot_none"):
        rot = {"rot_full": 8, "rot_none": 0}.get(case, 4)
        cfg = S.lerosun_config(40, 60, [S.lerosun_attention(4, 2, 8, 33, 48, rot_dims=rot, base=3.0 if case == "rot_full" else 10000.0)])
        w = S.lerosun_weights(cfg, 15)
        if case == "talk":
            w["l0.mix.talk"] = rng.standard_normal((4, 4)).astype(np.float32)
        if case == "temp":
            w["l0.mix.temp"] = np.array([2.0, -1.5, 0.25, 0.0], dtype=np.float32)
        if case == "sink_all":
            w["l0.mix.sink"][:] = 30.0
        if case == "sink_none":
            w["l0.mix.sink"][:] = -30.0
        if case == "gate":
            w["l0.mix.g"][1] = 0.0
            w["l0.mix.g"][2] *= 20.0
        w = bf16_values(w)
        ref_lg, ref_tr = O.forward(cfg, w64(w), toks, want_layers=True)
        if case == "sink_all":
            x0 = O.scalar_rms_norm(w64(w)["embed"][np.asarray(toks)], w64(w)["embed.norm"], cfg["norm"]["eps"])
            no_mixer = x0 + w64(w)["l0.ls2"] * O.relu_gated_ff(O.scalar_rms_norm(x0, w64(w)["l0.norm2"], cfg["norm"]["eps"]), w64(w), "l0.mlp.")
            assert rel_rms(ref_tr[0], no_mixer) < 1e-6
        plan = make_plan(pkg, cfg, w, batch=64, compute="float32")
        try:
            lg, tr = plan.forward_batch_logits(toks, 0, list(range(len(toks))), want_trace=True)
            assert rel_rms(tr[0], ref_tr[0]) <= TOL["float32"], case
            assert_rows(lg, ref_lg, TOL["float32"], case)
            step = np.stack([plan.forward_decode(t, p)[0] for p, t in enumerate(toks)])
            assert_rows(step, ref_lg, TOL_DECODE, case + " (decode)")
        finally:
            plan.free()


def test_each_delta_mechanism_alone(pkg):
    """The same for the delta mixer: decays near zero (the state forgets at once) and near one, betas driven to zero or one token by
    token (nothing is written / the old value is replaced), a convolution that only looks back (current tap zero), and the first tokens of a sequence (zeros before the start)."""
    S, O = pkg.synth, oracle()
    rng = np.random.default_rng(10)
    toks = rng.integers(0, 60, 37).tolist()
    for case in ("forget", "keep", "beta_extreme", "look_back"):
        cfg = S.lerosun_config(40, 60, [S.lerosun_delta(4, 2, 8, 12, 4, None)])
        w = S.lerosun_weights(cfg, 16)
        if case == "forget":
            w["l0.mix.A_log"][:] = 3.0
        if case == "keep":
            w["l0.mix.A_log"][:] = -12.0
        if case == "beta_extreme":
            w["l0.mix.b"] *= 20.0
        if case == "look_back":
            for n in ("q.conv", "k.conv", "v.conv"):
                w["l0.mix." + n][:, -1] = 0.0
        w = bf16_values(w)
        ref_lg, ref_tr = O.forward(cfg, w64(w), toks, want_layers=True)
        plan = make_plan(pkg, cfg, w, batch=64, compute="float32")
        try:
            lg, tr = plan.forward_batch_logits(toks, 0, list(range(len(toks))), want_trace=True)
            assert rel_rms(tr[0][:5], ref_tr[0][:5]) <= TOL["float32"], case + ": first tokens"
            assert rel_rms(tr[0], ref_tr[0]) <= TOL["float32"], case
            assert_rows(portions(plan, toks, [1, 2, 3, 2], 64), ref_lg, TOL["float32"], case + " (portions inside the taps, decode)")
        finally:
            plan.free()


def test_long_decoding_through_the_device_loop(pkg):
    """300 single-token steps in one call of the device-resident loop (teacher-forced): the argmax of every step equals the
    oracle's wherever the oracle's best two logits are not a near-tie, and the last logits agree."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["loop_once_end"]
    w = S.lerosun_weights(cfg, 16)
    toks = np.random.default_rng(10).integers(0, cfg["vocab"], 300).tolist()
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, ctx=320, batch=1, compute="bfloat16")
    try:
        ids, ms = plan.decode_sequence(toks, len(toks), 0, feedback=False)
        srt = np.sort(ref, axis=1)
        clear = (srt[:, -1] - srt[:, -2]) > 1e-3 * np.abs(ref).max()
        assert clear.sum() > 250 and np.array_equal(ids[clear], ref.argmax(1)[clear])
        assert rel_rms(plan.read_buffer("logits", cfg["vocab"]), ref[-1]) <= TOL_DECODE
        assert ms > 0
    finally:
        plan.free()


def test_greedy_generation_through_the_engine(pkg):
    """engine.generate_tokens_layered (chunked prefill, then the decode step with the device-side argmax) reproduces the oracle's
    greedy continuation; the device loop with feedback gives the same ids; the device sampler at temperature 0 too."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["loop_mid"]
    w = S.lerosun_weights(cfg, 17)
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


def test_random_layer_lists(pkg):
    """Ten random layer lists with random sizes and constants: whole, random portions, decode."""
    S, O = pkg.synth, oracle()
    rng = np.random.default_rng(2024)
    for trial in range(10):
        layers = []
        for _ in range(int(rng.integers(1, 5))):
            G = int(rng.choice([1, 2, 3]))
            H = G * int(rng.choice([1, 2, 3]))
            ff = None if rng.random() < 0.3 else int(rng.integers(8, 70))
            if rng.random() < 0.5:
                dk = int(rng.integers(2, 20))
                layers.append(S.lerosun_attention(H, G, dk, int(rng.integers(1, 40)), ff, rot_dims=2 * int(rng.integers(0, dk // 2 + 1)),
                                                  base=float(rng.choice([10.0, 1e4, 5e5])), scale=float(rng.uniform(0.05, 0.6))))
            else:
                layers.append(S.lerosun_delta(H, G, int(rng.integers(2, 20)), int(rng.integers(2, 80)), int(rng.integers(1, 6)), ff))
        n = len(layers)
        a = int(rng.integers(0, n))
        loop = None if rng.random() < 0.4 else (a, int(rng.integers(a + 1, n + 1)), int(rng.integers(1, 4)))
        cfg = S.lerosun_config(int(rng.integers(5, 20)) * 4 + int(rng.integers(0, 4)), int(rng.integers(30, 90)), layers, loop=loop, eps=float(rng.choice([1e-6, 1e-5, 1e-3])))
        w = S.lerosun_weights(cfg, 100 + trial)
        toks = rng.integers(0, cfg["vocab"], 45).tolist()
        ref = O.forward(cfg, w64(w), toks)
        for compute in ("float32", "bfloat16"):
            plan = make_plan(pkg, cfg, w, ctx=64, batch=9, compute=compute)
            try:
                assert_rows(prefill_all(plan, toks, 9), ref, TOL(compute, cfg), f"trial {trial} whole")
                sizes = [int(x) for x in rng.integers(2, 10, 5)]
                assert_rows(portions(plan, toks, sizes, 9), ref, TOL(compute, cfg), f"trial {trial} portions {sizes}")
            finally:
                plan.free()


def test_bad_arguments_are_refused(pkg):
    S = pkg.synth
    cfg = configs(S)["pair"]
    w = S.lerosun_weights(cfg, 19)
    for drop in ("l0.mix.q.conv", "l1.mix.talk", "l1.mix.sink", "embed.norm", "l1.ls2"):
        w2 = {k: v for k, v in w.items() if k != drop}
        with pytest.raises(pkg.native.B200Error):
            make_plan(pkg, cfg, w2)
    bad = S.lerosun_config(64, 96, [S.lerosun_attention(4, 2, 16, 6, 96)])
    bad["layers"][0]["mixer"]["vdim"] = 8  # values are keys: the sizes must agree
    wb = S.lerosun_weights(S.lerosun_config(64, 96, [S.lerosun_attention(4, 2, 16, 6, 96)]), 1)
    with pytest.raises(pkg.native.B200Error):
        make_plan(pkg, bad, wb)


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
    w = S.lerosun_weights(cfg, 23)
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
