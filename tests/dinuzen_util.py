"""Shared helpers of the Dinuzen tests: small configurations, weights with planted keys and writes, the float64 oracle."""
import importlib.util
import os
import sys

import numpy as np

from pibidra_util import bf16_values, rel_rms, w64  # noqa: F401

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def oracle():
    name = "dinuzen_oracle"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "oracle", "dinuzen_oracle.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def configs(S):
    """name -> config.  Sizes differ from one another on purpose: grouped, ungrouped and single key/value heads, key and value sizes
    that are no multiple of 4, rotation of all / part / none of a slice with and without frequency blending, keys shared over one
    and two layers and by several readers, 1 .. 5 taps, one and several gate blocks, state sizes below and above one register row
    per lane, one and several groups of B and C, norm groups of 1 and more in the residual and in the read-out, layers without a
    feed-forward, experts with and without identity experts / a shared expert, all experts chosen, one expert chosen."""
    A, R, M, D, X = S.dinuzen_attention, S.dinuzen_rglru, S.dinuzen_mamba2, S.dinuzen_dense, S.dinuzen_moe
    return {
        "trio": S.dinuzen_config(64, 96, [A(4, 2, 16, 16, D(96)), R(32, 2, 4, X(4, 2, 24, identity=1, scale=1.5, shared=40)), M(4, 8, 16, 2, 4, X(3, 1, 16))], groups=4),
        "shared_keys": S.dinuzen_config(48, 80, [A(3, 3, 10, 14, None, rot_dims=10, scaling=(4.0, 32, 8.0, 1.0), scale=0.3), M(2, 12, 20, 1, 3, D(40), norm_groups=3),
                                                 A(6, 3, 10, 14, X(5, 3, 20, identity=2, scale=2.0, shared=12), kv_from=0, rot_dims=10, scaling=(4.0, 32, 8.0, 1.0), softcap=5.0),
                                                 R(24, 3, 2, None), A(3, 3, 10, 14, D(24), kv_from=0, rot_dims=10, scaling=(4.0, 32, 8.0, 1.0), diff=0.6)], groups=3, eps=1e-6),
        "odd": S.dinuzen_config(36, 51, [R(21, 1, 1, X(2, 2, 10, identity=0, shared=None)), A(4, 1, 6, 9, X(1, 1, 8, identity=3, scale=0.7), rot_dims=2, base=50.0, softcap=0.0),
                                         M(3, 5, 7, 3, 5, None, norm_groups=1), A(2, 2, 7, 5, None, rot_dims=0)], groups=1, eps=1e-3),
        "recurrent_only": S.dinuzen_config(56, 70, [M(1, 40, 33, 1, 2, D(60)), R(70, 5, 3, D(30)), M(6, 4, 130, 2, 4, None, norm_groups=4), R(8, 8, 5, None)], groups=7),
        "attention_only": S.dinuzen_config(56, 70, [A(4, 1, 14, 8, D(60), rot_dims=6), A(8, 8, 4, 13, None, rot_dims=4, base=7.0), A(8, 8, 4, 13, X(6, 6, 8, identity=2), kv_from=1, rot_dims=4, base=7.0)], groups=2),
        # shapes the tensor-core prefill takes: widths in whole GEMM tiles, (key, value) sizes 64 / 64 and 128 / 128, expert widths of 64
        "tiles_a": S.dinuzen_config(128, 256, [A(2, 1, 64, 64, D(256)), R(128, 2, 4, X(4, 2, 64, identity=1, scale=2.0, shared=128)), M(2, 64, 32, 1, 4, X(3, 2, 128, shared=None)),
                                               A(4, 1, 64, 64, X(4, 3, 64, identity=2, shared=128), kv_from=0)], groups=4),
        "tiles_b": S.dinuzen_config(256, 384, [M(4, 32, 64, 2, 3, D(128), norm_groups=2), A(2, 2, 128, 128, X(6, 2, 64, identity=0, scale=1.75, shared=256), rot_dims=32),
                                               R(256, 4, 2, None), A(2, 2, 128, 128, D(384), rot_dims=32, kv_from=1)], groups=2),
    }


def decisive_routing(cfg, w, seed: int = 0):
    """Weights whose routers never face a close call, for comparisons in reduced precision (a flipped expert is a different
    function, not a rounding error).  The last R entries of the width are reserved for routing: a token's embedding holds there a
    ladder 0.5, 1, ... in an order of its own, no layer writes to them (both layer scales are zero there), the depth average keeps
    them (its weights sum to one), and router row e reads one of them; the corrections are small against the ladder's steps.
    Everything else stays random, and all other weights read the reserved entries like any other."""
    rng = np.random.default_rng(seed)
    E, V = cfg["width"], cfg["vocab"]
    counts = [lc["mlp"]["router"]["experts"] + lc["mlp"]["router"].get("identity", 0) for lc in cfg["layers"] if lc["mlp"] is not None and lc["mlp"]["kind"] == "moe"]
    R = max(counts + [1])
    w = {k: v.copy() for k, v in w.items()}
    for t in range(V):
        w["embed"][t, E - R:] = 0.5 * (1 + rng.permutation(R))
    for i, lc in enumerate(cfg["layers"]):
        w[f"l{i}.ls1"][E - R:] = 0.0
        w[f"l{i}.dwa"] = (w[f"l{i}.dwa"] / w[f"l{i}.dwa"].sum()).astype(np.float32)
        if lc["mlp"] is None:
            continue
        w[f"l{i}.ls2"][E - R:] = 0.0
        if lc["mlp"]["kind"] != "moe":
            continue
        n = lc["mlp"]["router"]["experts"] + lc["mlp"]["router"].get("identity", 0)
        pick = rng.permutation(R)[:n]
        r = np.zeros((n, E), dtype=np.float32)
        r[np.arange(n), E - R + pick] = 1.0
        w[f"l{i}.mlp.router"] = r
        w[f"l{i}.mlp.correction"] = (0.004 * rng.standard_normal(n)).astype(np.float32)
    return bf16_values(w)


def min_margin(O, cfg, w, toks):
    """Smallest gap, over all tokens and routers, between the choice scores of the last chosen and the first rejected expert."""
    gaps = []

    def probe(i, x):
        mlp = cfg["layers"][i]["mlp"]
        r = mlp["router"]
        z = x @ w[f"l{i}.mlp.router"].T
        s = np.exp(z - z.max(-1, keepdims=True))
        s /= s.sum(-1, keepdims=True)
        c = np.sort(s + w[f"l{i}.mlp.correction"], axis=-1)[:, ::-1]
        if r["top"] < c.shape[1]:
            gaps.append(float((c[:, r["top"] - 1] - c[:, r["top"]]).min()))

    O.forward(cfg, w, toks, on_moe_input=probe)
    return min(gaps) if gaps else 1.0


def _one_hot_model(S, layer, V: int, E: int, seed: int):
    """One layer over one-hot embeddings, no token shift, a depth average that passes the layer's result on."""
    cfg = S.dinuzen_config(E, V, [layer], groups=1)
    w = S.dinuzen_weights(cfg, seed)
    emb = np.zeros((V, E), dtype=np.float32)
    emb[np.arange(V), np.arange(V)] = 1.0
    w["embed"] = emb
    w["l0.shift"][:] = 0.0
    w["l0.dwa"] = np.asarray([0.0, 1.0], dtype=np.float32)
    return cfg, w


def needle_attention(S, kv_heads: int = 1, rot_dims: int = 8, seed: int = 3):
    """One attention layer decided by ONE planted key: with one-hot embeddings the first map's query of token A and key of token B
    are aligned in the unrotated entries of the slice (so the alignment holds at every distance) while all other pairs are
    unrelated directions; B's value is large and its direction decides the head's output.  Returns (config, weights, A, B, filler tokens)."""
    E, V, H, dk, dv = 64, 48, 4, 16, 12
    cfg, w = _one_hot_model(S, S.dinuzen_attention(H, kv_heads, dk, dv, None, rot_dims=rot_dims, scale=1.0, softcap=50.0, diff=0.2), V, E, seed)
    rng = np.random.default_rng(seed)
    w["l0.mix.q.norm"][:] = 1.0
    w["l0.mix.k.norm"][:] = 1.0
    A, B = 5, 9
    u = np.zeros(dk, dtype=np.float32)
    u[rot_dims:] = rng.standard_normal(dk - rot_dims)
    q = w["l0.mix.q"].reshape(H, 2, dk, E)
    k = w["l0.mix.k"].reshape(kv_heads, 2, dk, E)
    q[:, 0, :, A] = u
    k[:, 0, :, B] = u
    w["l0.mix.v"][:, B] = 6.0 * rng.standard_normal(kv_heads * dv).astype(np.float32)
    fill = [t for t in range(V) if t not in (A, B)]
    return cfg, bf16_values(w), A, B, fill


def needle_rglru(S, seed: int = 4):
    """One recurrent unit that keeps what token B wrote: decays of (nearly) one, the fillers feed zeros (one tap, no biases), B a
    large input; the read-out at A is the kept state times A's other branch.  Returns (config, weights, A, B, filler tokens)."""
    E, V, W = 64, 48, 32
    cfg, w = _one_hot_model(S, S.dinuzen_rglru(W, 2, 1, None), V, E, seed)
    rng = np.random.default_rng(seed)
    A, B = 5, 9
    w["l0.mix.lam"][:] = -9.0  # a = exp(-8 r softplus(-9)) = 1 - O(1e-3)
    w["l0.mix.x"][:] = 0.0
    w["l0.mix.x"][:, B] = 40.0 * rng.standard_normal(W).astype(np.float32)
    w["l0.mix.x.b"][:] = 0.0
    w["l0.mix.conv"][:] = 1.0
    w["l0.mix.conv.b"][:] = 0.0
    w["l0.mix.y"][:, A] = 2.0 + np.abs(rng.standard_normal(W)).astype(np.float32)
    fill = [t for t in range(V) if t not in (A, B)]
    return cfg, bf16_values(w), A, B, fill


def needle_ssd(S, seed: int = 5):
    """One state-space layer that keeps what token B wrote: decays of (nearly) one, the fillers' x is zero (one tap, no bias), B
    writes a large x along its B vector, A reads along the same direction.  Returns (config, weights, A, B, filler tokens)."""
    E, V, H, P, N = 64, 48, 2, 8, 16
    cfg, w = _one_hot_model(S, S.dinuzen_mamba2(H, P, N, 1, 1, None, norm_groups=1), V, E, seed)
    rng = np.random.default_rng(seed)
    A, B = 5, 9
    inner = H * P
    win = w["l0.mix.in"]
    win[inner:2 * inner] = 0.0                                    # x rows: zero for every filler
    win[inner:2 * inner, B] = 8.0 + np.abs(rng.standard_normal(inner)).astype(np.float32)
    u = (1.0 + np.abs(rng.standard_normal(N))).astype(np.float32)  # positive: SiLU keeps it roughly as it is
    win[2 * inner:2 * inner + N, B] = u                           # B of token B
    win[2 * inner + N:2 * inner + 2 * N, A] = u                   # C of token A
    win[:inner, A] = 2.0                                          # an open gate at A
    w["l0.mix.conv"][:] = 1.0
    w["l0.mix.conv.b"][:] = 0.0
    w["l0.mix.A_log"][:] = -9.0
    w["l0.mix.dt_bias"][:] = 0.5
    w["l0.mix.D"][:] = 0.0
    fill = [t for t in range(V) if t not in (A, B)]
    return cfg, bf16_values(w), A, B, fill
