"""Shared helpers of the Lerosun tests: small configurations, weights with planted keys, the float64 oracle."""
import importlib.util
import os
import sys

import numpy as np

from pibidra_util import bf16_values, rel_rms, w64  # noqa: F401

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def oracle():
    name = "lerosun_oracle"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "oracle", "lerosun_oracle.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def configs(S):
    """name -> config.  Sizes differ from one another on purpose: grouped, ungrouped and single key heads, key sizes that are no
    multiple of 4, value sizes above one state tile, 1 .. 5 taps, rotation of all / part / none of a head, windows of 1 and beyond
    the prompt, layers with and without feed-forward in both mixers, loops at the start / middle / end / of one pass / none."""
    A, D = S.lerosun_attention, S.lerosun_delta
    return {
        "pair": S.lerosun_config(64, 96, [D(4, 2, 16, 16, 3, None), A(4, 2, 16, 6, 96)]),
        "loop_mid": S.lerosun_config(48, 80, [D(2, 1, 8, 24, 4, 40), A(3, 3, 10, 9, None, rot_dims=10), A(4, 2, 12, 5, 72, rot_dims=4, base=50.0),
                                                D(6, 2, 6, 6, 2, None), A(2, 1, 20, 7, 56, rot_dims=0)], loop=(1, 4, 3), eps=1e-6),
        "loop_start_odd": S.lerosun_config(36, 51, [A(6, 2, 6, 3, 30, scale=0.4), D(3, 3, 5, 7, 1, 44), D(2, 1, 12, 72, 5, None)], loop=(0, 2, 2)),
        "loop_once_end": S.lerosun_config(40, 64, [D(5, 1, 8, 8, 3, 64), A(5, 1, 8, 11, None)], loop=(1, 2, 1)),
        "window_one": S.lerosun_config(32, 40, [A(2, 1, 16, 1, 48), D(1, 1, 4, 4, 2, 16), A(2, 2, 16, 200, 48)]),
        "delta_only": S.lerosun_config(56, 70, [D(4, 4, 9, 11, 3, 60), D(2, 1, 32, 130, 4, None)]),
        "attention_only": S.lerosun_config(56, 70, [A(4, 1, 14, 8, 60, rot_dims=6), A(8, 8, 4, 13, None, rot_dims=4, base=7.0)]),
        # key sizes beyond what the delta rule keeps in registers (the shared-memory kernel) and a wide folded key row
        "big_key": S.lerosun_config(44, 50, [D(2, 1, 136, 20, 2, None), A(4, 4, 36, 10, 32, rot_dims=18), D(3, 3, 130, 70, 3, 24)]),
        # shapes the tensor-core prefill takes: widths in whole GEMM tiles; folded key rows / value sizes of 128 / 64, 64 / 64, 128 / 128, 256 / 128
        "tiles_a": S.lerosun_config(128, 256, [A(2, 2, 64, 70, 256), D(2, 1, 64, 64, 4, 128), A(4, 1, 64, 9, 256, rot_dims=64)], loop=(0, 2, 2)),
        "tiles_b": S.lerosun_config(256, 384, [D(2, 2, 128, 128, 3, None), A(2, 1, 128, 33, 128, rot_dims=32), A(4, 2, 128, 129, 384)]),
    }


def needle_attention(S, window: int, kv_heads: int = 1, rot_dims: int = 8, seed: int = 3):
    """One attention layer decided by ONE planted key: the embedding is one-hot, so the query of token A and the key of token B
    can be aligned (in the unrotated entries of the head, so the alignment holds at every distance) while all other pairs stay
    small; B's key -- which is also its value -- is large.  Returns (config, weights, A, B, filler tokens)."""
    E, V, H, dk = 64, 48, 4, 16
    cfg = S.lerosun_config(E, V, [S.lerosun_attention(H, kv_heads, dk, window, 64, rot_dims=rot_dims, scale=1.0)])
    w = S.lerosun_weights(cfg, seed)
    rng = np.random.default_rng(seed)
    emb = np.zeros((V, E), dtype=np.float32)
    emb[np.arange(V), np.arange(V)] = 1.0
    w["embed"] = emb
    w["embed.norm"] = np.asarray(1.0 / 8.0, dtype=np.float32)  # a one-hot row of width 64 has root mean square 1/8: rows stay one-hot
    w["l0.norm1"] = np.asarray(1.0 / 8.0, dtype=np.float32)
    w["l0.mix.q"] *= 0.05
    w["l0.mix.k"] *= 0.05
    w["l0.mix.q.b"][:] = 0.0
    w["l0.mix.k.b"][:] = 0.0
    w["l0.mix.talk"] = (np.eye(H) + 0.25 * (1 - np.eye(H))).astype(np.float32)
    w["l0.mix.temp"][:] = 1.0
    w["l0.mix.sink"][:] = -4.0
    A, B = 5, 9
    u = np.zeros(dk, dtype=np.float32)
    u[rot_dims:] = rng.standard_normal(dk - rot_dims)
    u *= 4.0 / np.linalg.norm(u)
    w["l0.mix.q"][:, A] = np.tile(u, H)
    w["l0.mix.k"][:, B] = np.tile(u, kv_heads)
    fill = [t for t in range(V) if t not in (A, B)]
    return cfg, bf16_values(w), A, B, fill


def needle_delta(S, seed: int = 4):
    """One delta layer that keeps what token B wrote: decays of (nearly) one, B's key aligned with A's query, B's value large, all
    other tokens with small keys -- the read-out at A depends on a write that may be hundreds of tokens back.  One tap, so q, k, v
    are functions of their own token.  Returns (config, weights, A, B, filler tokens)."""
    E, V, H, G, dk, dv = 64, 48, 2, 1, 16, 16
    cfg = S.lerosun_config(E, V, [S.lerosun_delta(H, G, dk, dv, 1, None)])
    w = S.lerosun_weights(cfg, seed)
    rng = np.random.default_rng(seed)
    emb = np.zeros((V, E), dtype=np.float32)
    emb[np.arange(V), np.arange(V)] = 1.0
    w["embed"] = emb
    w["embed.norm"] = np.asarray(1.0 / 8.0, dtype=np.float32)
    w["l0.norm1"] = np.asarray(1.0 / 8.0, dtype=np.float32)
    w["l0.mix.A_log"][:] = -9.0   # decay exp(-exp(-9) softplus(.)) = 1 - O(1e-4) per token
    w["l0.mix.a"][:] = 0.0
    w["l0.mix.dt_bias"][:] = 0.0
    w["l0.mix.b"][:] = -6.0
    w["l0.mix.b"][:, 9] = 6.0      # token B writes with beta near one, the others hardly at all
    for n in ("q.conv", "k.conv", "v.conv"):
        w["l0.mix." + n][:] = 1.0
    A, B = 5, 9
    u = np.abs(rng.standard_normal(dk)).astype(np.float32) + 0.5  # silu keeps positive entries roughly as they are
    keys = (0.02 * rng.standard_normal((dk, E))).astype(np.float32)  # unit vectors afterwards: fillers point anywhere
    keys[:, B] = u
    w["l0.mix.k"] = keys
    w["l0.mix.q"][:, A] = u
    w["l0.mix.v"][:, B] = 5.0 * np.abs(rng.standard_normal(H * dv)).astype(np.float32)
    fill = [t for t in range(V) if t not in (A, B)]
    return cfg, bf16_values(w), A, B, fill
