"""Plain float64 restatement of the Lerosun forward pass (test infrastructure only).

One function per mechanism, no cache, no state object, no batching: every call recomputes the whole sequence with explicit
loops over positions, so windows, the sink, the head mixing and the recurrence are visible in the code.  The product path never
imports this file.

Notation.  x[t] is the residual row of token t (width E).  R(v; g) = v / sqrt(mean(v^2) + eps) * g with ONE number g.
    x <- R(embed[token]; g_embed)
    layer:  x <- x + s1 * mixer(R(x; g1))         x <- x + s2 * ff(R(x; g2))        (s1, s2: vectors of width E; ff optional)
    logits = head R(x; g_final)
A block of layers [start, stop) may run several passes over the same weights; every pass has its own history, nothing else
happens between passes.

Mixer "attention" (H query heads, G key heads, key size d, window W, constant score scale c):
    q = Wq a + bq,  k = Wk a + bk,  v = k  (the key as projected, before it is rotated)
    rotation of the first r entries of every head of q and k: pair (i, i + r/2), angle p * base^(-2i / r) at position p
    e_h(i, j) = c * t_h * <q_i^h, k_j^g(h)>,  g(h) = h // (H / G)
    e'_h(i, j) = sum_m T[h, m] e_m(i, j)                                       (scores mixed over the heads)
    p_h(i, j) = exp(e'_h(i, j)) / (exp(z_h) + sum_{j' visible} exp(e'_h(i, j')))   for 0 <= i - j < W   (z_h: a logit without a key or value)
    o_i^h = sigmoid(<wg_h, a_i>) * sum_j p_h(i, j) v_j^g(h);   out = Wo concat_h o^h

Mixer "delta" (H value heads of size dv, G query/key heads of size d, K-tap causal convolution per channel):
    q, k, v = silu(conv(Wq a)), silu(conv(Wk a)), silu(conv(Wv a));  conv(u)[t] = sum_m w[:, m] u[t - (K - 1) + m], zeros before the start
    q^g <- q^g / sqrt(|q^g|^2 + 1e-6) / sqrt(d),   k^g <- k^g / sqrt(|k^g|^2 + 1e-6)
    beta_h = sigmoid(<wb_h, a>),   gamma_h = exp(-exp(A_h) * softplus(<wa_h, a> + dt_h))
    per head h (g = h // (H / G)), state S [d, dv] starting at zero:
        S <- gamma S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
    y^h = o / sqrt(mean(o^2) + eps) * w_norm * silu(Wg a)^h;   out = Wo concat_h y^h

Feed-forward: Wdown (relu(Wgate a) * (Wup a)).
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np

UNIT_EPS = 1e-6  # inside the root of the delta mixer's unit-vector normalisation


def read_safetensors(path: str) -> dict:
    """name -> float64 array (BF16 / F32 widened exactly; I32 as int64)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, m in head.items():
        if name == "__metadata__":
            continue
        lo, hi = m["data_offsets"]
        raw = blob[lo:hi]
        if m["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif m["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif m["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"dtype {m['dtype']}")
        out[name] = a.reshape(m["shape"])
    return out


def scalar_rms_norm(v: np.ndarray, g: float, eps: float) -> np.ndarray:
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps) * float(g)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rotate_half_partial(x: np.ndarray, heads: int, d: int, r: int, base: float, first_position: int = 0) -> np.ndarray:
    """x [T, heads * d]: entries i and i + r/2 of every head turn by position * base^(-2i / r); entries from r on stay."""
    T = x.shape[0]
    out = x.copy().reshape(T, heads, d)
    src = x.reshape(T, heads, d)
    half = r // 2
    for t in range(T):
        p = first_position + t
        for i in range(half):
            a = p * base ** (-2.0 * i / r)
            c, s = math.cos(a), math.sin(a)
            u, v = src[t, :, i], src[t, :, i + half]
            out[t, :, i] = u * c - v * s
            out[t, :, i + half] = v * c + u * s
    return out.reshape(T, heads * d)


def mixed_head_scores(q_i, k, heads, kv_heads, d, scale, temp, talk):
    """Scores of one query row against key rows k [n, kv_heads * d]: per head scaled, then mixed over the heads.  -> [heads, n]"""
    group = heads // kv_heads
    e = np.zeros((heads, k.shape[0]))
    for h in range(heads):
        g = h // group
        e[h] = (k[:, g * d:(g + 1) * d] @ q_i[h * d:(h + 1) * d]) * scale * temp[h]
    return talk @ e


def sink_softmax(e: np.ndarray, sink: float) -> np.ndarray:
    """Weights of the visible keys; the denominator carries one more term exp(sink) that belongs to no key."""
    m = max(float(e.max()), float(sink))
    w = np.exp(e - m)
    return w / (w.sum() + math.exp(sink - m))


def window_attention(q, k, v, *, heads, kv_heads, d, dv, window, scale, temp, talk, sink):
    """q [T, heads*d] and k [T, kv_heads*d] rotated, v [T, kv_heads*dv] -> [T, heads*dv]; row i sees rows i-window+1 .. i."""
    T = q.shape[0]
    group = heads // kv_heads
    out = np.zeros((T, heads * dv))
    for i in range(T):
        lo = max(0, i - window + 1)
        e = mixed_head_scores(q[i], k[lo:i + 1], heads, kv_heads, d, scale, temp, talk)
        for h in range(heads):
            g = h // group
            out[i, h * dv:(h + 1) * dv] = sink_softmax(e[h], sink[h]) @ v[lo:i + 1, g * dv:(g + 1) * dv]
    return out


def attention_mixer(a, W, pre, m):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = a @ W[pre + "q"].T + W[pre + "q.b"]
    k = a @ W[pre + "k"].T + W[pre + "k.b"]
    v = k  # the values are the keys as projected
    q = rotate_half_partial(q, H, d, m["rot"]["dims"], m["rot"]["base"])
    kr = rotate_half_partial(k, G, d, m["rot"]["dims"], m["rot"]["base"])
    o = window_attention(q, kr, v, heads=H, kv_heads=G, d=d, dv=dv, window=m["mask"]["size"], scale=m["scale"],
                         temp=W[pre + "temp"], talk=W[pre + "talk"], sink=W[pre + "sink"])
    gate = sigmoid(a @ W[pre + "g"].T)  # [T, H]
    o = (o.reshape(-1, H, dv) * gate[:, :, None]).reshape(-1, H * dv)
    return o @ W[pre + "o"].T


def causal_conv(u: np.ndarray, w: np.ndarray) -> np.ndarray:
    """u [T, C], w [C, taps] (last column = the current token's tap): zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    out = np.zeros_like(u)
    for t in range(T):
        for m in range(taps):
            s = t - (taps - 1) + m
            if s >= 0:
                out[t] += w[:, m] * u[s]
    return out


def unit_heads(x: np.ndarray, heads: int, d: int) -> np.ndarray:
    y = x.reshape(-1, heads, d)
    return (y / np.sqrt(np.sum(y * y, axis=-1, keepdims=True) + UNIT_EPS)).reshape(x.shape)


def gated_delta_rule(q, k, v, beta, gamma, *, heads, kv_heads, d, dv):
    """q, k [T, kv_heads*d] (normalised), v [T, heads*dv], beta / gamma [T, heads] -> o [T, heads*dv]."""
    T = q.shape[0]
    group = heads // kv_heads
    out = np.zeros((T, heads * dv))
    for h in range(heads):
        g = h // group
        S = np.zeros((d, dv))
        for t in range(T):
            kt, qt, vt = k[t, g * d:(g + 1) * d], q[t, g * d:(g + 1) * d], v[t, h * dv:(h + 1) * dv]
            S = gamma[t, h] * S
            u = beta[t, h] * (vt - S.T @ kt)
            S = S + np.outer(kt, u)
            out[t, h * dv:(h + 1) * dv] = S.T @ qt
    return out


def delta_mixer(a, W, pre, m, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(a @ W[pre + "q"].T, W[pre + "q.conv"]))
    k = silu(causal_conv(a @ W[pre + "k"].T, W[pre + "k.conv"]))
    v = silu(causal_conv(a @ W[pre + "v"].T, W[pre + "v.conv"]))
    q = unit_heads(q, G, d) * d ** -0.5
    k = unit_heads(k, G, d)
    beta = sigmoid(a @ W[pre + "b"].T)
    gamma = np.exp(-np.exp(W[pre + "A_log"]) * softplus(a @ W[pre + "a"].T + W[pre + "dt_bias"]))
    o = gated_delta_rule(q, k, v, beta, gamma, heads=H, kv_heads=G, d=d, dv=dv).reshape(-1, H, dv)
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps) * W[pre + "norm"]
    y = o.reshape(-1, H * dv) * silu(a @ W[pre + "g"].T)
    return y @ W[pre + "o"].T


def relu_gated_ff(a, W, pre):
    return (np.maximum(a @ W[pre + "gate"].T, 0.0) * (a @ W[pre + "up"].T)) @ W[pre + "down"].T


def layer(x, W, i, spec, eps):
    pre = f"l{i}."
    a = scalar_rms_norm(x, W[pre + "norm1"], eps)
    if spec["type"] == "attention":
        y = attention_mixer(a, W, pre + "mix.", spec["mixer"])
    elif spec["type"] == "delta":
        y = delta_mixer(a, W, pre + "mix.", spec["mixer"], eps)
    else:
        raise ValueError(spec["type"])
    x = x + W[pre + "ls1"] * y
    if spec.get("mlp") is not None:
        if spec["mlp"]["kind"] != "dense":
            raise ValueError(spec["mlp"]["kind"])
        x = x + W[pre + "ls2"] * relu_gated_ff(scalar_rms_norm(x, W[pre + "norm2"], eps), W, pre + "mlp.")
    return x


def layer_runs(cfg) -> list:
    """Layer indices in execution order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return list(range(n))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))


def forward(cfg, W, tokens, want_layers: bool = False):
    """Logits [T, vocab] (and the residual stream after every layer run) of one whole sequence."""
    eps = cfg["norm"]["eps"]
    x = scalar_rms_norm(W["embed"][np.asarray(tokens)], W["embed.norm"], eps)
    trace = []
    for i in layer_runs(cfg):
        x = layer(x, W, i, cfg["layers"][i], eps)
        trace.append(x.copy())
    logits = scalar_rms_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, np.stack(trace)) if want_layers else logits


def load_dir(path: str):
    with open(f"{path}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{path}/model.safetensors")
