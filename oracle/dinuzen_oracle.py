"""Plain float64 restatement of the Dinuzen forward pass (test infrastructure only).

One function per mechanism, no cache, no state object, no batching: every call recomputes the whole sequence, recurrences run
token by token in explicit loops.  The product path never imports this file.

Notation.  x[t] is the residual row of token t (width E).  GN(v; w) splits v into `groups` equal consecutive parts, divides
each part by sqrt(mean(part^2) + eps) and multiplies the whole by w.
    X_0 = embed[token]
    layer i reads x (the depth average below; x = X_0 for layer 0):
        h[t] = x[t] + (x[t-1] - x[t]) * shift            (x[-1] = 0: the token shift; only the mixer reads h)
        x <- x + ls1 * GN(mixer(h); norm1)
        x <- x + ls2 * GN(ff(x); norm2)                   (when the layer has a feed-forward)
        X_(i+1) = x;   x <- sum_{j <= i+1} dwa[j] X_j     (depth average: what the next layer, or the output, reads)
    logits = head GN(x; final.norm)

Mixer "rglru" (width W, `blocks` diagonal blocks, K-tap causal convolution per channel):
    y = gelu_tanh(Wy h + by);  u = conv(Wx h + bx) + bc
    per block b: r_b = sigmoid(Ra[b] u_b + ra_b[b]),  i_b = sigmoid(Ri[b] u_b + ri_b[b])
    a = exp(-8 r softplus(lam));  S[t] = a S[t-1] + sqrt(1 - a^2) (i u),  S[-1] = 0;  out = Wo (S y)

Mixer "mamba2" (H heads of size P, state size N, G groups):
    Win h = [z (H P) | x (H P) | B (G N) | C (G N) | dt (H)];  [x | B | C] <- silu(conv([x | B | C]) + bc)
    dt <- softplus(dt + dt_bias);  per head h, group g = h // (H / G), state S [N, P] from zero:
        S <- exp(-exp(A_log_h) dt_h) S + dt_h B_g x_h^T;   y_h = S^T C_g + D_h x_h
    out = Wo (GNn(y * silu(z); norm)),  GNn = the same grouped norm with norm_groups parts

Mixer "attention" (H heads, G key/value heads, two score maps per head of key size d, value size dv):
    q = Wq h as [H][2][d],  k = Wk h as [G][2][d],  v = Wv h as [G][dv]
    every [d] slice of q and k:  RMS norm over d times q.norm / k.norm, then the rotation of its first `dims` entries in pairs
    (2i, 2i+1) by the angle p f_i (frequencies blended between f_i and f_i / factor along a ramp over i; cos and sin times
    0.1 ln(factor) + 1)
    e_m(t, j) = cap tanh(scale <q_t^{h,m}, k_j^{g,m}> / cap),  j <= t;   a_m = softmax_j(e_m) v^g      (m = 1, 2)
    lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff;   o = a_1 - lambda a_2;   o <- o / sqrt(mean(o^2) + eps) * (1 - diff)
    out = Wo concat_h o.  With kv_from = j the layer has no Wk, Wv, k.norm: it reads layer j's normalised, rotated keys and its values.

Feed-forward "dense": Wdown gelu_erf(Wup x).
Feed-forward "moe": z = Wrouter x over X experts + I identity experts;  s = softmax(z);  the `top` largest of s + correction are
    chosen;  w = s[chosen] / (sum s[chosen] + 1e-20) * scale;  expert e < X: Wdown (silu(Wgate x) * (Wup x)),  e >= X: x itself;
    out = sum w_e expert_e(x) + sigmoid(<sg, x>) * shared(x),  shared of the same gated form.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


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
            raise ValueError(f"{name}: dtype {m['dtype']}")
        out[name] = a.reshape(m["shape"])
    return out


# ---- elementwise -------------------------------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu_erf(z):
    return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))


# ---- norms, shift, depth average ---------------------------------------------------------------------------------------
def group_rms_norm(v, w, groups: int, eps: float):
    """v [..., n]: `groups` consecutive parts, each divided by the RMS of that part alone; the whole times w (None: no weight)."""
    n = v.shape[-1]
    p = v.reshape(v.shape[:-1] + (groups, n // groups))
    p = p / np.sqrt((p * p).mean(-1, keepdims=True) + eps)
    out = p.reshape(v.shape)
    return out if w is None else out * w


def token_shift(x, shift):
    """x [T, E]: h[t] = x[t] + (x[t-1] - x[t]) * shift with x[-1] = 0."""
    prev = np.vstack([np.zeros((1, x.shape[1])), x[:-1]])
    return x + (prev - x) * shift


def depth_average(streams: list, dwa):
    """sum_j dwa[j] * streams[j]."""
    return sum(dwa[j] * streams[j] for j in range(len(streams)))


def causal_conv(u, w, b):
    """u [T, C], w [C, K] (last column = current token), zeros before the start, bias b [C]."""
    T, C = u.shape
    K = w.shape[1]
    pad = np.vstack([np.zeros((K - 1, C)), u])
    out = np.zeros((T, C))
    for m in range(K):
        out += pad[m:m + T] * w[:, m]
    return out + b


# ---- rotation ----------------------------------------------------------------------------------------------------------
def rope_frequencies(rot: dict):
    """(frequencies [dims / 2], magnitude factor of cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(v, positions, rot: dict):
    """v [T, ..., d]: entries (2i, 2i+1), i < dims / 2, of the last axis turn by positions[t] * f_i; the rest pass unchanged."""
    f, mag = rope_frequencies(rot)
    dims = int(rot["dims"])
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    shape = (v.shape[0],) + (1,) * (v.ndim - 2) + (dims // 2,)
    c, s = (np.cos(ang) * mag).reshape(shape), (np.sin(ang) * mag).reshape(shape)
    out = v.copy()
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---- mixers ------------------------------------------------------------------------------------------------------------
def attention_keys_values(h, w: dict, pre: str, m: dict, eps: float):
    """Normalised, rotated keys [T, G, 2, d] and values [T, G, dv] of a layer with key/value projections of its own."""
    T = h.shape[0]
    G, d, dv = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    k = (h @ w[pre + "k"].T).reshape(T, G, 2, d)
    k = group_rms_norm(k, w[pre + "k.norm"], 1, eps)
    k = rotate_interleaved(k, np.arange(T), m["rot"])
    v = (h @ w[pre + "v"].T).reshape(T, G, dv)
    return k, v


def diff_lambda(w: dict, pre: str, diff: float) -> float:
    return math.exp(float(np.sum(w[pre + "lq1"] * w[pre + "lk1"]))) - math.exp(float(np.sum(w[pre + "lq2"] * w[pre + "lk2"]))) + diff


def softcap(e, cap: float):
    return cap * np.tanh(e / cap)


def mixer_attention(h, w: dict, pre: str, m: dict, eps: float, kv):
    """kv = (keys, values) as attention_keys_values returns them (this layer's own or another layer's)."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    q = (h @ w[pre + "q"].T).reshape(T, H, 2, d)
    q = group_rms_norm(q, w[pre + "q.norm"], 1, eps)
    q = rotate_interleaved(q, np.arange(T), m["rot"])
    k, v = kv
    lam = diff_lambda(w, pre, diff)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        maps = []
        for mp in range(2):
            e = (q[:, hd, mp] @ k[:, g, mp].T) * float(m["scale"])
            if m.get("softcap"):
                e = softcap(e, float(m["softcap"]))
            e = np.where(np.tril(np.ones((T, T), dtype=bool)), e, -np.inf)
            p = np.exp(e - e.max(-1, keepdims=True))
            p /= p.sum(-1, keepdims=True)
            maps.append(p @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, hd] = o / np.sqrt((o * o).mean(-1, keepdims=True) + eps) * (1.0 - diff)
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def rglru_gates(u, w: dict, pre: str, blocks: int):
    """(r, i) [T, W]: per diagonal block sigmoid(R[b] u_b + bias[b])."""
    T, W = u.shape
    ub = u.reshape(T, blocks, W // blocks)
    r = sigmoid(np.einsum("boi,tbi->tbo", w[pre + "ra"], ub) + w[pre + "ra.b"]).reshape(T, W)
    i = sigmoid(np.einsum("boi,tbi->tbo", w[pre + "ri"], ub) + w[pre + "ri.b"]).reshape(T, W)
    return r, i


def rglru_scan(u, r, i, lam):
    """S[t] = a S[t-1] + sqrt(1 - a^2) (i u) with a = exp(-8 r softplus(lam)), from S = 0; token 0 runs the same update as every other."""
    T, W = u.shape
    a = np.exp(-8.0 * r * softplus(lam))
    S = np.zeros(W)
    out = np.zeros((T, W))
    for t in range(T):
        S = a[t] * S + np.sqrt(1.0 - a[t] ** 2) * (i[t] * u[t])
        out[t] = S
    return out


def mixer_rglru(h, w: dict, pre: str, m: dict):
    y = gelu_tanh(h @ w[pre + "y"].T + w[pre + "y.b"])
    u = causal_conv(h @ w[pre + "x"].T + w[pre + "x.b"], w[pre + "conv"], w[pre + "conv.b"])
    r, i = rglru_gates(u, w, pre, int(m["blocks"]))
    S = rglru_scan(u, r, i, w[pre + "lam"])
    return (S * y) @ w[pre + "o"].T


def ssd_scan(x, B, C, dt, A_log, D, groups: int):
    """x [T, H, P], B, C [T, G, N], dt [T, H] (after softplus): y [T, H, P] of the state-space recurrence, state [N, P] per head."""
    T, H, P = x.shape
    N = B.shape[2]
    y = np.zeros((T, H, P))
    for hd in range(H):
        g = hd // (H // groups)
        S = np.zeros((N, P))
        for t in range(T):
            S = math.exp(-math.exp(A_log[hd]) * dt[t, hd]) * S + dt[t, hd] * np.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + D[hd] * x[t, hd]
    return y


def mixer_mamba2(h, w: dict, pre: str, m: dict, eps: float):
    T = h.shape[0]
    H, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * P
    p = h @ w[pre + "in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[pre + "dt_bias"])
    y = ssd_scan(x, B, C, dt, w[pre + "A_log"], w[pre + "D"], G).reshape(T, inner)
    y = group_rms_norm(y * silu(z), w[pre + "norm"], int(m["norm_groups"]), eps)
    return y @ w[pre + "o"].T


# ---- feed-forward ------------------------------------------------------------------------------------------------------
def ff_dense(x, w: dict, pre: str):
    return gelu_erf(x @ w[pre + "up"].T) @ w[pre + "down"].T


def gated_expert(x, w: dict, pre: str):
    return (silu(x @ w[pre + "gate"].T) * (x @ w[pre + "up"].T)) @ w[pre + "down"].T


def moe_route(x, w: dict, pre: str, router: dict):
    """(ids [T, top], weights [T, top]); ids >= experts are identity experts."""
    z = x @ w[pre + "router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    choice = s + w[pre + "correction"]
    top = int(router["top"])
    ids = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    sc = np.take_along_axis(s, ids, -1)
    wts = sc / (sc.sum(-1, keepdims=True) + 1e-20) * float(router["scale"])
    return ids, wts


def ff_moe(x, w: dict, pre: str, mlp: dict):
    router = mlp["router"]
    X = int(router["experts"])
    ids, wts = moe_route(x, w, pre, router)
    out = np.zeros_like(x)
    for t in range(x.shape[0]):
        for e, wt in zip(ids[t], wts[t]):
            out[t] += wt * (gated_expert(x[t:t + 1], w, f"{pre}e{e}.")[0] if e < X else x[t])
    if mlp.get("shared"):
        out += sigmoid(x @ w[pre + "shared.sg"].T) * gated_expert(x, w, pre + "shared.")
    return out


# ---- model -------------------------------------------------------------------------------------------------------------
def forward(cfg: dict, w: dict, tokens, return_layers: bool = False, on_moe_input=None):
    """Logits [T, vocab] of the whole sequence (and, optionally, the residual stream after every layer [layers, T, E]).
    on_moe_input(layer, x) is called with what every mixture of experts reads."""
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"])
    x = w["embed"][np.asarray(tokens)]
    streams = [x]
    kv = {}
    trace = []
    for i, lc in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", lc["mixer"]
        h = token_shift(x, w[pre + "shift"])
        if lc["type"] == "attention":
            if m.get("kv_from") is None:
                kv[i] = attention_keys_values(h, w, pre + "mix.", m, eps)
            y = mixer_attention(h, w, pre + "mix.", m, eps, kv[i if m.get("kv_from") is None else int(m["kv_from"])])
        elif lc["type"] == "rglru":
            y = mixer_rglru(h, w, pre + "mix.", m)
        elif lc["type"] == "mamba2":
            y = mixer_mamba2(h, w, pre + "mix.", m, eps)
        else:
            raise ValueError(lc["type"])
        x = x + w[pre + "ls1"] * group_rms_norm(y, w[pre + "norm1"], groups, eps)
        mlp = lc.get("mlp")
        if mlp is not None:
            if on_moe_input is not None and mlp["kind"] == "moe":
                on_moe_input(i, x)
            y = ff_dense(x, w, pre + "mlp.") if mlp["kind"] == "dense" else ff_moe(x, w, pre + "mlp.", mlp)
            x = x + w[pre + "ls2"] * group_rms_norm(y, w[pre + "norm2"], groups, eps)
        streams.append(x)
        x = depth_average(streams, w[pre + "dwa"])
        trace.append(x)
    logits = group_rms_norm(x, w["final.norm"], groups, eps) @ w["head"].T
    return (logits, np.stack(trace)) if return_layers else logits


def load_dir(path: str):
    with open(f"{path}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{path}/model.safetensors")
