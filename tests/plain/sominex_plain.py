"""Sominex, plainly: numpy in float64, one function per mechanism, a token at a time wherever the
design carries a state.  Shares no code with the package (own safetensors reader, own config walk).
Slow on purpose: every recurrence is the loop that defines it and attention is a loop over queries.

Notation: T tokens, width W; a mixer with H heads of key size D and value size V.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# ---- files -------------------------------------------------------------------------------
def read_safetensors(path) -> dict:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = raw[8 + n + a:8 + n + b]
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4")
        elif info["dtype"] == "I32":
            arr = np.frombuffer(buf, dtype="<i4")
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        out[name] = arr.reshape(info["shape"]).astype(np.float64 if info["dtype"] != "I32" else np.int64)
    return out


# ---- small functions -----------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def logsigmoid(z):
    return -np.logaddexp(0.0, -z)


def rms_divide(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


# ---- token shift -----------------------------------------------------------------------------
def token_shift(h, mu):
    """h [T, W] of ONE sequence from its first token: row t becomes h_t + (h_{t-1} - h_t) * mu,
    with zeros in front of the first row; the rows mixed in are the unshifted ones."""
    prev = np.vstack([np.zeros((1, h.shape[1])), h[:-1]])
    return h + (prev - h) * mu[None, :]


# ---- rotation with stretched frequencies ---------------------------------------------------------
def stretched_frequencies(base, dims, scaling):
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` (factor, original, fast, slow) the slow
    turning pairs are divided by ``factor`` along a linear ramp between two pair indices.  Returns the
    frequencies and the number that multiplies cos and sin."""
    half = dims // 2
    i = np.arange(half, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns):            # the pair that makes ``turns`` turns over ``original`` positions
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, freqs, mult):
    """x [T, heads, D]: entries i and i + r/2 of every head (r = 2 len(freqs)) turn by p f_i, cos and
    sin times ``mult``; entries from r on pass."""
    out = x.copy()
    half = len(freqs)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]
    c, s = (np.cos(ang) * mult)[:, None, :], (np.sin(ang) * mult)[:, None, :]
    a, b = x[..., :half], x[..., half:2 * half]
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = b * c + a * s
    return out


# ---- attention: a window of tokens and, in front of it, means of whole blocks ---------------------
def window_pool_attention(q, k, v, scale, window, pool, round_cache=None):
    """q [T, H, D], k [T, G, D], v [T, G, V] of ONE sequence from its first token (k turned, v normed:
    as they are kept).  Query i sees the tokens j with 0 <= i - j < window and, for every block b of
    ``pool`` tokens with b pool + pool - 1 <= i - window, the mean key and the mean value of the
    block; one softmax over both.  ``round_cache``: a function applied to what is kept (keys, values
    and the means), to follow a store of fewer bits."""
    T, H, D = q.shape
    G, V = k.shape[1], v.shape[2]
    keep = round_cache or (lambda a: a)
    k, v = keep(k), keep(v)
    out = np.zeros((T, H, V))
    whole = T // pool if pool > 0 else 0
    if whole:
        mk = keep(np.stack([k[b * pool:(b + 1) * pool].mean(axis=0) for b in range(whole)]))      # [blocks, G, D]
        mv = keep(np.stack([v[b * pool:(b + 1) * pool].mean(axis=0) for b in range(whole)]))
    for i in range(T):
        lo = max(0, i - window + 1)
        n_blocks = max(0, (i - window + 1) // pool) if pool > 0 else 0
        for h in range(H):
            g = h // (H // G)
            keys, vals = k[lo:i + 1, g], v[lo:i + 1, g]
            if n_blocks:
                keys, vals = np.vstack([keys, mk[:n_blocks, g]]), np.vstack([vals, mv[:n_blocks, g]])
            s = (keys @ q[i, h]) * scale
            p = np.exp(s - s.max())
            out[i, h] = (p / p.sum()) @ vals
    return out


def attention_mixer(h, w, pre, m, eps, positions=None, round_cache=None):
    """The whole mixer on ONE sequence's rows from its first token."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).reshape(T, H, D)
    k = (h @ w[pre + "k"].T).reshape(T, G, D)
    v = (h @ w[pre + "v"].T).reshape(T, G, V)
    rot = m.get("rot")
    if rot:
        f, mult = stretched_frequencies(float(rot["base"]), int(rot["dims"]), rot.get("scaling"))
        pos = np.arange(T) if positions is None else positions
        q, k = rotate_half(q, pos, f, mult), rotate_half(k, pos, f, mult)
    v = rms_divide(v, eps)
    mask = m.get("mask") or {}
    o = window_pool_attention(q, k, v, float(m["scale"]), int(mask.get("size") or T + 1), int(mask.get("pool") or 0),
                              round_cache)
    return o.reshape(T, H * V) @ w[pre + "o"].T


# ---- state-space mixer with a scalar decay per head ------------------------------------------------
def causal_conv(x, w, b):
    """x [T, C] of ONE sequence from its first token; w [C, taps], the last column the current
    token's; zeros in front."""
    T, C = x.shape
    taps = w.shape[1]
    xp = np.vstack([np.zeros((taps - 1, C)), x])
    out = np.zeros((T, C))
    for t in range(T):
        out[t] = (xp[t:t + taps] * w.T).sum(axis=0) + b
    return out


def ssd_scan(x, B, C, dt, A_log, Dskip):
    """x [T, H, V], B and C [T, G, N], dt [T, H] (after softplus).  Per head
    S = exp(-exp(A_log) dt) S + dt B x^T (S [N, V]); y = S^T C + D x."""
    T, H, V = x.shape
    G, N = B.shape[1], B.shape[2]
    S = np.zeros((H, N, V))
    y = np.zeros((T, H, V))
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = math.exp(-math.exp(A_log[h]) * dt[t, h]) * S[h] + dt[t, h] * np.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g] + Dskip[h] * x[t, h]
    return y


def mamba2_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    p = h @ w[pre + "in"].T
    z, xBC, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xBC = silu(causal_conv(xBC, w[pre + "conv"], w[pre + "conv.b"]))
    x = xBC[:, :inner].reshape(T, H, V)
    B = xBC[:, inner:inner + G * N].reshape(T, G, N)
    C = xBC[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[pre + "dt_bias"][None, :])
    y = ssd_scan(x, B, C, dt, w[pre + "A_log"], w[pre + "D"]).reshape(T, inner)
    y = y * silu(z)
    parts = int(m["norm_groups"])
    y = rms_divide(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[pre + "norm"][None, :]
    return y @ w[pre + "o"].T


# ---- matrix memory with exponential gates and a running maximum -------------------------------------
def mlstm_scan(q, k, v, i_gate, f_gate):
    """q, k [T, H, D], v [T, H, V], log gates [T, H].  m = max(f + m, i) from m = 0;
    S = exp(f + m_old - m) S + exp(i - m) k v^T; n likewise with k; o = S^T q / (max(|n.q|, exp(-m)) + 1e-6)."""
    T, H, D = q.shape
    V = v.shape[2]
    S, n, m = np.zeros((H, D, V)), np.zeros((H, D)), np.zeros(H)
    o = np.zeros((T, H, V))
    for t in range(T):
        for h in range(H):
            m_new = max(f_gate[t, h] + m[h], i_gate[t, h])
            a, b = math.exp(f_gate[t, h] + m[h] - m_new), math.exp(i_gate[t, h] - m_new)
            S[h] = a * S[h] + b * np.outer(k[t, h], v[t, h])
            n[h] = a * n[h] + b * k[t, h]
            m[h] = m_new
            o[t, h] = S[h].T @ q[t, h] / (max(abs(n[h] @ q[t, h]), math.exp(-m_new)) + 1e-6)
    return o


def mlstm_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[pre + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[pre + "k"].T).reshape(T, H, D)
    v = (h @ w[pre + "v"].T).reshape(T, H, V)
    i_gate = cap * np.tanh((h @ w[pre + "i"].T + w[pre + "i.b"][None, :]) / cap)
    f_gate = logsigmoid(cap * np.tanh((h @ w[pre + "f"].T + w[pre + "f.b"][None, :]) / cap))
    o = rms_divide(mlstm_scan(q, k, v, i_gate, f_gate), eps).reshape(T, H * V)
    o = o * w[pre + "norm"][None, :] * sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


# ---- feed-forwards ------------------------------------------------------------------------------
def capped_glu(h, w, pre, limit):
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    g = np.minimum(h @ w[pre + "gate"].T, limit)
    u = np.clip(h @ w[pre + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def silu_glu(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w_router, top, scale):
    """Softmax over all experts; the ``top`` largest scores (ties to the lower index); their scores
    times ``scale`` are the weights.  Returns (indices [T, top], weights [T, top], scores [T, E])."""
    z = h @ w_router.T
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s /= s.sum(axis=-1, keepdims=True)
    idx = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return idx, np.take_along_axis(s, idx, axis=-1) * scale, s


def routed_experts(h, w, pre, mlp):
    r = mlp["router"]
    idx, wt, _ = route(h, w[pre + "router"], int(r["top"]), float(r["scale"]))
    out = np.zeros((h.shape[0], w[pre + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, a in zip(idx[t], wt[t]):
            out[t] += a * silu_glu(h[t:t + 1], w, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out += silu_glu(h, w, pre + "shared.")
    return out


def feed_forward(h, w, pre, mlp):
    if mlp is None:
        return np.zeros_like(h)
    if mlp["kind"] == "dense":
        return capped_glu(h, w, pre, float(mlp["limit"]))
    if mlp["kind"] == "moe":
        return routed_experts(h, w, pre, mlp)
    raise ValueError(mlp["kind"])


# ---- the model ------------------------------------------------------------------------------------
def mixer(kind, hs, w, pre, m, eps, round_cache=None):
    if kind == "attention":
        return attention_mixer(hs, w, pre, m, eps, round_cache=round_cache)
    if kind == "mamba2":
        return mamba2_mixer(hs, w, pre, m, eps)
    if kind == "mlstm":
        return mlstm_mixer(hs, w, pre, m, eps)
    raise ValueError(kind)


def forward(cfg, w, tokens, layers_out=None, round_cache=None):
    """Logits [T, vocab] of ONE sequence from its first token.  ``layers_out``: a list that gets the
    stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_divide(x, eps) * w[p + "norm1"][None, :]
        hs = token_shift(h, w[p + "shift"])
        x = x + (mixer(layer["type"], hs, w, p + "mix.", layer["mixer"], eps, round_cache)
                 + feed_forward(h, w, p + "mlp.", layer.get("mlp")))
        if layers_out is not None:
            layers_out.append(x.copy())
    return (rms_divide(x, eps) * w["final.norm"][None, :]) @ w["head"].T


def load(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")
