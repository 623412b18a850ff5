"""Mopitar, plainly: numpy in float64, one function per mechanism, a token at a time wherever the
design carries a state.  Shares no code with the package (own safetensors reader, own config walk).
Slow on purpose: attention is a loop over queries and keys' masks are written out as the rule says.

Notation: T tokens of ONE sequence from its first token, width W; an attention with H query heads
on G key/value heads, key size D, value size V.
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


def rms_divide(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def tanh_norm(x, alpha, w, b):
    """The norm without statistics: tanh(alpha x) w + b, alpha one number."""
    return np.tanh(float(alpha) * x) * w + b


# ---- rotation ------------------------------------------------------------------------------
def rotation_frequencies(rot):
    """(frequency of every pair, multiplier of cos and sin) from a mixer's ``rot`` entry."""
    r, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / r) for i in range(r // 2)])
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_that_turns(times):
        return r * math.log(original / (2.0 * math.pi * times)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_that_turns(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_that_turns(float(sc["slow"]))), r - 1)
    ramp = np.clip((np.arange(r // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x, positions, rot):
    """x [T, heads, D]: entries 2i and 2i+1 of the first rot.dims of every head turn together by
    position * f_i; the rest stay."""
    if rot is None:
        return x
    f, mult = rotation_frequencies(rot)
    r = int(rot["dims"])
    out = x.copy()
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]          # [T, r/2]
    c, s = (np.cos(ang) * mult)[:, None, :], (np.sin(ang) * mult)[:, None, :]
    u, v = x[..., 0:r:2], x[..., 1:r:2]
    out[..., 0:r:2] = u * c - v * s
    out[..., 1:r:2] = v * c + u * s
    return out


# ---- attention over prepared queries, keys, values ----------------------------------------------
def visible(i, j, window=0, keep_first=0):
    """May the query at position i see the key at position j?"""
    if j > i:
        return False
    if window <= 0:
        return True
    return i - j < window or j < keep_first


def visible_keys(i, window=0, keep_first=0):
    """The positions that ``visible`` lets the query at position i see, in ascending order."""
    j = np.arange(i + 1)
    if window <= 0:
        return j
    return j[(i - j < window) | (j < keep_first)]


def attend(q, k, v, scale, *, softcap=0.0, sink=None, window=0, keep_first=0):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V].  Scores (q . k) scale, optionally capped as
    cap tanh(s / cap); softmax over the visible keys, with exp(sink_h) as one more term of the
    denominator that has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = visible_keys(i, window, keep_first)
            s = (k[js, g, :] @ q[i, h, :]) * scale
            if softcap:
                s = softcap * np.tanh(s / softcap)
            m = s.max() if sink is None else max(s.max(), float(sink[h]))
            e = np.exp(s - m)
            den = e.sum() + (math.exp(float(sink[h]) - m) if sink is not None else 0.0)
            out[i, h] = (e / den) @ v[js, g, :]
    return out


def project_heads(h, w, heads):
    return (h @ w.T).reshape(h.shape[0], heads, -1)


# ---- the three mixers -----------------------------------------------------------------------------
def attention_mixer(h, m, t, pre, eps, borrowed=None):
    """Capped attention with a learned sink.  Returns (output [T, W], (k, v) as a cache would hold
    them).  ``borrowed``: another layer's (k, v); then this layer has no key and value matrices."""
    T = h.shape[0]
    H, G = int(m["heads"]), int(m["kv_heads"])
    pos = np.arange(T)
    q = rotate_neighbours(project_heads(h, t[pre + "q"], H), pos, m.get("rot"))
    if borrowed is None:
        k = rotate_neighbours(project_heads(h, t[pre + "k"], G), pos, m.get("rot"))
        v = project_heads(h, t[pre + "v"], G)
    else:
        k, v = borrowed
    o = attend(q, k, v, float(m["scale"]), softcap=float(m.get("softcap") or 0.0), sink=t.get(pre + "sink"))
    return o.reshape(T, -1) @ t[pre + "o"].T, (k, v)


def difference_lambda(t, pre, diff):
    return math.exp(float(t[pre + "lq1"] @ t[pre + "lk1"])) - math.exp(float(t[pre + "lq2"] @ t[pre + "lk2"])) + diff


def difference_mixer(h, m, t, pre, eps):
    """Two attention maps per head over one set of values, the second subtracted."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    diff = float(m["diff"])
    pos = np.arange(T)
    q = project_heads(h, t[pre + "q"], H * 2)                       # head by head: map 1, map 2
    k = project_heads(h, t[pre + "k"], G * 2)
    v = project_heads(h, t[pre + "v"], G)
    q = rotate_neighbours(rms_divide(q, eps) * t[pre + "q.norm"], pos, m.get("rot"))
    k = rotate_neighbours(rms_divide(k, eps) * t[pre + "k.norm"], pos, m.get("rot"))
    mask = m.get("mask") or {}
    maps = []
    for which in (0, 1):
        maps.append(attend(q[:, which::2, :], k[:, which::2, :], v, float(m["scale"]),
                           window=int(mask.get("size") or 0), keep_first=int(mask.get("keep_first") or 0)))
    lam = difference_lambda(t, pre, diff)
    o = maps[0] - lam * maps[1]
    o = rms_divide(o, eps) * (1.0 - diff)
    return o.reshape(T, -1) @ t[pre + "o"].T


def gated_unit_attention(h, m, t, pre, eps):
    """The attention branch of the two-branch mixer: q and k unit-normed after the rotation, capped
    scores, every head times the sigmoid of its own gate."""
    T = h.shape[0]
    H, G = int(m["heads"]), int(m["kv_heads"])
    pos = np.arange(T)
    q = rms_divide(rotate_neighbours(project_heads(h, t[pre + "q"], H), pos, m.get("rot")), eps)
    k = rms_divide(rotate_neighbours(project_heads(h, t[pre + "k"], G), pos, m.get("rot")), eps)
    v = project_heads(h, t[pre + "v"], G)
    o = attend(q, k, v, float(m["scale"]), softcap=float(m.get("softcap") or 0.0))
    o = o * sigmoid(h @ t[pre + "g"].T)[:, :, None]
    return o.reshape(T, -1) @ t[pre + "o"].T


def causal_taps(x, w, b):
    """x [T, C], w [C, taps] (last column: the current token), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = np.vstack([np.zeros((taps - 1, C)), x])
    out = np.zeros((T, C))
    for i in range(T):
        out[i] = (padded[i:i + taps].T * w).sum(axis=1) + b
    return out


def selective_scan(h, m, t, pre):
    """The state-space branch: a state S [inner, state] per sequence, from zero, a token at a time."""
    T = h.shape[0]
    inner, N, R = int(m["inner"]), int(m["state"]), int(m["dt_rank"])
    xz = h @ t[pre + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_taps(x, t[pre + "conv"], t[pre + "conv.b"]))
    p = x @ t[pre + "x"].T
    dt = softplus(p[:, :R] @ t[pre + "dt"].T + t[pre + "dt.b"])       # [T, inner]
    B, C = p[:, R:R + N], p[:, R + N:R + 2 * N]
    A = -np.exp(t[pre + "A_log"])                                     # [inner, N]
    S = np.zeros((inner, N))
    y = np.zeros((T, inner))
    for i in range(T):
        S = np.exp(dt[i][:, None] * A) * S + (dt[i] * x[i])[:, None] * B[i][None, :]
        y[i] = S @ C[i] + t[pre + "D"] * x[i]
    return (y * silu(z)) @ t[pre + "o"].T


def two_branch_mixer(h, m, t, pre, eps):
    left = gated_unit_attention(h, m["left"], t, pre + "left.", eps)
    right = selective_scan(h, m["right"], t, pre + "right.")
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---- feed-forwards ------------------------------------------------------------------------------
def squared_relu_ff(h, t, pre):
    return np.square(np.maximum(h @ t[pre + "up"].T, 0.0)) @ t[pre + "down"].T


def gated_ff(h, t, pre):
    return (silu(h @ t[pre + "gate"].T) * (h @ t[pre + "up"].T)) @ t[pre + "down"].T


def route(z, top, groups, keep):
    """Router logits z [E] of one token -> (chosen experts, their weights).  Scores are sigmoids;
    experts in ``groups`` equal groups of neighbours, a group scored by the sum of its two best,
    only the ``keep`` best groups stay eligible; the ``top`` best of those, weights = scores over
    their sum (+ 1e-20)."""
    s = sigmoid(z)
    E = len(s)
    per = E // groups
    gs = np.array([np.sort(s[g * per:(g + 1) * per])[::-1][:2].sum() for g in range(groups)])
    kept = np.argsort(-gs, kind="stable")[:keep]
    ok = np.zeros(E, dtype=bool)
    for g in kept:
        ok[g * per:(g + 1) * per] = True
    masked = np.where(ok, s, -np.inf)
    chosen = np.argsort(-masked, kind="stable")[:top]
    w = s[chosen]
    return chosen, w / (w.sum() + 1e-20)


def routed_ff(h, mlp, t, pre):
    r = mlp["router"]
    E, top = int(r["experts"]), int(r["top"])
    g = r.get("groups") or {}
    groups, keep = int(g.get("count") or 1), int(g.get("keep") or g.get("count") or 1)
    out = np.zeros_like(h)
    z = h @ t[pre + "router"].T
    for i in range(h.shape[0]):
        chosen, w = route(z[i], top, groups, keep)
        for e, we in zip(chosen, w):
            out[i] += we * gated_ff(h[i:i + 1], t, f"{pre}e{e}.")[0]
    if mlp.get("shared") is not None:
        out += gated_ff(h, t, pre + "shared.")
    return out


def feed_forward(h, mlp, t, pre):
    if mlp is None:
        return np.zeros_like(h)
    if mlp["kind"] == "dense":
        return squared_relu_ff(h, t, pre)
    if mlp["kind"] == "moe":
        return routed_ff(h, mlp, t, pre)
    raise ValueError(mlp["kind"])


# ---- the model --------------------------------------------------------------------------------------
def routing_margin(z, top, groups, keep):
    """How clear one token's choice is: the smaller of (last group kept - best group left out) and (last
    expert chosen - best eligible expert left out), each as a fraction of the larger of the two scores;
    inf where nothing is left out."""
    s = sigmoid(z)
    E = len(s)
    per = E // groups
    gs = np.array([np.sort(s[g * per:(g + 1) * per])[::-1][:2].sum() for g in range(groups)])
    order = np.argsort(-gs, kind="stable")
    worst = np.inf
    if keep < groups:
        worst = (gs[order[keep - 1]] - gs[order[keep]]) / gs[order[keep - 1]]
    ok = np.concatenate([s[g * per:(g + 1) * per] for g in sorted(order[:keep])])
    ranked = -np.sort(-ok)
    if top < len(ranked):
        worst = min(worst, (ranked[top - 1] - ranked[top]) / ranked[top - 1])
    return worst


def forward(cfg, t, tokens, layers_out=None, watch=None):
    """Logits [T, vocab] of one sequence's tokens from its first.  ``layers_out``: a list that gets the
    stream after every layer.  ``watch(i, h)``: called with every layer's normed rows."""
    eps = float(cfg["norm"]["eps"])
    x = t["embed"][np.asarray(tokens)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = tanh_norm(x, t[pre + "norm1.alpha"], t[pre + "norm1"], t[pre + "norm1.b"])
        if watch is not None:
            watch(i, h)
        m = layer["mixer"]
        kind = layer["type"]
        if kind == "attention":
            src = m.get("kv_from")
            y, kept[i] = attention_mixer(h, m, t, pre + "mix.", eps, None if src is None else kept[int(src)])
        elif kind == "attention_2":
            y = difference_mixer(h, m, t, pre + "mix.", eps)
        elif kind == "parallel":
            y = two_branch_mixer(h, m, t, pre + "mix.", eps)
        else:
            raise ValueError(kind)
        y = y * t[pre + "ls1"]
        if layer.get("mlp") is not None:
            y = y + feed_forward(h, layer["mlp"], t, pre + "mlp.") * t[pre + "ls2"]
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    h = tanh_norm(x, t["final.norm.alpha"], t["final.norm"], t["final.norm.b"])
    return h @ t["head"].T


def load(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")
