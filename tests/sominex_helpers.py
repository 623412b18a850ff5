"""Shared by the Sominex tests: small configurations that differ from one another in every size and
option, weights at a scale where every mechanism matters, model folders in temporary places, token
sequences whose routing choices are clear, and the plain implementation's results."""
from __future__ import annotations

import functools
from pathlib import Path

import numpy as np

from helpers import tmp_root
from plain import sominex_plain as SP
from senotar_helpers import to_bf16_values, write_folder


def _attention(heads, kv, dim, vdim, scale, window=None, pool=None, rot=None, scaling=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if window is not None:
        m["mask"] = dict(size=window) if pool is None else dict(size=window, pool=pool)
    if rot is not None:
        m["rot"] = dict(dims=rot[0], base=rot[1])
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def _mamba2(heads, groups, state, vdim, conv, norm_groups):
    return dict(heads=heads, groups=groups, state=state, vdim=vdim, conv=conv, norm_groups=norm_groups)


def _mlstm(heads, dim, vdim, cap):
    return dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap)


def _dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


def _moe(ff, experts, top, scale, shared=None):
    m = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=scale))
    if shared is not None:
        m["shared"] = dict(ff=shared)
    return m


def _layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def _config(width, vocab, eps, scale, layers):
    return dict(architecture="Sominex", width=width, vocab=vocab, norm=dict(eps=eps), embedding=dict(scale=scale),
                layers=layers)


CONFIGS = {
    # unequal key and value sizes everywhere; rotation of part of a head with stretched frequencies whose
    # ramp lies inside the pairs; blocks of 5 (they straddle page borders) behind a window of 20; three
    # taps; more heads than groups and norm parts that are not the groups; a layer without a feed-forward
    "p": _config(64, 203, 1e-6, 3.0, [
        _layer("attention", _attention(4, 2, 16, 24, 0.3, 20, 5, (8, 100.0), (8.0, 40, 4.0, 1.5)), _dense(40, 1.0)),
        _layer("mamba2", _mamba2(4, 2, 16, 8, 3, 4), _moe(24, 5, 2, 1.7, 16)),
        _layer("mlstm", _mlstm(3, 16, 8, 6.0), None),
        _layer("attention", _attention(2, 1, 8, 8, 0.4, 33, 16, (8, 1e4)), _moe(16, 4, 3, 0.6)),
    ]),
    # a state mixer first; attention heads of 64 on one kv head (the sizes the tensor-core kernels take)
    # with a window longer than a page and blocks of 12; two taps; one group; a router with a single
    # choice and no shared expert; a window without blocks; attention that sees everything
    "q": _config(96, 300, 1e-5, 1.0, [
        _layer("mlstm", _mlstm(2, 40, 24, 15.0), _moe(56, 3, 1, 1.0)),
        _layer("attention", _attention(3, 1, 64, 64, 0.125, 70, 12, (64, 5e4), (4.0, 96, 8.0, 0.5)), _dense(72, 2.5)),
        _layer("mamba2", _mamba2(2, 1, 40, 20, 2, 1), _dense(48, 0.7)),
        _layer("attention", _attention(4, 2, 64, 32, 0.2, 40, None, (32, 1e4)), _moe(32, 6, 2, 2.0, 40)),
        _layer("attention", _attention(2, 2, 24, 40, 0.25), None),
    ]),
    # a width that is no multiple of 8; one tap (the convolution sees the token itself only); one head;
    # every expert chosen; a window of 7 behind blocks of 3, a window of one token behind blocks of one
    "r": _config(60, 130, 1e-6, 0.5, [
        _layer("mamba2", _mamba2(1, 1, 12, 20, 1, 5), _moe(20, 2, 2, 1.2, 12)),
        _layer("attention", _attention(6, 3, 12, 8, 0.3, 7, 3, (12, 1e3), (2.0, 16, 2.0, 1.0)), _dense(36, 1.5)),
        _layer("mlstm", _mlstm(1, 8, 12, 3.0), _dense(28, 4.0)),
        _layer("attention", _attention(2, 2, 8, 12, 0.35, 1, 1, (4, 50.0)), None),
        _layer("mamba2", _mamba2(6, 3, 8, 4, 4, 2), None),
    ]),
}
SEEDS = {"p": 31, "q": 32, "r": 33}


def mixer_weights(rng, kind, m, d, pre=""):
    """The tensors of one mixer, name -> array, at a scale where its gates, decays and norms all matter."""
    def mat(n, k, gain=1.0):
        return rng.standard_normal((n, k)) * gain / np.sqrt(k)
    W = {}
    if kind == "attention":
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        W[pre + "q"], W[pre + "k"], W[pre + "v"] = mat(H * D, d, 2.0), mat(G * D, d, 2.0), mat(G * V, d)
        W[pre + "o"] = mat(d, H * V)
    elif kind == "mamba2":
        H, G, N, V, taps = m["heads"], m["groups"], m["state"], m["vdim"], m["conv"]
        inner, C = H * V, H * V + 2 * G * N
        W[pre + "in"] = mat(2 * inner + 2 * G * N + H, d, 1.5)
        W[pre + "conv"], W[pre + "conv.b"] = rng.standard_normal((C, taps)) * 0.7, rng.standard_normal(C) * 0.3
        W[pre + "dt_bias"], W[pre + "A_log"] = rng.standard_normal(H) - 1.0, rng.standard_normal(H) * 0.7 - 1.5
        W[pre + "D"], W[pre + "norm"] = rng.standard_normal(H), 1 + 0.3 * rng.standard_normal(inner)
        W[pre + "o"] = mat(d, inner)
    elif kind == "mlstm":
        H, D, V = m["heads"], m["dim"], m["vdim"]
        W[pre + "q"], W[pre + "k"], W[pre + "v"] = mat(H * D, d, 2.0), mat(H * D, d, 2.0), mat(H * V, d)
        W[pre + "g"], W[pre + "o"] = mat(H * V, d, 2.0), mat(d, H * V)
        W[pre + "i"], W[pre + "f"] = mat(H, d, 3.0), mat(H, d, 3.0)
        W[pre + "i.b"], W[pre + "f.b"] = rng.standard_normal(H), rng.standard_normal(H) + 3.0
        W[pre + "norm"] = 1 + 0.3 * rng.standard_normal(H * V)
    else:
        raise ValueError(kind)
    return W


def mlp_weights(rng, mlp, d, pre=""):
    def mat(n, k, gain=1.0):
        return rng.standard_normal((n, k)) * gain / np.sqrt(k)

    def glu(p, ff):
        return {p + "gate": mat(ff, d, 2.0), p + "up": mat(ff, d, 2.0), p + "down": mat(d, ff)}
    if mlp is None:
        return {}
    if mlp["kind"] == "dense":
        return glu(pre, mlp["ff"])
    W = {pre + "router": mat(mlp["router"]["experts"], d, 1.5)}
    for e in range(mlp["router"]["experts"]):
        W.update(glu(f"{pre}e{e}.", mlp["expert"]["ff"]))
    if mlp.get("shared"):
        W.update(glu(pre + "shared.", mlp["shared"]["ff"]))
    return W


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> float32 array whose values bfloat16 holds exactly."""
    rng = np.random.default_rng(seed)
    d, V = cfg["width"], cfg["vocab"]
    W = {"embed": rng.standard_normal((V, d)), "final.norm": 1 + 0.2 * rng.standard_normal(d),
         "head": rng.standard_normal((V, d)) / np.sqrt(d)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        W[p + "norm1"] = 1 + 0.2 * rng.standard_normal(d)
        W[p + "shift"] = rng.uniform(0.0, 1.0, d)
        W.update(mixer_weights(rng, layer["type"], layer["mixer"], d, p + "mix."))
        W.update(mlp_weights(rng, layer["mlp"], d, p + "mlp."))
    return {k: to_bf16_values(v) for k, v in W.items()}


@functools.lru_cache(maxsize=None)
def weights(name: str):
    return {k: v.astype(np.float64) for k, v in make_weights(CONFIGS[name], SEEDS[name]).items()}


@functools.lru_cache(maxsize=None)
def model_folder(name: str, storage: str = "bfloat16") -> Path:
    return write_folder(tmp_root() / f"sominex_{name}_{storage}", CONFIGS[name],
                        make_weights(CONFIGS[name], SEEDS[name]), storage)


CLEAR = 0.2      # how far the last expert chosen must stand above the best one left out, as a fraction of its score


def routing_margins(cfg, W, tokens) -> np.ndarray:
    """For every token the smallest margin over the routed layers (inf when nothing is routed or every
    expert is chosen), from a plain run that keeps every layer's normed rows."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
    worst = np.full(len(tokens), np.inf)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = SP.rms_divide(x, eps) * W[p + "norm1"][None, :]
        mlp = layer.get("mlp")
        if mlp is not None and mlp["kind"] == "moe" and mlp["router"]["top"] < mlp["router"]["experts"]:
            _, _, s = SP.route(h, W[p + "mlp.router"], mlp["router"]["top"], 1.0)
            ranked = -np.sort(-s, axis=-1)
            top = mlp["router"]["top"]
            worst = np.minimum(worst, (ranked[:, top - 1] - ranked[:, top]) / ranked[:, top - 1])
        hs = SP.token_shift(h, W[p + "shift"])
        x = x + SP.mixer(layer["type"], hs, W, p + "mix.", layer["mixer"], eps) + SP.feed_forward(h, W, p + "mlp.", mlp)
    return worst


@functools.lru_cache(maxsize=None)
def clear_tokens(name: str, n: int, seed: int) -> tuple:
    """``n`` random tokens, redrawn from the first unclear position on until every routed layer's choice
    at every position stands ``CLEAR`` above the best expert left out: a 16-bit run then makes the same
    choices as the plain one, and the comparison is about arithmetic, not about the side of a tie."""
    rng = np.random.default_rng(9000 + seed)
    cfg, W = CONFIGS[name], weights(name)
    toks = rng.integers(0, cfg["vocab"], n)
    for _ in range(400):
        bad = np.nonzero(routing_margins(cfg, W, toks) <= CLEAR)[0]
        if not len(bad):
            return tuple(int(t) for t in toks)
        toks[bad[0]] = rng.integers(0, cfg["vocab"])      # everything behind it changes: look again
    raise AssertionError("no sequence with clear routing choices found")


_plain: dict = {}


def plain_logits(name: str, tokens) -> np.ndarray:
    key = (name, tuple(tokens))
    if key not in _plain:
        _plain[key] = SP.forward(CONFIGS[name], weights(name), list(tokens))
    return _plain[key]
