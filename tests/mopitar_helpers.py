"""Shared by the Mopitar tests: small configurations that differ from one another in every size and
option, weights at a scale where every mechanism matters, model folders in temporary places, token
sequences whose routing choices are clear, and the plain implementation's results."""
from __future__ import annotations

import functools
from pathlib import Path

import numpy as np

from helpers import tmp_root
from plain import mopitar_plain as MP
from senotar_helpers import to_bf16_values, write_folder


def _rot(dims, base, scaling=None):
    r = dict(dims=dims, base=base)
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _attention(heads, kv, dim, vdim, scale, softcap=None, rot=None, kv_from=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = rot
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _attention_2(heads, kv, dim, vdim, scale, diff, window=None, keep=None, rot=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, diff=diff)
    if window is not None:
        m["mask"] = dict(size=window) if keep is None else dict(size=window, keep_first=keep)
    if rot is not None:
        m["rot"] = rot
    return m


def _parallel(left, right, left_scale, right_scale):
    return dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale)


def _ssm(inner, state, dt_rank, conv):
    return dict(inner=inner, state=state, dt_rank=dt_rank, conv=conv)


def _dense(ff):
    return dict(kind="dense", ff=ff)


def _moe(ff, experts, top, groups=None, shared=None):
    r = dict(experts=experts, top=top)
    if groups is not None:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    m = dict(kind="moe", expert=dict(ff=ff), router=r)
    if shared is not None:
        m["shared"] = dict(ff=shared)
    return m


def _layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def _config(width, vocab, eps, layers):
    return dict(architecture="Mopitar", width=width, vocab=vocab, norm=dict(eps=eps), layers=layers)


CONFIGS = {
    # unequal key and value sizes everywhere; part of a head turned; stretched frequencies whose ramp lies
    # inside the pairs; a window of 20 behind 3 kept tokens; three taps; a state of 12 entries (three a
    # lane); experts in 3 groups of which 2 stay; a layer that borrows keys and values two layers back
    "p": _config(64, 203, 1e-6, [
        _layer("attention_2", _attention_2(4, 2, 16, 24, 0.3, 0.4, 20, 3, _rot(8, 100.0, (8.0, 40, 4.0, 1.5))), _dense(40)),
        _layer("parallel", _parallel(_attention(3, 1, 16, 8, 0.35, 20.0, _rot(16, 1e4)), _ssm(40, 12, 5, 3), 0.7, 1.3),
               _moe(24, 6, 2, (3, 2), 16)),
        _layer("attention", _attention(4, 2, 24, 16, 0.25, 15.0, _rot(12, 1e3)), None),
        _layer("attention", _attention(2, 2, 24, 16, 0.3, 8.0, _rot(12, 1e3), kv_from=2), _dense(56)),
    ]),
    # the two-branch mixer first; heads of 64 and 128 (the sizes the tensor-core kernels take) with a
    # window longer than a page and more kept tokens than a page has; two taps; a state that takes 16 lanes;
    # a router without groups and with a single choice; two borrowers of one lender
    "q": _config(96, 300, 1e-5, [
        _layer("parallel", _parallel(_attention(2, 1, 64, 64, 0.2, 30.0, _rot(64, 5e4)), _ssm(48, 40, 8, 2), 1.0, 0.5),
               _moe(56, 3, 1)),
        _layer("attention", _attention(3, 3, 128, 128, 0.1, 50.0, _rot(32, 1e4)), _dense(72)),
        _layer("attention_2", _attention_2(2, 1, 64, 64, 0.15, 0.7, 70, 66, _rot(64, 1e4, (4.0, 96, 8.0, 0.5))),
               _moe(32, 8, 3, (2, 1), 40)),
        _layer("attention", _attention(6, 3, 128, 128, 0.08, 50.0, _rot(32, 1e4), kv_from=1), None),
        _layer("attention", _attention(3, 3, 128, 128, 0.12, 25.0, _rot(32, 1e4), kv_from=1), _dense(48)),
    ]),
    # a width that is no multiple of 8; one tap (the convolution sees the token itself only); one head;
    # every expert chosen, a group an expert; a window of the token itself behind one kept token; no
    # rotation; a window without kept tokens; a state of 3 entries; no cap on one attention's scores
    "r": _config(60, 130, 1e-6, [
        _layer("attention", _attention(1, 1, 12, 20, 0.3, 10.0, None), _moe(20, 4, 4, (4, 4), 12)),
        _layer("attention_2", _attention_2(3, 3, 8, 12, 0.4, 0.25, 1, 1, _rot(8, 50.0)), _dense(36)),
        _layer("parallel", _parallel(_attention(2, 2, 8, 12, 0.5, 5.0, _rot(4, 1e3)), _ssm(28, 3, 7, 1), 1.5, 0.8), None),
        _layer("attention_2", _attention_2(2, 1, 12, 8, 0.3, 0.5, 7, None, _rot(12, 1e3, (2.0, 16, 2.0, 1.0))), _dense(28)),
        _layer("attention", _attention(3, 1, 12, 20, 0.3, None, None, kv_from=0), _moe(16, 6, 2, (2, 2))),
    ]),
}
SEEDS = {"p": 41, "q": 42, "r": 43}


def mixer_weights(rng, kind, m, d, pre=""):
    """The tensors of one mixer, name -> array, at a scale where its gates, decays, sinks and norms matter."""
    def mat(n, k, gain=1.0):
        return rng.standard_normal((n, k)) * gain / np.sqrt(k)
    W = {}
    if kind == "attention":
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        W[pre + "q"], W[pre + "o"] = mat(H * D, d, 2.0), mat(d, H * V)
        W[pre + "sink"] = rng.standard_normal(H) * 1.5
        if m.get("kv_from") is None:
            W[pre + "k"], W[pre + "v"] = mat(G * D, d, 2.0), mat(G * V, d)
    elif kind == "attention_2":
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        W[pre + "q"], W[pre + "k"], W[pre + "v"] = mat(2 * H * D, d, 2.0), mat(2 * G * D, d, 2.0), mat(G * V, d)
        W[pre + "o"] = mat(d, H * V)
        W[pre + "q.norm"], W[pre + "k.norm"] = 1 + 0.3 * rng.standard_normal(D), 1 + 0.3 * rng.standard_normal(D)
        for k in ("lq1", "lk1", "lq2", "lk2"):
            W[pre + k] = rng.standard_normal(D) * 0.7 / D ** 0.25
    elif kind == "left":
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        W[pre + "q"], W[pre + "k"], W[pre + "v"] = mat(H * D, d, 2.0), mat(G * D, d, 2.0), mat(G * V, d)
        W[pre + "g"], W[pre + "o"] = mat(H, d, 2.0), mat(d, H * V)
    elif kind == "right":
        inner, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
        W[pre + "in"] = mat(2 * inner, d, 1.5)
        W[pre + "conv"], W[pre + "conv.b"] = rng.standard_normal((inner, taps)) * 0.7, rng.standard_normal(inner) * 0.3
        W[pre + "x"], W[pre + "dt"] = mat(R + 2 * N, inner, 1.5), mat(inner, R, 1.5)
        W[pre + "dt.b"] = rng.standard_normal(inner) - 1.0
        W[pre + "A_log"] = rng.standard_normal((inner, N)) * 0.7 - 0.5
        W[pre + "D"], W[pre + "o"] = rng.standard_normal(inner), mat(d, inner)
    elif kind == "parallel":
        W.update(mixer_weights(rng, "left", m["left"], d, pre + "left."))
        W.update(mixer_weights(rng, "right", m["right"], d, pre + "right."))
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
        return {pre + "up": mat(mlp["ff"], d, 1.5), pre + "down": mat(d, mlp["ff"])}
    W = {pre + "router": mat(mlp["router"]["experts"], d, 2.0)}
    for e in range(mlp["router"]["experts"]):
        W.update(glu(f"{pre}e{e}.", mlp["expert"]["ff"]))
    if mlp.get("shared"):
        W.update(glu(pre + "shared.", mlp["shared"]["ff"]))
    return W


def norm_weights(rng, d, name):
    return {name: 1 + 0.2 * rng.standard_normal(d), name + ".b": 0.2 * rng.standard_normal(d),
            name + ".alpha": np.array(0.4 + 0.4 * rng.random())}


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> float32 array whose values bfloat16 holds exactly."""
    rng = np.random.default_rng(seed)
    d, V = cfg["width"], cfg["vocab"]
    W = {"embed": rng.standard_normal((V, d)) * 1.5, "head": rng.standard_normal((V, d)) / np.sqrt(d)}
    W.update(norm_weights(rng, d, "final.norm"))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        W.update(norm_weights(rng, d, p + "norm1"))
        W[p + "ls1"] = 0.6 + 0.3 * rng.standard_normal(d)
        if layer["mlp"] is not None:
            W[p + "ls2"] = 0.6 + 0.3 * rng.standard_normal(d)
        W.update(mixer_weights(rng, layer["type"], layer["mixer"], d, p + "mix."))
        W.update(mlp_weights(rng, layer["mlp"], d, p + "mlp."))
    return {k: to_bf16_values(v).reshape(np.shape(v)) for k, v in W.items()}      # the norm's alpha has no shape


@functools.lru_cache(maxsize=None)
def weights(name: str):
    return {k: v.astype(np.float64) for k, v in make_weights(CONFIGS[name], SEEDS[name]).items()}


@functools.lru_cache(maxsize=None)
def model_folder(name: str, storage: str = "bfloat16") -> Path:
    return write_folder(tmp_root() / f"mopitar_{name}_{storage}", CONFIGS[name],
                        make_weights(CONFIGS[name], SEEDS[name]), storage)


CLEAR = 0.06     # how far a choice must stand above the best one left out, as a fraction of its score


def router_settings(mlp):
    r = mlp["router"]
    g = r.get("groups") or {}
    return int(r["top"]), int(g.get("count") or 1), int(g.get("keep") or g.get("count") or 1)


def routing_margins(cfg, W, tokens) -> np.ndarray:
    """For every token the smallest margin over the routed layers (inf when nothing is routed or every
    expert is chosen), from a plain run that hands over every layer's normed rows."""
    worst = np.full(len(tokens), np.inf)

    def watch(i, h):
        mlp = cfg["layers"][i].get("mlp")
        if mlp is None or mlp["kind"] != "moe":
            return
        z = h @ W[f"l{i}.mlp.router"].T
        top, groups, keep = router_settings(mlp)
        for t in range(len(tokens)):
            worst[t] = min(worst[t], MP.routing_margin(z[t], top, groups, keep))
    MP.forward(cfg, W, list(tokens), watch=watch)
    return worst


@functools.lru_cache(maxsize=None)
def clear_tokens(name: str, n: int, seed: int) -> tuple:
    """``n`` random tokens, redrawn from the first unclear position on until every routed layer's choice
    at every position stands ``CLEAR`` above the best group and expert left out: a 16-bit run then makes
    the same choices as the plain one, and the comparison is about arithmetic, not about the side of a tie."""
    from threadpoolctl import threadpool_limits
    with threadpool_limits(1):                            # many small products: threads only get in each other's way
        return _clear_tokens(name, n, seed)


def _clear_tokens(name: str, n: int, seed: int) -> tuple:
    rng = np.random.default_rng(7000 + seed)
    cfg, W = CONFIGS[name], weights(name)
    toks = rng.integers(0, cfg["vocab"], n)
    good = 0                                              # tokens in front of here are settled (the model is causal)
    for _ in range(2000):
        if good >= n:
            return tuple(int(t) for t in toks)
        upto = min(n, max(2 * good, 16))
        bad = np.nonzero(routing_margins(cfg, W, toks[:upto]) <= CLEAR)[0]
        if not len(bad):
            good = upto
            continue
        toks[bad[0]] = rng.integers(0, cfg["vocab"])      # everything behind it changes: look again
        good = int(bad[0])
    raise AssertionError("no sequence with clear routing choices found")


_plain: dict = {}


def plain_logits(name: str, tokens) -> np.ndarray:
    key = (name, tuple(tokens))
    if key not in _plain:
        _plain[key] = MP.forward(CONFIGS[name], weights(name), list(tokens))
    return _plain[key]
