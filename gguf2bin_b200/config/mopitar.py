"""Mopitar: the configuration read from ``config.json`` and its translation into a ``ModelSpec``.

The design: a token embedding; layers of the ``parallel_scaled`` arrangement (one ``tanh_norm`` whose output
both sublayers read; each sublayer's result times a learned vector before the sum); three kinds of mixer,
chosen per layer; a dense or a routed feed-forward, or none; a final ``tanh_norm`` and a head of its own.

* ``attention``: ``gqa_attention`` without biases: neighbouring-pair rotation of the first ``rot.dims``
  entries of a head, a score scale of its own, capped scores (``softcap``), every key visible, a learned
  sink per head in the softmax's denominator.  With ``kv_from: j`` the layer has no key and value matrices
  and reads the pages of layer j (``shared_kv``, the schedule's ``cache_of``).
* ``attention_2``: ``diff_attention``: two score maps per head over one set of values; queries and keys
  normed per head and map (one weight of ``dim``) before the rotation; stretched frequencies
  (``rot.scaling``); a window of ``mask.size`` tokens behind which the first ``mask.keep_first`` stay visible;
  plain softmax; the maps' difference normed per head and times 1 - ``diff``.
* ``parallel``: two branches on the same input, each times its scale.  ``left``: ``gqa_attention`` whose q and
  k are divided by their root mean square per head AFTER the rotation, capped scores, every key, plain
  softmax, one sigmoid gate per head.  ``right``: ``selective_ssm``.
* ``dense`` feed-forward: ``act_mlp`` with the squared rectifier.
* ``moe`` feed-forward: ``routed_experts`` with sigmoid scores, groups of neighbouring experts of which the
  best ``groups.keep`` stay eligible, weights renormalised over the chosen, an optional shared expert.

config.json: ``width``, ``vocab``, ``norm.eps`` and a list ``layers`` whose entries give ``type``, ``mixer`` and
``mlp``.  Every size and constant comes from there; ``rot``, ``rot.scaling``, ``mask``, ``mask.keep_first``,
``softcap``, ``router.groups``, ``mlp.shared`` and ``mlp`` may be absent (no rotation, plain frequencies, every key,
no kept tokens, no cap, one group, no shared expert, no feed-forward); a type or kind this reader does not
know is refused, never skipped.
"""
from __future__ import annotations

from typing import Any, Mapping

from .senotar import _float, _get, _int
from .specs import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Mopitar"
MAX_POSITIONS = 1 << 24          # positions are turned into angles in 32-bit: exact integers up to here


def _rotation(m: Mapping[str, Any], where: str, head_dim: int) -> PartSpec:
    rot = m.get("rot")
    if rot is None:
        return PartSpec.make("none")
    dims = _int(rot, "dims")
    if dims % 2 or dims <= 0 or dims > head_dim:
        raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most dim {head_dim}")
    scaling = rot.get("scaling")
    if scaling is None:
        return PartSpec.make("rope_interleaved", theta=_float(rot, "base"), rotary_dim=dims)
    return PartSpec.make("rope_stretched", theta=_float(rot, "base"), rotary_dim=dims, interleaved=True,
                         factor=_float(scaling, "factor"), original=_float(scaling, "original"),
                         fast=_float(scaling, "fast"), slow=_float(scaling, "slow"))


def _heads(m, where: str):
    heads, kv, dim, vdim = _int(m, "heads"), _int(m, "kv_heads"), _int(m, "dim"), _int(m, "vdim")
    if min(heads, kv, dim, vdim) <= 0 or heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
    return heads, kv, dim, vdim


def _mask(m, where: str):
    mask = m.get("mask")
    if mask is None:
        return 0, 0
    window = _int(mask, "size")
    keep = _int(mask, "keep_first", 0) if mask.get("keep_first") is not None else 0
    if window <= 0 or keep < 0:
        raise ConfigError(f"config.json: {where}.mask: size must be positive, keep_first not negative")
    return window, keep


def _softcap(m, where: str) -> float:
    cap = _float(m, "softcap") if m.get("softcap") is not None else 0.0
    if cap < 0:
        raise ConfigError(f"config.json: {where}.softcap must be positive")
    return cap


def _attention(m, where: str, eps: float, pre: str = "mix.", **more) -> PartSpec:
    heads, kv, dim, vdim = _heads(m, where)
    window, keep = _mask(m, where)
    shared = m.get("kv_from") is not None
    names = [("q", pre + "q"), ("o", pre + "o"), ("sink", pre + "sink"), ("k", pre + "k"), ("v", pre + "v")]
    return PartSpec.make(
        "gqa_attention", n_heads=heads, n_kv_heads=kv, head_dim=dim, v_dim=vdim, position=_rotation(m, where, dim),
        window=window, keep_first=keep, scale=_float(m, "scale"), softcap=_softcap(m, where), sink="learned",
        shared_kv=shared, one_pass_prologue=True, names=tuple(names), **more)


def _attention_2(m, where: str, eps: float) -> PartSpec:
    heads, kv, dim, vdim = _heads(m, where)
    window, keep = _mask(m, where)
    diff = _float(m, "diff")
    pre = "mix."
    return PartSpec.make(
        "diff_attention", n_heads=heads, n_kv_heads=kv, head_dim=dim, v_dim=vdim, position=_rotation(m, where, dim),
        window=window, keep_first=keep, scale=_float(m, "scale"), softcap=_softcap(m, where), diff=diff,
        out_norm_eps=eps, qk_norm=PartSpec.make("rmsnorm", eps=eps), qk_norm_span="head",
        names=tuple((k, pre + v) for k, v in (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_norm", "q.norm"),
                                              ("k_norm", "k.norm"), ("lq1", "lq1"), ("lk1", "lk1"), ("lq2", "lq2"),
                                              ("lk2", "lk2"))))


def _left(m, where: str, eps: float, scale: float) -> PartSpec:
    heads, kv, dim, vdim = _heads(m, where)
    window, keep = _mask(m, where)
    pre = "mix.left."
    return PartSpec.make(
        "gqa_attention", n_heads=heads, n_kv_heads=kv, head_dim=dim, v_dim=vdim, position=_rotation(m, where, dim),
        window=window, keep_first=keep, scale=_float(m, "scale"), softcap=_softcap(m, where), qk_unit_eps=eps,
        out_gate="head_sigmoid", out_scale=scale, one_pass_prologue=True,
        names=tuple((k, pre + k) for k in ("q", "k", "v", "o")) + (("gate", pre + "g"),))


def _right(m, where: str, scale: float) -> PartSpec:
    pre = "mix.right."
    return PartSpec.make(
        "selective_ssm", inner=_int(m, "inner"), state_dim=_int(m, "state"), dt_rank=_int(m, "dt_rank"),
        conv_taps=_int(m, "conv"), out_scale=scale,
        names=(("in", pre + "in"), ("conv", pre + "conv"), ("conv_bias", pre + "conv.b"), ("x", pre + "x"),
               ("dt", pre + "dt"), ("dt_bias", pre + "dt.b"), ("a_log", pre + "A_log"), ("skip", pre + "D"),
               ("o", pre + "o")))


def _parallel(m, where: str, eps: float) -> PartSpec:
    for side in ("left", "right"):
        if not isinstance(m.get(side), Mapping):
            raise ConfigError(f"config.json: {where}.mixer.{side} must be an object")
    return PartSpec.make("parallel", branches=(
        ("left", _left(m["left"], where + ".mixer.left", eps, _float(m, "left_scale"))),
        ("right", _right(m["right"], where + ".mixer.right", _float(m, "right_scale")))))


_MIXERS = {"attention": _attention, "attention_2": _attention_2, "parallel": _parallel}


def _mixer(kind, m, where: str, eps: float) -> PartSpec:
    if kind not in _MIXERS:
        raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of {ARCHITECTURE} "
                          f"(known: {', '.join(repr(k) for k in _MIXERS)})")
    if not isinstance(m, Mapping):
        raise ConfigError(f"config.json: {where}.mixer must be an object")
    return _MIXERS[kind](m, where, eps)


def _glu(pre: str, ff: int) -> PartSpec:
    return PartSpec.make("swiglu", intermediate_size=ff,
                         names=(("gate", pre + "gate"), ("up", pre + "up"), ("down", pre + "down")))


def _feed_forward(mlp, where: str):
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, Mapping) else mlp
    if kind == "dense":
        return PartSpec.make("act_mlp", intermediate_size=_int(mlp, "ff"), activation="relu2",
                             names=(("up", "mlp.up"), ("down", "mlp.down")))
    if kind == "moe":
        r = _get(mlp, "router")
        experts, top = _int(r, "experts"), _int(r, "top")
        g = r.get("groups")
        groups = _int(g, "count") if g is not None else 1
        kept = _int(g, "keep") if g is not None else 1
        if groups <= 0 or experts % groups or not (1 <= kept <= groups) or not (1 <= top <= kept * (experts // groups)):
            raise ConfigError(f"config.json: {where}.mlp.router: {experts} experts in {groups} equal groups of which "
                              f"{kept} are kept must hold {top} choices")
        shared = mlp.get("shared")
        return PartSpec.make(
            "routed_experts", n_experts=experts, n_identity=0, top=top, intermediate_size=_int(mlp, "expert.ff"),
            correction=False, renormalise=True, score="sigmoid", groups=groups, groups_kept=kept,
            shared=_glu("mlp.shared.", _int(shared, "ff")) if shared is not None else None,
            names=(("router", "mlp.router"), ("gate", "mlp.e{}.gate"), ("up", "mlp.e{}.up"), ("down", "mlp.e{}.down")))
    raise ConfigError(f"config.json: {where}.mlp.kind {kind!r} is not a feed-forward of {ARCHITECTURE} "
                      "(known: 'dense', 'moe', or null for none)")


def _kv_source(i: int, entry, layers_in, where: str):
    """The layer whose pages layer i reads (None: its own), checked against the rule that the lender
    projects keys and values itself and has this layer's head counts, sizes and rotation."""
    m = entry.get("mixer")
    src = m.get("kv_from") if isinstance(m, Mapping) else None
    if src is None:
        return None
    if entry.get("type") != "attention":
        raise ConfigError(f"config.json: {where}: only an 'attention' mixer reads another layer's keys and values")
    if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < i):
        raise ConfigError(f"config.json: {where}.mixer.kv_from {src!r} must name an earlier layer")
    lender = layers_in[src]
    lm = lender.get("mixer") if isinstance(lender, Mapping) else None
    if lender.get("type") != "attention" or not isinstance(lm, Mapping) or lm.get("kv_from") is not None:
        raise ConfigError(f"config.json: {where}.mixer.kv_from {src}: that layer has no keys and values of its own "
                          "to lend")
    for key in ("kv_heads", "dim", "vdim", "rot"):
        if lm.get(key) != m.get(key):
            raise ConfigError(f"config.json: {where}.mixer.kv_from {src}: {key!r} differs between the two layers")
    return int(src)


def mopitar_model_spec(d: Mapping[str, Any]) -> ModelSpec:
    width, vocab = _int(d, "width"), _int(d, "vocab")
    eps = _float(d, "norm.eps")
    if not eps > 0:
        raise ConfigError("config.json: 'norm.eps' must be positive")
    norm = PartSpec.make("tanh_norm")
    layers_in = _get(d, "layers")
    if not isinstance(layers_in, (list, tuple)) or not layers_in:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    block = PartSpec.make("parallel_scaled", names=(("norm", "norm1"), ("mixer_scale", "ls1"), ("ffn_scale", "ls2")))
    layers, schedule = [], []
    for i, entry in enumerate(layers_in):
        where = f"layers[{i}]"
        if not isinstance(entry, Mapping):
            raise ConfigError(f"config.json: {where} must be an object")
        layers.append(LayerSpec(block=block, mixer=_mixer(entry.get("type"), entry.get("mixer"), where, eps),
                                feed_forward=_feed_forward(entry.get("mlp"), where), norm=norm, prefix=f"l{i}."))
        schedule.append(ScheduleEntry(i, _kv_source(i, entry, layers_in, where)))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab, max_positions=MAX_POSITIONS,
        layers=tuple(layers), schedule=tuple(schedule),
        embedding=PartSpec.make("token_embedding", name="embed"),
        final_norm=PartSpec.make("tanh_norm", name="final.norm"),
        head=PartSpec.make("lm_head", tied=False, name="head"), stop_token_ids=(), source=dict(d))
    spec.validate()
    return spec
