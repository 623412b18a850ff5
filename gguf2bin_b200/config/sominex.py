"""Sominex: the configuration read from ``config.json`` and its translation into a ``ModelSpec``.

The design: a token embedding times a constant; layers of the ``parallel_shift`` arrangement (one RMS
norm whose output both sublayers read, the mixer's copy shifted towards the token before); three kinds
of mixer, chosen per layer; a dense or a routed feed-forward, or none; a final norm and a head of its own.

* ``attention``: grouped-query attention without biases, half-split rotation of part of each head with
  stretched frequencies, values divided by their root mean square per head before they are stored, a
  score scale of its own, a window of tokens with mean keys and values of whole blocks in front of it.
* ``mamba2``: the ``ssd`` mixer (state-space duality: a scalar decay per head and token behind a short
  convolution, a skip, a gate in front of a grouped norm).
* ``mlstm``: the ``mlstm`` mixer (matrix memory, exponential gates capped by a tanh, a running maximum).
* ``dense`` feed-forward: ``swiglu`` with ``limit`` (capped gate and up value, sigmoid slope 1.702, up + 1).
* ``moe`` feed-forward: ``routed_experts`` with softmax scores times ``router.scale``, not renormalised,
  and an optional shared expert that every token uses.

config.json: ``width``, ``vocab``, ``norm.eps``, ``embedding.scale`` and a list ``layers`` whose entries give
``type``, ``mixer`` and ``mlp``.  Every size and constant comes from there; ``rot``, ``rot.scaling``, ``mask``,
``mask.pool`` and ``mlp.shared`` may be absent (no rotation, plain frequencies, every key, no blocks, no
shared expert); a type or kind this reader does not know is refused, never skipped.
"""
from __future__ import annotations

from typing import Any, Mapping

from .senotar import _float, _get, _int
from .specs import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Sominex"
MAX_POSITIONS = 1 << 24          # positions are turned into angles in 32-bit: exact integers up to here
GLU_SLOPE = 1.702                # slope of the sigmoid in the dense feed-forward's gate


def _rotation(m: Mapping[str, Any], where: str, head_dim: int) -> PartSpec:
    rot = m.get("rot")
    if rot is None:
        return PartSpec.make("none")
    dims = _int(rot, "dims")
    if dims % 2 or dims > head_dim:
        raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most dim {head_dim}")
    scaling = rot.get("scaling")
    if scaling is None:
        return PartSpec.make("rope_neox", theta=_float(rot, "base"), rotary_dim=dims)
    return PartSpec.make("rope_stretched", theta=_float(rot, "base"), rotary_dim=dims,
                         factor=_float(scaling, "factor"), original=_float(scaling, "original"),
                         fast=_float(scaling, "fast"), slow=_float(scaling, "slow"))


def _attention(m, where: str, eps: float) -> PartSpec:
    heads, kv, dim, vdim = _int(m, "heads"), _int(m, "kv_heads"), _int(m, "dim"), _int(m, "vdim")
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
    mask = m.get("mask")
    window = _int(mask, "size") if mask is not None else 0
    pool = _int(mask, "pool") if mask is not None and mask.get("pool") is not None else 0
    return PartSpec.make(
        "gqa_attention", n_heads=heads, n_kv_heads=kv, head_dim=dim, v_dim=vdim,
        position=_rotation(m, where, dim), window=window, pool=pool, scale=_float(m, "scale"), v_norm_eps=eps,
        names=(("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("o", "mix.o")))


def _ssd(m, where: str, eps: float) -> PartSpec:
    heads, groups = _int(m, "heads"), _int(m, "groups")
    if heads % groups:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {groups} groups")
    inner, parts = heads * _int(m, "vdim"), _int(m, "norm_groups")
    if inner % parts:
        raise ConfigError(f"config.json: {where}: norm_groups {parts} does not divide heads * vdim = {inner}")
    return PartSpec.make(
        "ssd", n_heads=heads, n_groups=groups, state_dim=_int(m, "state"), v_dim=_int(m, "vdim"),
        conv_taps=_int(m, "conv"), norm_groups=parts, eps=eps,
        names=(("in", "mix.in"), ("conv", "mix.conv"), ("conv_bias", "mix.conv.b"), ("dt_bias", "mix.dt_bias"),
               ("a_log", "mix.A_log"), ("skip", "mix.D"), ("norm", "mix.norm"), ("o", "mix.o")))


def _mlstm(m, where: str, eps: float) -> PartSpec:
    return PartSpec.make(
        "mlstm", n_heads=_int(m, "heads"), qk_dim=_int(m, "dim"), v_dim=_int(m, "vdim"),
        gate_cap=_float(m, "gate_cap"), eps=eps,
        names=(("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("gate", "mix.g"), ("o", "mix.o"),
               ("norm", "mix.norm"), ("i", "mix.i"), ("i_bias", "mix.i.b"), ("f", "mix.f"), ("f_bias", "mix.f.b")))


_MIXERS = {"attention": _attention, "mamba2": _ssd, "mlstm": _mlstm}


def _mixer(kind, m, where: str, eps: float) -> PartSpec:
    if kind not in _MIXERS:
        raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of {ARCHITECTURE} "
                          f"(known: {', '.join(repr(k) for k in _MIXERS)})")
    if not isinstance(m, Mapping):
        raise ConfigError(f"config.json: {where}.mixer must be an object")
    return _MIXERS[kind](m, where, eps)


def _glu(pre: str, ff: int, **more) -> PartSpec:
    return PartSpec.make("swiglu", intermediate_size=ff,
                         names=(("gate", pre + "gate"), ("up", pre + "up"), ("down", pre + "down")), **more)


def _feed_forward(mlp, where: str):
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, Mapping) else mlp
    if kind == "dense":
        limit = _float(mlp, "limit")
        if not limit > 0:
            raise ConfigError(f"config.json: {where}.mlp.limit must be positive")
        return _glu("mlp.", _int(mlp, "ff"), limit=limit, alpha=GLU_SLOPE)
    if kind == "moe":
        r = _get(mlp, "router")
        shared = mlp.get("shared")
        return PartSpec.make(
            "routed_experts", n_experts=_int(r, "experts"), n_identity=0, top=_int(r, "top"),
            intermediate_size=_int(mlp, "expert.ff"), correction=False, renormalise=False,
            scale=_float(r, "scale") if r.get("scale") is not None else 1.0,
            shared=_glu("mlp.shared.", _int(shared, "ff")) if shared is not None else None,
            names=(("router", "mlp.router"), ("gate", "mlp.e{}.gate"), ("up", "mlp.e{}.up"),
                   ("down", "mlp.e{}.down")))
    raise ConfigError(f"config.json: {where}.mlp.kind {kind!r} is not a feed-forward of {ARCHITECTURE} "
                      "(known: 'dense', 'moe', or null for none)")


def sominex_model_spec(d: Mapping[str, Any]) -> ModelSpec:
    width, vocab = _int(d, "width"), _int(d, "vocab")
    eps = _float(d, "norm.eps")
    if not eps > 0:
        raise ConfigError("config.json: 'norm.eps' must be positive")
    scale = _float(d, "embedding.scale") if isinstance(d.get("embedding"), Mapping) and \
        d["embedding"].get("scale") is not None else 1.0
    norm = PartSpec.make("rmsnorm", eps=eps)
    layers_in = _get(d, "layers")
    if not isinstance(layers_in, (list, tuple)) or not layers_in:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    block = PartSpec.make("parallel_shift", names=(("norm", "norm1"), ("shift", "shift")))
    layers = []
    for i, entry in enumerate(layers_in):
        where = f"layers[{i}]"
        if not isinstance(entry, Mapping):
            raise ConfigError(f"config.json: {where} must be an object")
        layers.append(LayerSpec(block=block, mixer=_mixer(entry.get("type"), entry.get("mixer"), where, eps),
                                feed_forward=_feed_forward(entry.get("mlp"), where), norm=norm, prefix=f"l{i}."))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab, max_positions=MAX_POSITIONS,
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        embedding=PartSpec.make("token_embedding", name="embed", scale=scale),
        final_norm=PartSpec.make("rmsnorm", eps=eps, name="final.norm"),
        head=PartSpec.make("lm_head", tied=False, name="head"), stop_token_ids=(), source=dict(d))
    spec.validate()
    return spec
