"""Sominex without a device: the configuration reader and its refusals, the tensor list, what each
layer asks of the cache, and facts about the plain mechanisms that the device tests lean on."""
import copy
import math

import numpy as np
import pytest

from plain import sominex_plain as SP
from sominex_helpers import CONFIGS, SEEDS, make_weights


def spec_of(cfg):
    from gguf2bin_b200.config import model_spec_from_dict
    return model_spec_from_dict(cfg)


def test_reader_takes_every_size_and_constant_from_the_configuration():
    spec = spec_of(CONFIGS["p"])
    assert (spec.architecture, spec.hidden_size, spec.vocab_size, len(spec.layers)) == ("Sominex", 64, 203, 4)
    assert spec.embedding["scale"] == 3.0 and spec.head.get("tied") is False and spec.final_norm["eps"] == 1e-6
    a = spec.layers[0]
    assert a.block.kind == "parallel_shift" and a.norm.kind == "rmsnorm" and a.norm["eps"] == 1e-6 and a.prefix == "l0."
    m = a.mixer
    assert (m.kind, m["n_heads"], m["n_kv_heads"], m["head_dim"], m["v_dim"]) == ("gqa_attention", 4, 2, 16, 24)
    assert (m["window"], m["pool"], m["scale"], m["v_norm_eps"]) == (20, 5, 0.3, 1e-6)
    pos = m["position"]
    assert (pos.kind, pos["rotary_dim"], pos["theta"]) == ("rope_stretched", 8, 100.0)
    assert (pos["factor"], pos["original"], pos["fast"], pos["slow"]) == (8.0, 40.0, 4.0, 1.5)
    f = a.feed_forward
    assert (f.kind, f["intermediate_size"], f["limit"], f["alpha"]) == ("swiglu", 40, 1.0, 1.702)
    s = spec.layers[1]
    assert (s.mixer.kind, s.mixer["n_heads"], s.mixer["n_groups"], s.mixer["state_dim"], s.mixer["v_dim"],
            s.mixer["conv_taps"], s.mixer["norm_groups"]) == ("ssd", 4, 2, 16, 8, 3, 4)
    r = s.feed_forward
    assert (r.kind, r["n_experts"], r["top"], r["intermediate_size"], r["scale"]) == ("routed_experts", 5, 2, 24, 1.7)
    assert r["renormalise"] is False and r["shared"].kind == "swiglu" and r["shared"]["intermediate_size"] == 16
    x = spec.layers[2]
    assert (x.mixer.kind, x.mixer["n_heads"], x.mixer["qk_dim"], x.mixer["v_dim"], x.mixer["gate_cap"]) == ("mlstm", 3, 16, 8, 6.0)
    assert x.feed_forward is None
    plain = spec.layers[3]
    assert plain.mixer["position"].kind == "rope_neox" and plain.feed_forward["shared"] is None
    everything = spec_of(CONFIGS["q"]).layers[4].mixer
    assert (everything["window"], everything["pool"], everything["position"].kind) == (0, 0, "none")
    assert spec_of(CONFIGS["q"]).layers[3].mixer["pool"] == 0 and spec_of(CONFIGS["q"]).layers[3].mixer["window"] == 40


def test_tensor_list_matches_the_checkpoint_names():
    from gguf2bin_b200.engine.model import expected_tensors
    for name, cfg in CONFIGS.items():
        exp = expected_tensors(spec_of(cfg))
        have = make_weights(cfg, SEEDS[name])
        assert {k for k, e in exp.items() if not e.optional} == set(have) - {k for k, e in exp.items() if e.optional}
        for k, v in have.items():
            assert tuple(exp[k].shape) == v.shape, k


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="retention"), "not a mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "not a feed-forward"),
    (lambda c: c["layers"][0]["mlp"].update(limit=0.0), "positive"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "even and at most"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "does not divide"),
    (lambda c: c["layers"][2]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][1]["mlp"]["router"].pop("top"), "top"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c.update(layers=[]), "non-empty"),
])
def test_refusals(change, message):
    from gguf2bin_b200.config import ConfigError
    cfg = copy.deepcopy(CONFIGS["p"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        spec_of(cfg)


def test_cache_needs_of_the_layers():
    torch = pytest.importorskip("torch")
    from gguf2bin_b200.cache.storage import PAGE_SIZE, KVNeed, StateNeed
    from gguf2bin_b200.parts import mixer_class
    spec = spec_of(CONFIGS["p"])

    def need(i, dtype=torch.bfloat16):
        m = spec.layers[i].mixer
        return mixer_class(m)(m, 64, dtype, "cpu").cache_need()
    assert need(0) == {"kv": KVNeed(2, 24, 20), "pool": KVNeed(2, 24, 0, rows=-(-PAGE_SIZE // 5))}
    assert need(1) == {"state": StateNeed((4, 8, 16), torch.float32),
                       "conv": StateNeed((3, 4 * 8 + 2 * 2 * 16), torch.bfloat16, by_position=True)}
    assert need(2) == {"state": StateNeed((3, 8 + 1, 16), torch.float32), "max": StateNeed((3,), torch.float32)}
    one_tap = spec_of(CONFIGS["r"]).layers[0].mixer
    assert set(mixer_class(one_tap)(one_tap, 60, torch.float32, "cpu").cache_need()) == {"state"}
    # the block keeps the normed row of the latest token, whatever its mixer keeps
    from gguf2bin_b200.parts import block_class
    layer = spec.layers[2]
    blk = block_class(layer.block)(layer, 64, torch.float32, "cpu")
    assert blk.cache_need()["shift"] == StateNeed((64,), torch.float32)
    assert set(blk.cache_need()) == {"shift", "mixer.state", "mixer.max"}


def test_stretched_frequencies():
    torch = pytest.importorskip("torch")
    from gguf2bin_b200.config.specs import PartSpec
    from gguf2bin_b200.parts import position_class
    for dims, base, sc in [(8, 100.0, (8.0, 40, 4.0, 1.5)), (64, 5e4, (4.0, 96, 8.0, 0.5)), (12, 1e3, (2.0, 16, 2.0, 1.0)),
                           (32, 1e4, (16.0, 4096, 32.0, 1.0)), (6, 10.0, (3.0, 8, 1.0, 1.0))]:
        scaling = dict(zip(("factor", "original", "fast", "slow"), sc))
        f, mult = SP.stretched_frequencies(base, dims, scaling)
        spec = PartSpec.make("rope_stretched", theta=base, rotary_dim=dims, factor=sc[0], original=float(sc[1]),
                             fast=sc[2], slow=sc[3])
        part = position_class(spec)(spec, dims, "cpu")
        inv, rot, interleaved = part.table_rotation()
        assert rot == dims and not interleaved and abs(part.mult - mult) < 1e-7
        assert np.allclose(inv.double().numpy(), f, rtol=2e-6, atol=0)
        # the fast pairs keep their frequency, the slowest are divided by the factor, none goes up
        plain, _ = SP.stretched_frequencies(base, dims, None)
        assert np.all(f <= plain * (1 + 1e-12)) and np.all(f >= plain / sc[0] * (1 - 1e-12))
        assert mult == pytest.approx(0.1 * math.log(sc[0]) + 1.0)


def test_plain_mechanisms():
    rng = np.random.default_rng(0)
    # token shift: the first row mixes with zeros, later rows with the unshifted row before
    h, mu = rng.standard_normal((4, 6)), rng.uniform(0, 1, 6)
    s = SP.token_shift(h, mu)
    assert np.allclose(s[0], h[0] * (1 - mu)) and np.allclose(s[2], h[2] + (h[1] - h[2]) * mu)
    # rotation: position 0 turns nothing, lengths scale by the multiplier, the tail passes
    x = rng.standard_normal((5, 2, 12))
    f, mult = SP.stretched_frequencies(1e3, 8, dict(factor=4.0, original=32, fast=4.0, slow=1.0))
    y = SP.rotate_half(x, np.arange(5), f, mult)
    assert np.allclose(y[0, :, :8], x[0, :, :8] * mult) and np.allclose(y[..., 8:], x[..., 8:])
    assert np.allclose((y[..., :8] ** 2).sum(-1), (x[..., :8] ** 2).sum(-1) * mult * mult)
    # the window and the blocks: with equal keys every visible entry weighs the same, so the output is the
    # mean of what is seen; token 11 with a window of 4 and blocks of 3 sees tokens 8..11 and blocks 0, 1
    # (positions 0..5); positions 6, 7 are in no block that lies wholly before the window
    T = 12
    q, k = np.ones((T, 1, 2)), np.ones((T, 1, 2))
    v = np.arange(T, dtype=np.float64).reshape(T, 1, 1)
    o = SP.window_pool_attention(q, k, v, 1.0, 4, 3)
    assert o[11, 0, 0] == pytest.approx((8 + 9 + 10 + 11 + 1.0 + 4.0) / 6)
    assert o[6, 0, 0] == pytest.approx((3 + 4 + 5 + 6 + 1.0) / 5)          # block 0 ends at 2 = 6 - 4: just seen
    assert o[5, 0, 0] == pytest.approx((2 + 3 + 4 + 5) / 4)                # not yet
    assert SP.window_pool_attention(q, k, v, 1.0, 4, 0)[11, 0, 0] == pytest.approx(9.5)
    # the state-space scan equals its unrolled sum
    x, B, C = rng.standard_normal((6, 1, 3)), rng.standard_normal((6, 1, 2)), rng.standard_normal((6, 1, 2))
    dt, A_log, D = rng.uniform(0.1, 1, (6, 1)), np.array([0.3]), np.array([0.7])
    y = SP.ssd_scan(x, B, C, dt, A_log, D)
    a = math.exp(A_log[0])
    want = sum(math.exp(-a * dt[j + 1:6, 0].sum()) * dt[j, 0] * (B[j, 0] @ C[5, 0]) * x[j, 0] for j in range(6)) + D[0] * x[5, 0]
    assert np.allclose(y[5, 0], want)
    # matrix memory: the running maximum starts at 0, so a first token with a very negative input gate
    # reads out against exp(-m) = 1, not against its own tiny normaliser
    q1, k1, v1 = np.ones((1, 1, 2)), np.ones((1, 1, 2)), np.array([[[3.0, -1.0]]])
    o = SP.mlstm_scan(q1, k1, v1, np.array([[-9.0]]), np.array([[-0.1]]))
    assert np.allclose(o[0, 0], math.exp(-9.0) * 2 * v1[0, 0] / (1.0 + 1e-6))
    o = SP.mlstm_scan(q1, k1, v1, np.array([[4.0]]), np.array([[-0.1]]))       # m = 4: n.q = 2 > exp(-4)
    assert np.allclose(o[0, 0], 2 * v1[0, 0] / (2.0 + 1e-6))
    # the capped feed-forward: the gate is capped from above only, the up value on both sides
    W = {"gate": np.array([[10.0], [-10.0]]), "up": np.array([[10.0], [-10.0]]), "down": np.eye(2)}
    y = SP.capped_glu(np.array([[1.0]]), W, "", 2.0)
    assert np.allclose(y[0], [2.0 * SP.sigmoid(1.702 * 2.0) * 3.0, -10.0 * SP.sigmoid(-17.02) * -1.0])
    # routing: the weights are the scores times the scale, and do not sum to one
    idx, wt, s = SP.route(rng.standard_normal((3, 5)), rng.standard_normal((4, 5)), 2, 2.5)
    assert np.allclose(wt, 2.5 * np.take_along_axis(s, idx, -1)) and np.all(wt.sum(-1) < 2.5)
