"""Mopitar without a device: the configuration reader and its refusals, the tensor list, what each
layer asks of the cache, and facts about the plain mechanisms that the device tests lean on."""
import copy
import math

import numpy as np
import pytest

from mopitar_helpers import CONFIGS, SEEDS, make_weights, weights
from plain import mopitar_plain as MP


def spec_of(cfg):
    from gguf2bin_b200.config import model_spec_from_dict
    return model_spec_from_dict(cfg)


def test_reader_takes_every_size_and_constant_from_the_configuration():
    spec = spec_of(CONFIGS["p"])
    assert (spec.architecture, spec.hidden_size, spec.vocab_size, len(spec.layers)) == ("Mopitar", 64, 203, 4)
    assert spec.final_norm.kind == "tanh_norm" and spec.head.get("tied") is False
    a = spec.layers[0]
    assert a.block.kind == "parallel_scaled" and a.norm.kind == "tanh_norm" and a.prefix == "l0."
    m = a.mixer
    assert (m.kind, m["n_heads"], m["n_kv_heads"], m["head_dim"], m["v_dim"]) == ("diff_attention", 4, 2, 16, 24)
    assert (m["window"], m["keep_first"], m["scale"], m["diff"], m["out_norm_eps"]) == (20, 3, 0.3, 0.4, 1e-6)
    assert m["qk_norm"]["eps"] == 1e-6 and m["qk_norm_span"] == "head"
    pos = m["position"]
    assert (pos.kind, pos["rotary_dim"], pos["theta"], pos["interleaved"]) == ("rope_stretched", 8, 100.0, True)
    assert (pos["factor"], pos["original"], pos["fast"], pos["slow"]) == (8.0, 40.0, 4.0, 1.5)
    f = a.feed_forward
    assert (f.kind, f["intermediate_size"], f["activation"]) == ("act_mlp", 40, "relu2")
    two = spec.layers[1].mixer
    assert two.kind == "parallel" and [n for n, _ in two["branches"]] == ["left", "right"]
    left, right = (s for _, s in two["branches"])
    assert (left.kind, left["n_heads"], left["n_kv_heads"], left["head_dim"], left["v_dim"]) == ("gqa_attention", 3, 1, 16, 8)
    assert (left["softcap"], left["qk_unit_eps"], left["out_gate"], left["out_scale"]) == (20.0, 1e-6, "head_sigmoid", 0.7)
    assert left["position"].kind == "rope_interleaved" and left.get("sink") is None
    assert (right.kind, right["inner"], right["state_dim"], right["dt_rank"], right["conv_taps"], right["out_scale"]) == \
        ("selective_ssm", 40, 12, 5, 3, 1.3)
    r = spec.layers[1].feed_forward
    assert (r.kind, r["n_experts"], r["top"], r["intermediate_size"]) == ("routed_experts", 6, 2, 24)
    assert (r["score"], r["groups"], r["groups_kept"], r["renormalise"]) == ("sigmoid", 3, 2, True)
    assert r["shared"].kind == "swiglu" and r["shared"]["intermediate_size"] == 16
    capped = spec.layers[2]
    assert (capped.mixer["softcap"], capped.mixer["sink"], capped.mixer["window"]) == (15.0, "learned", 0)
    assert capped.feed_forward is None and not capped.mixer["shared_kv"]
    assert spec.layers[3].mixer["shared_kv"] and spec.layers[3].mixer["softcap"] == 8.0
    other = spec_of(CONFIGS["r"])
    assert other.layers[0].mixer["position"].kind == "none" and other.layers[4].mixer["softcap"] == 0.0
    assert other.layers[3].mixer["keep_first"] == 0 and other.layers[3].mixer["window"] == 7
    assert spec_of(CONFIGS["q"]).layers[0].feed_forward["groups"] == 1


def test_a_borrowing_layer_runs_on_its_lenders_storage():
    assert [e.cache_of for e in spec_of(CONFIGS["p"]).schedule] == [None, None, None, 2]
    assert [e.cache_of for e in spec_of(CONFIGS["q"]).schedule] == [None, None, None, 1, 1]
    assert [e.cache_of for e in spec_of(CONFIGS["r"]).schedule] == [None, None, None, None, 0]


def test_tensor_list_matches_the_checkpoint_names():
    from gguf2bin_b200.engine.model import expected_tensors
    for name, cfg in CONFIGS.items():
        exp = expected_tensors(spec_of(cfg))
        have = make_weights(cfg, SEEDS[name])
        assert {k for k, e in exp.items() if not e.optional} == set(have) - {k for k, e in exp.items() if e.optional}
        for k, v in have.items():
            assert tuple(exp[k].shape) == v.shape, k
        assert exp["final.norm.alpha"].shape == () and exp["l0.norm1.b"].shape == (cfg["width"],)
    exp = expected_tensors(spec_of(CONFIGS["p"]))
    assert exp["l0.mix.q"].shape == (2 * 4 * 16, 64) and exp["l0.mix.k"].shape == (2 * 2 * 16, 64)
    assert exp["l0.mix.v"].shape == (2 * 24, 64) and exp["l0.mix.lq1"].shape == (16,)
    assert "l3.mix.k" not in exp and exp["l2.mix.sink"].shape == (4,) and exp["l1.mix.left.g"].shape == (3, 64)
    assert exp["l1.mix.right.x"].shape == (5 + 2 * 12, 40) and exp["l1.mix.right.A_log"].shape == (40, 12)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="retention"), "not a mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "not a feed-forward"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "must be even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "at most dim"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "at least 1"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=4), "equal groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "equal groups"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "must be an object"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "no keys and values of its own"),
    (lambda c: c["layers"][3]["mixer"].update(kv_heads=1), "differs"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "no keys and values of its own"),
    (lambda c: c.pop("norm"), "norm.eps"),
    (lambda c: c.update(layers=[]), "non-empty"),
])
def test_reader_refuses_what_it_cannot_build(change, message):
    from gguf2bin_b200.config import ConfigError
    cfg = copy.deepcopy(CONFIGS["p"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        spec_of(cfg)


def test_random_weights_for_the_design_can_be_written_and_read(tmp_path):
    """``synth``'s writer knows the design's tensors, the one without a shape included."""
    from gguf2bin_b200.weights import write_random_model
    write_random_model(tmp_path / "m", CONFIGS["r"], 5, "float32")
    W = MP.read_safetensors(tmp_path / "m" / "model.safetensors")
    assert W["final.norm.alpha"].shape == () and W["l2.mix.right.A_log"].shape == (28, 3)
    logits = MP.forward(CONFIGS["r"], W, [3, 1, 4, 1, 5, 9, 2, 6])
    assert logits.shape == (8, 130) and np.isfinite(logits).all()


# ---- facts about the plain mechanisms -------------------------------------------------------------
def test_visibility_rule():
    assert all(MP.visible(i, j) for i in range(9) for j in range(i + 1)) and not MP.visible(3, 4)
    assert MP.visible(25, 6, 20, 3) and not MP.visible(26, 6, 20, 3)          # the window's far edge
    assert MP.visible(500, 2, 20, 3) and not MP.visible(500, 3, 20, 3)        # the last kept token, and the next one
    assert MP.visible(9, 9, 1, 0) and not MP.visible(9, 8, 1, 0)
    for i in range(70):
        for w, k in [(0, 0), (5, 0), (5, 3), (1, 1), (7, 20)]:
            assert list(MP.visible_keys(i, w, k)) == [j for j in range(i + 1) if MP.visible(i, j, w, k)]


def test_the_sink_takes_its_share_and_gives_nothing():
    """With all scores zero and a sink s, n visible keys share n / (n + e^s) of the weight equally."""
    rng = np.random.default_rng(0)
    v = rng.standard_normal((5, 1, 3))
    q, k = np.zeros((5, 2, 4)), rng.standard_normal((5, 1, 4))
    sink = np.array([0.0, 1.3])
    out = MP.attend(q, k, v, 0.5, sink=sink)
    for i in range(5):
        for h in range(2):
            assert np.allclose(out[i, h], v[:i + 1, 0].sum(0) / (i + 1 + math.exp(sink[h])))
    assert np.allclose(MP.attend(q, k, v, 0.5)[4, 0], v[:, 0].mean(0))


def test_capped_scores_stay_below_the_cap():
    """A huge score counts as the cap: two keys far above it share the weight equally."""
    q = np.full((2, 1, 2), 100.0)
    k = np.array([[[50.0, 50.0]], [[500.0, 500.0]]])
    v = np.array([[[1.0]], [[3.0]]])
    assert abs(MP.attend(q, k, v, 1.0, softcap=5.0)[1, 0, 0] - 2.0) < 1e-9
    assert abs(MP.attend(q, k, v, 1.0)[1, 0, 0] - 3.0) < 1e-9


def test_rotation_frequencies():
    f, mult = MP.rotation_frequencies(dict(dims=8, base=100.0))
    assert mult == 1.0 and np.allclose(f, [1.0, 100.0 ** -0.25, 0.1, 100.0 ** -0.75])
    g, mult = MP.rotation_frequencies(dict(dims=8, base=100.0, scaling=dict(factor=8.0, original=40, fast=4.0, slow=1.5)))
    assert abs(mult - (0.1 * math.log(8.0) + 1.0)) < 1e-12
    # pair(t) = 8 ln(40 / (2 pi t)) / (2 ln 100): 0.40 at 4 turns, 1.26 at 1.5: the ramp runs from pair 0 to pair 2
    assert np.allclose(g, [f[0], f[1] * (0.5 + 0.5 / 8.0), f[2] / 8.0, f[3] / 8.0])
    x = np.arange(12.0).reshape(1, 1, 12)
    y = MP.rotate_neighbours(x, [3], dict(dims=4, base=10.0))
    assert np.allclose(y[0, 0, 4:], x[0, 0, 4:])
    a = 3 * 1.0
    assert np.allclose(y[0, 0, :2], [0 * math.cos(a) - 1 * math.sin(a), 1 * math.cos(a) + 0 * math.sin(a)])


def test_router_groups():
    z = np.log(np.array([0.9, 0.1, 0.5, 0.45, 0.6, 0.2]) / (1 - np.array([0.9, 0.1, 0.5, 0.45, 0.6, 0.2])))
    chosen, w = MP.route(z, 2, 1, 1)
    assert list(chosen) == [0, 4] and np.allclose(w, [0.9 / 1.5, 0.6 / 1.5])
    # three groups of two score 1.0, 0.95, 0.8: with two kept, expert 4 (0.6) is out of reach
    chosen, w = MP.route(z, 2, 3, 2)
    assert list(chosen) == [0, 2] and np.allclose(w, [0.9 / 1.4, 0.5 / 1.4])
    chosen, _ = MP.route(z, 2, 3, 1)
    assert list(chosen) == [0, 1]
    assert MP.routing_margin(z, 2, 3, 2) == pytest.approx(min((0.95 - 0.8) / 0.95, (0.5 - 0.45) / 0.5))


def test_state_space_branch_forgets_nothing_it_should_keep():
    """The recurrence a token at a time equals the closed form for a constant input."""
    m = dict(inner=2, state=3, dt_rank=1, conv=1)
    t = {"in": np.array([[1.0], [0.0], [0.0], [0.0]]), "conv": np.ones((2, 1)), "conv.b": np.zeros(2),
         "x": np.array([[0.0, 0.0]] + [[1.0, 0.0]] * 6), "dt": np.zeros((2, 1)), "dt.b": np.array([0.3, 0.0]),
         "A_log": np.zeros((2, 3)), "D": np.zeros(2), "o": np.eye(2)}
    h = np.ones((6, 1))
    y = MP.selective_scan(h, m, t, "")
    x = MP.silu(1.0)
    dt = MP.softplus(0.3)
    a = math.exp(-dt)
    S = 0.0
    for i in range(6):
        S = a * S + dt * x * x                       # B = C = x on every state entry of channel 0
        assert abs(y[i, 0] - 3 * S * x * MP.silu(0.0)) < 1e-12       # z = 0: the gate is silu(0) = 0
    assert np.allclose(y, 0.0)


def test_difference_of_maps():
    W = weights("p")
    lam = MP.difference_lambda(W, "l0.mix.", 0.4)
    assert lam == pytest.approx(math.exp(W["l0.mix.lq1"] @ W["l0.mix.lk1"]) - math.exp(W["l0.mix.lq2"] @ W["l0.mix.lk2"]) + 0.4)
