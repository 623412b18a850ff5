"""Mopitar on the device against the plain implementation: each mechanism's part alone (with weights
or inputs made so that a far key, a window's edge, the kept first tokens, a sink or a lost state
shows), then whole models of three small configurations in every way of cutting the work (whole
prompts, token by token, portions down to two tokens, unequal batches, slots and pages used again,
long decoding over page and window borders), and greedy generation through the library's entry
point, its command line and trace replay."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import assert_close
from levolix_helpers import assert_rows_close
from mopitar_helpers import CONFIGS, clear_tokens, mixer_weights, mlp_weights, model_folder, plain_logits
from part_runner import DEV, DTYPES, bf, close, dev, run_part, step_ctx
from plain import mopitar_plain as MP

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
EPS = 1e-5

CUTS = [([], []), ([1] * 199, [1] * 99), ([2] * 99, [2] * 50), ([3, 1, 1, 2, 30], [17, 2])]


def bind(part, W, dtype, pre="mix."):
    part.bind({pre + k: dev(v, DTYPES[dtype]) for k, v in W.items()})
    return part


def rot_of(dims, scaling=None, base=1e4):
    if not dims:
        return None
    r = dict(dims=dims, base=base)
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


# ----------------------------------------------------------------------------
# the norm without statistics, the scaled join, the squared rectifier
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("T,H", [(5, 64), (3, 61), (70, 256)])
def test_tanh_norm_and_scaled_join(T, H):
    from gguf2bin_b200 import kernels
    rng = np.random.default_rng(T + H)
    x, w, b = rng.standard_normal((T, H)) * 3, 1 + 0.3 * rng.standard_normal(H), rng.standard_normal(H)
    alpha = 0.37
    ref = np.tanh(alpha * x) * w + b
    for dtype in ("float32", "bfloat16"):
        out = torch.empty((T, H), dtype=DTYPES[dtype], device=DEV)
        kernels.tanh_norm(dev(x), dev([alpha]), dev(w), dev(b), out)
        close(out.float().cpu().numpy(), ref, dtype, "tanh norm", loose=0.5)
    rows = [T - 1, 0, T // 2]
    out = torch.empty((3, H), dtype=torch.float32, device=DEV)
    kernels.tanh_norm(dev(x), dev([alpha]), dev(w), dev(b), out, torch.tensor(rows, dtype=torch.int32, device=DEV))
    close(out.cpu().numpy(), ref[rows], "float32", "tanh norm of chosen rows")
    y1, y2, s1, s2 = rng.standard_normal((T, H)), rng.standard_normal((T, H)), rng.standard_normal(H), rng.standard_normal(H)
    xs = dev(x)
    kernels.scaled_join(xs, dev(y1), dev(s1), dev(y2), dev(s2))
    close(xs.cpu().numpy(), x + y1 * s1 + y2 * s2, "float32", "scaled join of two")
    xs = dev(x)
    kernels.scaled_join(xs, dev(y1), dev(s1))
    close(xs.cpu().numpy(), x + y1 * s1, "float32", "scaled join of one")
    for dtype in ("float32", "bfloat16"):          # the next layer's norm in the same pass
        xs, out = dev(x), torch.empty((T, H), dtype=DTYPES[dtype], device=DEV)
        kernels.scaled_join(xs, dev(y1), dev(s1), dev(y2), dev(s2), norm=(dev([alpha]), dev(w), dev(b)), normed_out=out)
        joined = x + y1 * s1 + y2 * s2
        close(xs.cpu().numpy(), joined, "float32", "scaled join in front of a norm")
        close(out.float().cpu().numpy(), np.tanh(alpha * joined) * w + b, dtype, "the norm behind a scaled join", loose=0.5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("ff,width", [(40, 64), (36, 60), (72, 96)])
def test_squared_rectifier_feed_forward(ff, width, dtype):
    from gguf2bin_b200.config.mopitar import _feed_forward
    from gguf2bin_b200.parts.feed_forward import ActMLP
    rng = np.random.default_rng(ff)
    W = {k: bf(v) for k, v in mlp_weights(rng, dict(kind="dense", ff=ff), width).items()}
    part = bind(ActMLP(_feed_forward(dict(kind="dense", ff=ff), "test"), width, DTYPES[dtype], DEV), W, dtype, "mlp.")
    h = bf(rng.standard_normal((77, width)))
    ctx = step_ctx([77], [0], [0], dtype)
    y = torch.zeros((77, width), dtype=torch.float32, device=DEV)
    part.forward(dev(h, DTYPES[dtype]), ctx, y)
    close(y.cpu().numpy(), MP.squared_relu_ff(h, W, ""), dtype, "squared rectifier")


# ----------------------------------------------------------------------------
# routed experts: sigmoid scores, groups
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,groups,shared", [(6, 2, (3, 2), 16), (8, 3, (2, 1), None), (4, 4, (4, 4), 12),
                                                      (3, 1, None, None), (16, 3, (4, 2), 24), (12, 4, (6, 2), None)])
def test_routed_experts(experts, top, groups, shared, dtype):
    """Choices and weights as the plain router makes them, a row alone and among 76 others."""
    from gguf2bin_b200.config.mopitar import _feed_forward
    from gguf2bin_b200.parts.feed_forward import RoutedExperts
    rng = np.random.default_rng(experts * 10 + top)
    width = 48
    mlp = dict(kind="moe", expert=dict(ff=24), router=dict(experts=experts, top=top))
    if groups:
        mlp["router"]["groups"] = dict(count=groups[0], keep=groups[1])
    if shared:
        mlp["shared"] = dict(ff=shared)
    W = {k: bf(v) for k, v in mlp_weights(rng, mlp, width).items()}
    part = bind(RoutedExperts(_feed_forward(mlp, "test"), width, DTYPES[dtype], DEV), W, dtype, "mlp.")
    g = (groups or (1, 1))
    h = []
    while len(h) < 77:                                  # rows whose choice is clear in 16 bits too
        row = bf(rng.standard_normal(width))
        if MP.routing_margin(row @ W["router"].T, top, g[0], g[1]) > 0.08:
            h.append(row)
    h = np.array(h)
    ref = MP.routed_ff(h, mlp, W, "")
    for rows in (slice(0, 77), slice(5, 6), slice(40, 42)):
        n = rows.stop - rows.start
        ctx = step_ctx([n], [0], [0], dtype)
        y = torch.zeros((n, width), dtype=torch.float32, device=DEV)
        part.forward(dev(h[rows], DTYPES[dtype]), ctx, y)
        close(y.cpu().numpy(), ref[rows], dtype, f"routed rows {rows}")
        y2 = torch.full((n, width), 9.0, dtype=torch.float32, device=DEV)
        part.forward_into(dev(h[rows], DTYPES[dtype]), ctx, y2)
        close(y2.cpu().numpy(), ref[rows], dtype, f"routed rows {rows}, stored")


# ----------------------------------------------------------------------------
# capped attention with a learned sink
# ----------------------------------------------------------------------------
def capped_part(m, W, width, dtype):
    from gguf2bin_b200.config.mopitar import _attention
    from gguf2bin_b200.parts.mixers import GQAAttention
    return bind(GQAAttention(_attention(m, "test", EPS), width, DTYPES[dtype], DEV), W, dtype)


def capped_config(H, G, D, V, rot, cap, scale=None):
    m = dict(heads=H, kv_heads=G, dim=D, vdim=V, scale=scale if scale is not None else 1.5 / np.sqrt(D))
    if cap:
        m["softcap"] = cap
    if rot:
        m["rot"] = rot_of(rot)
    return m


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,rot,cap", [
    (4, 2, 16, 24, 8, 4.0),          # part of a head turned, value heads larger than key heads
    (3, 1, 64, 64, 64, 6.0),         # a size the tensor-core kernels take
    (2, 2, 24, 8, 24, 3.0),
    (6, 3, 128, 128, 32, 10.0),
    (2, 1, 40, 56, 0, 5.0),          # no rotation
    (5, 5, 8, 8, 4, 0.0),            # no cap
    (1, 1, 80, 80, 80, 25.0),
    (2, 1, 64, 32, 64, 5.0),         # value heads smaller than key heads of a tensor-core size
    (2, 2, 64, 128, 32, 6.0),        # and larger: keys padded to 128
])
def test_capped_attention_part(H, G, D, V, rot, cap, dtype):
    """Rotation of neighbouring pairs, the score scale, the cap (the queries are large enough for it to
    bend the scores) and the sink, over two sequences and every way of cutting them."""
    rng = np.random.default_rng(H * 1000 + D)
    width = 40
    m = capped_config(H, G, D, V, rot, cap)
    W = {k: bf(v) for k, v in mixer_weights(rng, "attention", m, width).items()}
    part = capped_part(m, W, width, dtype)
    sharp = 2.0 if dtype == "float32" else 0.7
    hs = [bf(rng.standard_normal((n, width)) * sharp) for n in (200, 37)]
    ref = [MP.attention_mixer(h, m, W, "", EPS)[0] for h in hs]
    for cuts in CUTS + [([63, 1, 2, 62, 1, 1], [1, 1, 1]), ([64, 64, 1], [2, 2, 2])]:
        got = run_part(part, part.cache_need(), hs, cuts, dtype)
        for b in range(2):
            close(got[b], ref[b], dtype, f"capped attention {cuts[0][:4]} sequence {b}", loose=2.0)


def flagged_attention(D=16, rot=8, bump=14.0, width=24, seed=1, cap=30.0):
    """A capped attention whose scores get ``bump`` more for every key whose input row has its channel 0
    set to one (channel 1 of every row is one and feeds the query; both sit in the part of a head that
    is not turned): a flagged token takes nearly all the weight of every query that sees it."""
    rng = np.random.default_rng(seed)
    m = capped_config(2, 1, D, D, rot, cap, scale=0.25)
    W = mixer_weights(rng, "attention", m, width)
    for name in ("q", "k"):
        W[name] *= 0.3
        W[name][:, :2] = 0.0
    for head in range(2):
        W["q"][head * D + D - 1] = 0.0
        W["q"][head * D + D - 1, 1] = 8.0
    W["k"][D - 1] = 0.0
    W["k"][D - 1, 0] = bump / (8.0 * m["scale"])
    W["sink"][:] = 0.5
    return m, {k: bf(v) for k, v in W.items()}, width


def flagged_rows(rng, n, width, targets):
    h = rng.standard_normal((n, width))
    h[:, 0], h[:, 1] = 0.0, 1.0
    for t in targets:
        h[t, 0] = 1.0
    return bf(h)


@pytest.mark.parametrize("dtype,D", [("float32", 16), ("bfloat16", 16), ("bfloat16", 64), ("bfloat16", 128)])
@pytest.mark.parametrize("target", [0, 1, 63, 64, 127, 128, 300])
def test_a_far_key_among_hundreds(target, dtype, D):
    """One key of 700 takes the weight, at the first positions, at page borders and far back: every later
    query of a prompt, and every decoded one, must find it (heads of 64 and 128 in 16 bits run the
    tensor-core kernels)."""
    rng = np.random.default_rng(target)
    m, W, width = flagged_attention(D=D)
    part = capped_part(m, W, width, dtype)
    h = flagged_rows(rng, 700, width, [target])
    ref, (k, v) = MP.attention_mixer(h, m, W, "", EPS)
    plain = MP.attention_mixer(flagged_rows(np.random.default_rng(target), 700, width, []), m, W, "", EPS)[0]
    assert np.abs(ref[699] - plain[699]).max() > 0.2          # the key does matter at the far end
    for cuts in ([[]], [[690] + [1] * 10], [[target + 1, 650] + [1] * 49]):
        got = run_part(part, part.cache_need(), [h], cuts, dtype, slots=(2,), pages_per_seq=11)
        close(got[0], ref, dtype, f"far key at {target}, cuts {cuts[0][:3]}", loose=2.0)


def test_queries_of_zero_leave_the_sink_its_share():
    """All queries zero: every visible key and the sink (0.5) weigh exp(0) and exp(0.5)."""
    m, W, width = flagged_attention()
    W["q"][:] = 0.0
    part = capped_part(m, W, width, "float32")
    h = bf(np.random.default_rng(3).standard_normal((70, width)))
    got = run_part(part, part.cache_need(), [h], [[40] + [1] * 30], "float32", slots=(1,))[0]
    v = h @ W["v"].T
    mean = np.cumsum(v, 0) / (np.arange(1, 71) + np.exp(0.5))[:, None]
    close(got, np.concatenate([mean, mean], 1) @ W["o"].T, "float32", "sink's share")


# ----------------------------------------------------------------------------
# two score maps per head
# ----------------------------------------------------------------------------
def difference_part(m, W, width, dtype):
    from gguf2bin_b200.config.mopitar import _attention_2
    from gguf2bin_b200.parts.mixers import DiffAttention
    return bind(DiffAttention(_attention_2(m, "test", EPS), width, DTYPES[dtype], DEV), W, dtype)


def difference_config(H, G, D, V, window, keep, rot, scaling=None, diff=0.4):
    m = dict(heads=H, kv_heads=G, dim=D, vdim=V, scale=2.0 / np.sqrt(D), diff=diff)
    if window:
        m["mask"] = dict(size=window, keep_first=keep) if keep is not None else dict(size=window)
    if rot:
        m["rot"] = rot_of(rot, scaling)
    return m


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,window,keep,rot,scaling", [
    (4, 2, 16, 24, 20, 3, 8, (8.0, 40, 4.0, 1.5)),
    (2, 1, 64, 64, 70, 66, 64, (4.0, 96, 8.0, 0.5)),     # more kept tokens than a page has, a window longer than a page
    (3, 3, 8, 12, 1, 1, 8, None),                        # the token itself and the first one
    (2, 1, 128, 128, 64, 4, 32, (2.0, 64, 2.0, 1.0)),
    (2, 2, 24, 8, 7, None, 24, None),                    # a window alone
    (2, 1, 32, 16, 0, None, 16, None),                   # everything seen
    (1, 1, 12, 20, 33, 40, 0, None),                     # more kept tokens than the window is long; no rotation
    (2, 1, 128, 64, 40, 2, 64, None),                    # value heads half the size of key heads of 128
    (4, 2, 32, 64, 24, 5, 16, None),                     # and twice the size, stored at 64
])
def test_difference_attention_part(H, G, D, V, window, keep, rot, scaling, dtype):
    rng = np.random.default_rng(H * 1000 + D + window)
    width = 40
    m = difference_config(H, G, D, V, window, keep, rot, scaling)
    W = {k: bf(v) for k, v in mixer_weights(rng, "attention_2", m, width).items()}
    part = difference_part(m, W, width, dtype)
    hs = [bf(rng.standard_normal((n, width))) for n in (200, 37)]
    ref = [MP.difference_mixer(h, m, W, "", EPS) for h in hs]
    edge = max(window, 1)
    more = [([edge - 1, 1, 1, 1], [edge, 2]), ([63, 1, 2, 62, 1, 1], [1, 1, 1]), ([edge + (keep or 0), 1, 1, 2, 5], [2, 2, 2])]
    for cuts in CUTS + more:
        got = run_part(part, part.cache_need(), hs, cuts, dtype)
        for b in range(2):
            close(got[b], ref[b], dtype, f"two maps {cuts[0][:4]} sequence {b}", loose=3.0)


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype,D", [("float32", 16), ("bfloat16", 64), ("bfloat16", 128)])
@pytest.mark.parametrize("window,keep", [(20, 3), (64, 5), (70, 66), (9, 1), (40, 0), (130, 129), (70, 300)])
def test_window_edges_and_kept_tokens_stand_out(window, keep, decode, dtype, D):
    """Channel 0 of the input feeds nothing but a large value; tokens that carry it sit at the last kept
    position, at the first one that is not kept, and in the middle.  A query sees a flagged token or does
    not: the normed difference of the maps then points another way altogether, in the prompt's rows and
    in rows decoded one by one."""
    rng = np.random.default_rng(window * 7 + keep)
    width = 24
    m = difference_config(2, 1, D, D, window, keep, 8)
    W = mixer_weights(rng, "attention_2", m, width)
    W["q"][:, 0] = W["k"][:, 0] = 0.0
    W["v"][:, 0] = 40.0
    W = {k: bf(v) for k, v in W.items()}
    n = keep + 3 * window + 70
    mid = keep + window + 30
    flagged = [t for t in (keep - 1, keep, mid) if t >= 0]
    h = rng.standard_normal((n, width))
    h[:, 0] = 0.0
    for t in flagged:
        h[t, 0] = 1.0
    h = bf(h)
    ref = MP.difference_mixer(h, m, W, "", EPS)
    # a window or a count of kept tokens that is one off changes rows by far more than the comparison allows
    allowed = (2e-5 if dtype == "float32" else 3e-2) * 2.0 * max(1.0, np.abs(ref).max())
    for dw, dk in ((1, 0), (-1, 0), (0, 1), (0, -1)):
        if window + dw < 1 or keep + dk < 0:
            continue
        off = difference_config(2, 1, D, D, window + dw, keep + dk, 8)
        assert np.abs(MP.difference_mixer(h, off, W, "", EPS) - ref).max() > 1.5 * allowed, (dw, dk)
    part = difference_part(m, W, width, dtype)
    cuts = [[mid + window - 3] + [1] * (n - mid - window + 3)] if decode else [[mid + window - 1, 1, 1, 2]]
    got = run_part(part, part.cache_need(), [h], cuts, dtype, slots=(4,), pages_per_seq=11)[0]
    close(got, ref, dtype, f"window {window} keep {keep}", loose=2.0)


# ----------------------------------------------------------------------------
# the two-branch mixer: unit-normed gated attention beside the selective scan
# ----------------------------------------------------------------------------
def left_part(m, W, width, dtype, scale=1.0):
    from gguf2bin_b200.config.mopitar import _left
    from gguf2bin_b200.parts.mixers import GQAAttention
    return bind(GQAAttention(_left(m, "test", EPS, scale), width, DTYPES[dtype], DEV), W, dtype, "mix.left.")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,rot,cap", [(3, 1, 16, 8, 16, 20.0), (2, 1, 64, 64, 64, 6.0), (6, 2, 40, 64, 40, 3.0),
                                             (2, 2, 8, 12, 4, 2.0), (4, 4, 128, 128, 64, 10.0)])
def test_gated_unit_attention_part(H, G, D, V, rot, cap, dtype):
    rng = np.random.default_rng(H * 100 + D)
    width = 40
    m = capped_config(H, G, D, V, rot, cap, scale=4.0 / D)       # unit-normed q and k: |q . k| <= D
    W = {k: bf(v) for k, v in mixer_weights(rng, "left", m, width).items()}
    part = left_part(m, W, width, dtype, 0.7)
    hs = [bf(rng.standard_normal((n, width))) for n in (150, 37)]
    ref = [0.7 * MP.gated_unit_attention(h, m, W, "", EPS) for h in hs]
    for cuts in CUTS + [([63, 1, 2, 62, 1, 1], [1, 1, 1])]:
        got = run_part(part, part.cache_need(), hs, cuts, dtype)
        for b in range(2):
            close(got[b], ref[b], dtype, f"gated unit attention {cuts[0][:4]} sequence {b}", loose=2.0)


def ssm_part(m, W, width, dtype, scale=1.0):
    from gguf2bin_b200.config.mopitar import _right
    from gguf2bin_b200.parts.recurrent import SelectiveSSM
    return bind(SelectiveSSM(_right(m, "test", scale), width, DTYPES[dtype], DEV), W, dtype, "mix.right.")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inner,state,rank,taps", [(40, 12, 5, 3), (48, 40, 8, 2), (28, 3, 7, 1), (192, 20, 10, 3),
                                                   (36, 1, 1, 4), (20, 130, 16, 2), (130, 16, 8, 4), (64, 128, 4, 3)])
def test_selective_scan_part(inner, state, rank, taps, dtype):
    """States of 1 to 130 entries a channel (one to 32 lanes), channel counts that fill no block, 1 to 4
    taps; the first token is made huge, so that a state that is lost or not cleared shows later on."""
    rng = np.random.default_rng(inner + state)
    width = 40
    m = dict(inner=inner, state=state, dt_rank=rank, conv=taps)
    W = {k: bf(v) for k, v in mixer_weights(rng, "right", m, width).items()}
    part = ssm_part(m, W, width, dtype, 1.3)
    hs = [bf(rng.standard_normal((n, width))) for n in (120, 37)]
    hs[0][0] *= 6.0
    ref = [1.3 * MP.selective_scan(h, m, W, "") for h in hs]
    for cuts in CUTS + [([15, 1, 16, 17, 1, 1], [1, 1, 1]), ([64, 1, 1], [16, 16, 5])]:
        got = run_part(part, part.cache_need(), hs, cuts, dtype)
        for b in range(2):
            close(got[b], ref[b], dtype, f"selective scan {cuts[0][:4]} sequence {b}", loose=2.0)


def test_a_state_carried_over_hundreds_of_tokens():
    """500 tokens in one step, then 20 one by one: the slowest channels still hold the first token."""
    rng = np.random.default_rng(9)
    width = 32
    m = dict(inner=24, state=8, dt_rank=4, conv=2)
    W = mixer_weights(rng, "right", m, width)
    W["A_log"][:6] = -7.0                                   # six channels that forget very slowly
    W["dt.b"][:6] = -3.0
    W = {k: bf(v) for k, v in W.items()}
    h = bf(rng.standard_normal((520, width)))
    h[0] *= 20.0
    ref = MP.selective_scan(h, m, W, "")
    calm = h.copy()
    calm[0] /= 20.0
    assert np.abs(ref[519] - MP.selective_scan(calm, m, W, "")[519]).max() > 1e-3       # still the first token's doing
    part = ssm_part(m, W, width, "float32")
    got = run_part(part, part.cache_need(), [h], [[500] + [1] * 20], "float32", slots=(2,), pages_per_seq=9)[0]
    close(got, ref, "float32", "long state", loose=2.0)


# ----------------------------------------------------------------------------
# whole models
# ----------------------------------------------------------------------------
CASES = [(n, d) for n in ("p", "q", "r") for d in ("float32", "bfloat16")]
LENGTHS = {"p": [70, 9, 131, 1, 33], "q": [80, 1, 140, 17], "r": [131, 2, 64, 65, 23]}


@pytest.fixture(scope="module")
def engines():
    from gguf2bin_b200.engine import Engine, Model
    made = {}

    def get(name, dtype, max_tokens=2048):
        key = (name, dtype, max_tokens)
        if key not in made:
            made[key] = Engine(Model.from_folder(model_folder(name), dtype=dtype), max_tokens=max_tokens)
        return made[key]
    return get


def requests_of(name):
    return [list(clear_tokens(name, n, i)) for i, n in enumerate(LENGTHS[name])]


def run_in_portions(eng, toks, sizes):
    from gguf2bin_b200.engine import StepEntry
    seq, got, done = eng.open_sequence(), [], 0
    sizes = list(sizes)
    while done < len(toks):
        n = min(sizes.pop(0) if sizes else len(toks), len(toks) - done)
        got.append(eng.step([StepEntry(seq, toks[done:done + n], range(n))]).cpu().numpy())
        done += n
    eng.close_sequence(seq)
    return np.concatenate(got)


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts(engines, name, dtype):
    eng = engines(name, dtype)
    for i, toks in enumerate(requests_of(name)):
        assert_rows_close(run_in_portions(eng, toks, []), plain_logits(name, toks), dtype,
                          f"mopitar {name}/{dtype} request {i} whole")


@pytest.mark.parametrize("name,dtype", CASES)
def test_token_by_token_and_portions(engines, name, dtype):
    """The same logits however the prompt is cut: every token alone from the first one on; portions
    of two; mixed portions that end on, before and behind page and window borders."""
    eng = engines(name, dtype)
    toks = requests_of(name)[2 if name != "r" else 0][:110]
    ref = plain_logits(name, toks)
    whole = run_in_portions(eng, toks, [])
    for what, sizes in [("one by one", [1] * len(toks)), ("twos", [2] * len(toks)), ("mixed", [3, 2, 5, 1, 2, 50, 1, 2, 2]),
                        ("window edge", [19, 1, 1, 4, 1, 6, 1, 1, 36, 1]), ("page edge", [63, 1, 1, 2]), ("page", [64, 2, 2])]:
        got = run_in_portions(eng, toks, sizes)
        assert_rows_close(got, ref, dtype, f"mopitar {name}/{dtype} {what}")
        if dtype == "float32":       # the cut changes nothing but the order of a few additions
            assert np.abs(got - whole).max() <= 2e-5 * max(1.0, np.abs(ref).max()), what


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_with_reuse(engines, name, dtype):
    """Batches of up to three requests: prompts (all but the last 6 tokens, at least one) in one step,
    then one token each, shorter requests ending earlier; the cache holds one batch, so every batch
    gets the slots, states and pages that the one before gave back."""
    from gguf2bin_b200.engine import StepEntry
    reqs = requests_of(name)
    batches = [reqs[i:i + 3] for i in range(0, len(reqs), 3)] * 2
    need = max(sum(-(-len(t) // 64) * 64 for t in b) for b in batches)
    eng = engines(name, dtype, need)
    for bi, batch in enumerate(batches):
        seqs = [eng.open_sequence() for _ in batch]
        heads = [max(1, len(t) - 6) for t in batch]
        got = [[] for _ in batch]
        out = eng.step([StepEntry(s, t[:h], range(h)) for s, t, h in zip(seqs, batch, heads)]).cpu().numpy()
        o = 0
        for j, h in enumerate(heads):
            got[j].append(out[o:o + h])
            o += h
        done = list(heads)
        live = [j for j in range(len(batch)) if done[j] < len(batch[j])]
        for j in range(len(batch)):
            if j not in live:
                eng.close_sequence(seqs[j])
        while live:
            out = eng.step([StepEntry(seqs[j], [batch[j][done[j]]], [0]) for j in live]).cpu().numpy()
            for r, j in enumerate(live):
                got[j].append(out[r:r + 1])
                done[j] += 1
            for j in [j for j in live if done[j] == len(batch[j])]:
                eng.close_sequence(seqs[j])
            live = [j for j in live if done[j] < len(batch[j])]
        for j, toks in enumerate(batch):
            assert_rows_close(np.concatenate(got[j]), plain_logits(name, toks), dtype,
                              f"mopitar {name}/{dtype} batch {bi} request {j}")
    assert eng.cache.table.pages.n_held == 0 and eng.cache.table.slots.n_held == 0


@pytest.mark.parametrize("name,dtype", [("p", "float32"), ("q", "bfloat16"), ("r", "bfloat16"), ("q", "float32")])
def test_long_decoding(engines, name, dtype):
    """A short prompt, then 120 tokens one by one: the window passes over decoded tokens and past the
    kept ones, pages begin; beside a second sequence that started elsewhere."""
    from gguf2bin_b200.engine import StepEntry
    eng = engines(name, dtype)
    a, b = list(clear_tokens(name, 150, 70)), list(clear_tokens(name, 181, 71))
    sa, sb = eng.open_sequence(), eng.open_sequence()
    out = eng.step([StepEntry(sa, a[:30], range(30)), StepEntry(sb, b[:61], range(61))]).cpu().numpy()
    ga, gb = [out[:30]], [out[30:]]
    for t in range(120):
        out = eng.step([StepEntry(sa, [a[30 + t]], [0]), StepEntry(sb, [b[61 + t]], [0])]).cpu().numpy()
        ga.append(out[:1])
        gb.append(out[1:])
    eng.close_sequence(sa)
    eng.close_sequence(sb)
    assert_rows_close(np.concatenate(ga), plain_logits(name, a), dtype, f"mopitar {name}/{dtype} long decoding a")
    assert_rows_close(np.concatenate(gb), plain_logits(name, b), dtype, f"mopitar {name}/{dtype} long decoding b")


def plain_greedy(name, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(plain_logits(name, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["p", "r"])
def test_greedy_generation_through_the_entry_point(name):
    """LLM.generate (scheduler, decode session with its graph) against the plain implementation's
    argmax, several unequal prompts at once."""
    from gguf2bin_b200.api import LLM
    llm = LLM(model_folder(name), dtype="float32", max_tokens=2048)
    prompts = [list(clear_tokens(name, n, 90 + i)) for i, n in enumerate([9, 1, 66, 30])]
    for _ in range(2):                         # the second call finds slots, pages and graphs of the first
        outs = llm.generate(prompts, n=30, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0)
        for p, o in zip(prompts, outs):
            toks = list(p)
            for t in o.tokens:
                row = plain_logits(name, toks)[-1]
                assert row[t] >= row.max() - 2e-5 * max(1.0, np.abs(row).max())
                toks.append(t)
            assert len(o.tokens) == 30
    a = llm.generate(prompts[:2], n=12, seed=5)
    b = llm.generate(prompts[:2], n=12, seed=5)
    assert [o.tokens for o in a] == [o.tokens for o in b]
    assert llm.engine.cache.table.pages.n_held == 0 and llm.engine.cache.table.slots.n_held == 0


def test_the_programs(tmp_path):
    """info and run of the command line, random weights for the design's config.json, and trace replay."""
    folder = model_folder("p")
    exe = [sys.executable, str(ROOT / "bin" / "gguf2bin_b200")]
    out = subprocess.run(exe + ["info", str(folder)], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "Mopitar" in out.stdout + out.stderr, out.stderr[-2000:]
    prompt = list(clear_tokens("p", 7, 40))
    out = subprocess.run(exe + ["run", str(folder), "--tokens", ",".join(map(str, prompt)), "-n", "6", "-t", "0",
                                "--repeat-penalty", "1", "--dtype", "float32", "--ignore-eos"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert [int(t) for t in out.stdout.split()] == prompt + plain_greedy("p", prompt, 6)
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(CONFIGS["r"]))
    made = tmp_path / "made"
    out = subprocess.run(exe + ["synth", str(made), "--config", str(cfg_file), "--seed", "3", "--dtype", "float32"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    W = MP.read_safetensors(made / "model.safetensors")
    toks = np.random.default_rng(4).integers(0, CONFIGS["r"]["vocab"], 9).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:6], "want": [0, 5]},
                                     {"id": "b", "tokens": toks[:1], "want": [0]}], "end": ["b"]},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[6:7], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[7:8], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": toks[8:], "want": [0]}], "end": ["a"]}]
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(made), "--dtype", "float32",
                           "--out", str(out_dir), "--max-tokens", "64"],
                          input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    assert not (out_dir / "1.f32").exists()
    got = np.concatenate([np.fromfile(out_dir / f"{i}.f32", "<f4").reshape(-1, CONFIGS["r"]["vocab"]) for i in (0, 2, 3)])
    ref = MP.forward(CONFIGS["r"], W, toks)
    assert_close(got, ref[[0, 5, 0, 7, 8]], "float32", "mopitar trace replay")
