"""Sominex on the device against the plain implementation: each mechanism's part alone (with weights
or inputs made so that a far block, a window's or a block's edge, the first tokens or a lost state
shows), then whole models of three small configurations in every way of cutting the work (whole
prompts, token by token, portions down to two tokens, unequal batches, slots and pages used again,
long decoding over page, window and block borders), and greedy generation through the library's
entry point, its command line and trace replay."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import assert_close
from levolix_helpers import assert_rows_close
from part_runner import DEV, DTYPES, bf, close, dev, names_of, run_part, step_ctx
from plain import sominex_plain as SP
from sominex_helpers import CONFIGS, clear_tokens, mixer_weights, mlp_weights, model_folder, plain_logits

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
EPS = 1e-5

CUTS = [([], []), ([1] * 199, [1] * 99), ([2] * 99, [2] * 50), ([3, 1, 1, 2, 30], [17, 2])]


# ----------------------------------------------------------------------------
# attention: a window of tokens, means of whole blocks in front of it
# ----------------------------------------------------------------------------
def attention_part(m, W, width, dtype):
    """The part as the configuration reader describes it (tensor names under ``mix.``)."""
    from gguf2bin_b200.config.sominex import _attention
    from gguf2bin_b200.parts.mixers import GQAAttention
    part = GQAAttention(_attention(m, "test", EPS), width, DTYPES[dtype], DEV)
    part.bind({"mix." + k: dev(v, DTYPES[dtype]) for k, v in W.items()})
    return part


def attention_config(H, G, D, V, window, pool, rot, scaling=None, scale=None):
    m = dict(heads=H, kv_heads=G, dim=D, vdim=V, scale=scale if scale is not None else 1.5 / np.sqrt(D))
    if window:
        m["mask"] = dict(size=window, pool=pool) if pool else dict(size=window)
    if rot:
        m["rot"] = dict(dims=rot, base=1e4)
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,window,pool,rot,scaling", [
    (4, 2, 16, 24, 20, 5, 8, (8.0, 40, 4.0, 1.5)),       # blocks that straddle page borders, part of a head turned
    (3, 1, 64, 64, 70, 12, 64, (4.0, 96, 8.0, 0.5)),     # a window longer than a page
    (2, 2, 24, 8, 7, 3, 24, None),
    (6, 3, 128, 128, 64, 16, 32, (2.0, 64, 2.0, 1.0)),   # window and blocks that divide a page
    (2, 1, 64, 32, 33, 70, 64, None),                    # a block longer than the window and than a page
    (4, 4, 128, 128, 100, 64, 128, None),                # a block that is a page
    (2, 1, 8, 8, 1, 1, 4, None),                         # a window of the token itself behind blocks of one
    (2, 2, 40, 24, 3, 10, 0, None),                      # tokens that no query sees for a while; no rotation
    (3, 1, 16, 16, 50, 0, 16, (4.0, 32, 4.0, 1.0)),      # a window without blocks
    (2, 2, 32, 16, 0, 0, 16, None),                      # everything seen
    (5, 1, 64, 64, 20, 4, 32, None),                     # more query heads on a kv head than one block of threads takes
])
def test_attention_part(H, G, D, V, window, pool, rot, scaling, dtype):
    """Value norm, stretched rotation of part of a head, the score scale, the window and the blocks in
    front of it, over two sequences and every way of cutting them.  In 32-bit the queries are large, so
    that the softmax is sharp and a key or block wrongly seen, or wrongly hidden, changes the row."""
    rng = np.random.default_rng(H * 1000 + D + window)
    width = 40
    m = attention_config(H, G, D, V, window, pool, rot, scaling)
    W = {k: bf(v) for k, v in mixer_weights(rng, "attention", m, width).items()}
    part = attention_part(m, W, width, dtype)
    sharp = 2.0 if dtype == "float32" else 0.7         # in 16 bits a sharp softmax multiplies the scores' rounding
    hs = [bf(rng.standard_normal((n, width)) * sharp) for n in (200, 37)]
    keep = (lambda a: bf(a)) if dtype == "bfloat16" else None
    ref = [SP.attention_mixer(h, W, "", m, EPS, round_cache=keep) for h in hs]
    edge = max(window, 1)
    more = [([edge - 1, 1, 1, 1], [edge, 2]), ([63, 1, 2, 62, 1, 1], [1, 1, 1]),
            ([edge + (pool or 1) - 1, 1, 1, 2, 5], [2, 2, 2])]
    for cuts in CUTS + more:
        got = run_part(part, part.cache_need(), hs, cuts, dtype)
        for b in range(2):
            close(got[b], ref[b], dtype, f"attention {cuts[0][:4]} sequence {b}", loose=2.0)


def flagged_attention(window, pool, D=16, rot=8, bump=14.0, width=24, seed=1):
    """An attention part whose scores get ``bump`` more for every key whose input row has its channel 0
    set to one (channel 1 of every row is one and feeds the query; both sit in the part of a head that
    is not turned).  A flagged token takes nearly all the weight of every query that sees it; a block
    that holds it takes bump / pool more than its neighbours."""
    rng = np.random.default_rng(seed)
    m = attention_config(2, 1, D, D, window, pool, rot, scale=0.25)
    W = mixer_weights(rng, "attention", m, width)
    for name in ("q", "k"):
        W[name] *= 0.3
        W[name][:, :2] = 0.0
    for head in range(2):
        W["q"][head * D + D - 1] = 0.0
        W["q"][head * D + D - 1, 1] = 8.0
    W["k"][D - 1] = 0.0
    W["k"][D - 1, 0] = bump / (8.0 * m["scale"])
    W = {k: bf(v) for k, v in W.items()}
    return m, W, width


def flagged_rows(rng, n, width, targets):
    h = rng.standard_normal((n, width))
    h[:, 0], h[:, 1] = 0.0, 1.0
    for t in targets:
        h[t, 0] = 1.0
    return bf(h)


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window,pool", [(20, 5), (64, 16), (70, 12), (9, 24)])
def test_window_and_block_edges_stand_out(window, pool, decode):
    """One token's key is made to take the weight.  The last query of its window sees it, the next one
    does not; it comes back, as a share of its block's mean, with the first query that sees the whole
    block, and not one query earlier.  Targets: a block's first token, its last, one on a page border."""
    m, W, width = flagged_attention(window, pool)
    part = attention_part(m, W, width, "float32")
    rng = np.random.default_rng(window)
    n = 64 + 2 * window + 3 * pool
    for target in (pool, 2 * pool - 1, 63, 64):
        h = flagged_rows(rng, n, width, [target])
        ref = SP.attention_mixer(h, W, "", m, EPS)
        last_in = target + window - 1                                # the last query whose window holds it
        first_block = (target // pool) * pool + pool - 1 + window    # the first query that sees its block
        assert last_in + 1 < n and first_block < n
        rows = np.abs(ref).max()
        assert np.abs(ref[last_in] - ref[last_in + 1]).max() > 0.05 * rows
        if first_block - 1 > last_in:
            assert np.abs(ref[first_block] - ref[first_block - 1]).max() > 0.02 * rows
        cuts = ([target + 1] + [1] * n,) if decode else ([],)
        got = run_part(part, part.cache_need(), [h], cuts, "float32", slots=(2,))[0]
        close(got, ref, "float32", f"window {window} pool {pool} target {target}")


@pytest.mark.parametrize("decode", [False, True])
def test_a_block_far_back_among_hundreds(decode):
    """700 tokens: one early token is flagged, so its block's mean key stands above the forty-odd other
    blocks and the window's tokens at every late query.  Without it the late rows differ by much."""
    window, pool = 48, 16
    m, W, width = flagged_attention(window, pool, bump=16.0 * 16)
    part = attention_part(m, W, width, "float32")
    rng = np.random.default_rng(3)
    h = flagged_rows(rng, 700, width, [37])
    ref = SP.attention_mixer(h, W, "", m, EPS)
    plain = h.copy()
    plain[37, 0] = 0.0
    share = np.abs(ref[-30:] - SP.attention_mixer(plain, W, "", m, EPS)[-30:]).max()
    assert share > 0.3 * np.abs(ref[-30:]).max()
    cuts = ([600] + [1] * 100,) if decode else ([],)
    got = run_part(part, part.cache_need(), [h], cuts, "float32", slots=(4,), pages_per_seq=11)[0]
    close(got, ref, "float32", "a block far back")
    assert np.abs(got[-30:] - ref[-30:]).max() < 1e-3 * share


@pytest.mark.parametrize("D,window,pool", [(64, 10, 2), (128, 40, 3), (64, 130, 1)])
def test_hundreds_of_blocks_in_front_of_a_prompt_tile(D, window, pool):
    """16-bit prompts on the tensor cores: 900 tokens give several panels of 64 blocks in front of the
    window's pages, a last panel that is partly filled, and tiles whose rows see different numbers of
    blocks.  Two early tokens are flagged so that their blocks carry weight in every late row; the cuts
    put a tile's first row before, on and behind a block's and a page's edge."""
    m, W, width = flagged_attention(window, pool, D=D, rot=D // 2, bump=6.0 * pool)
    part = attention_part(m, W, width, "bfloat16")
    rng = np.random.default_rng(D + pool)
    hs = [flagged_rows(rng, 900, width, [5, 401]), flagged_rows(rng, 333, width, [64])]
    ref = [SP.attention_mixer(h, W, "", m, EPS, round_cache=bf) for h in hs]
    plain = hs[0].copy()
    plain[[5, 401], 0] = 0.0
    share = np.abs(ref[0][-50:] - SP.attention_mixer(plain, W, "", m, EPS, round_cache=bf)[-50:]).max()
    assert share > 0.1 * np.abs(ref[0][-50:]).max()
    for cuts in (([], []), ([129, 500], [200]), ([window + pool, 64, 2, 381], [65, 3]), ([700] + [1] * 200, [300] + [1] * 33)):
        got = run_part(part, part.cache_need(), hs, cuts, "bfloat16", pages_per_seq=15)
        for b in range(2):
            close(got[b], ref[b], "bfloat16", f"blocks in front of a tile {cuts[0][:3]} sequence {b}")


def test_first_tokens_of_a_sequence():
    """The first query sees itself alone (its output is its own normed value through the output
    product); the first ``window`` queries see everything so far and no block."""
    m, W, width = flagged_attention(6, 2)
    part = attention_part(m, W, width, "float32")
    rng = np.random.default_rng(8)
    h = flagged_rows(rng, 12, width, [])
    ref = SP.attention_mixer(h, W, "", m, EPS)
    v0 = SP.rms_divide((W["v"] @ h[0]).reshape(1, -1), EPS)[0]
    alone = np.tile(v0, 2) @ W["o"].T
    assert np.abs(ref[0] - alone).max() < 1e-9
    for cuts in (([],), ([1] * 12,), ([2, 1, 3],)):
        got = run_part(part, part.cache_need(), [h], cuts, "float32", slots=(1,))[0]
        close(got, ref, "float32", f"first tokens {cuts[0][:3]}")


# ----------------------------------------------------------------------------
# the two state mixers
# ----------------------------------------------------------------------------
def state_part(kind, m, W, width, dtype):
    from gguf2bin_b200.config.sominex import _mixer
    from gguf2bin_b200.parts.registry import mixer_class
    spec = _mixer(kind, m, "test", EPS)
    part = mixer_class(spec)(spec, width, DTYPES[dtype], DEV)
    part.bind({"mix." + k: dev(v, DTYPES[dtype]) for k, v in W.items()})
    return part


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,N,V,taps,parts", [(4, 2, 16, 8, 3, 4), (2, 1, 40, 20, 2, 1), (1, 1, 12, 20, 1, 5),
                                                (6, 3, 8, 4, 4, 2), (3, 3, 128, 64, 4, 3), (8, 2, 64, 32, 4, 1)])
def test_state_space_part(H, G, N, V, taps, parts, dtype):
    """Convolution with its bias over the three joined inputs, step sizes, scalar decays, the skip, the
    gate in front of the grouped norm.  The first token is made huge and one head forgets slowly, so a
    state that is lost or cleared on the way shows at every later token."""
    rng = np.random.default_rng(H * 100 + N + taps)
    width = 48
    m = dict(heads=H, groups=G, state=N, vdim=V, conv=taps, norm_groups=parts)
    W = mixer_weights(rng, "mamba2", m, width)
    W["A_log"][0] = -6.0
    W = {k: bf(v) for k, v in W.items()}
    part = state_part("mamba2", m, W, width, dtype)
    hs = [bf(rng.standard_normal((n, width))) for n in (70, 21)]
    hs[0][0] *= 20.0
    ref = [SP.mamba2_mixer(h, W, "", m, EPS) for h in hs]
    for cuts in CUTS + [([64, 1, 2], [1, 1, 19])]:
        got = run_part(part, part.cache_need(), hs, cuts, dtype)
        for b in range(2):
            close(got[b], ref[b], dtype, f"state space {cuts[0][:3]} sequence {b}", loose=2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,V,cap", [(3, 16, 8, 6.0), (2, 40, 24, 15.0), (1, 8, 12, 3.0), (4, 64, 64, 12.0),
                                       (2, 128, 32, 1.0), (5, 24, 48, 30.0)])
def test_mlstm_part(H, D, V, cap, dtype):
    """Capped gates, the running maximum from zero, the normaliser and its floor exp(-m), the norm per
    head with a weight over all heads, the sigmoid gate."""
    rng = np.random.default_rng(H * 100 + D)
    width = 48
    m = dict(heads=H, dim=D, vdim=V, gate_cap=cap)
    W = mixer_weights(rng, "mlstm", m, width)
    W["f.b"][0] = 9.0                                     # a head that forgets slowly
    W = {k: bf(v) for k, v in W.items()}
    part = state_part("mlstm", m, W, width, dtype)
    hs = [bf(rng.standard_normal((n, width))) for n in (70, 21)]
    hs[0][0] *= 6.0
    ref = [SP.mlstm_mixer(h, W, "", m, EPS) for h in hs]
    for cuts in CUTS + [([64, 1, 2], [1, 1, 19])]:
        got = run_part(part, part.cache_need(), hs, cuts, dtype)
        for b in range(2):
            close(got[b], ref[b], dtype, f"mlstm {cuts[0][:3]} sequence {b}", loose=2.0)


def test_mlstm_maximum_starts_at_zero_and_floors_the_normaliser():
    """Input gates far below zero: the running maximum stays at its start, 0, not at the largest gate seen,
    so the weights exp(i - m) are tiny and the read-out's denominator is its floor exp(-m) = 1."""
    rng = np.random.default_rng(5)
    width, H, D, V = 32, 2, 16, 8
    m = dict(heads=H, dim=D, vdim=V, gate_cap=20.0)
    W = mixer_weights(rng, "mlstm", m, width)
    W["i"] *= 0.05
    W["i.b"][:] = -9.0
    W = {k: bf(v) for k, v in W.items()}
    h = bf(rng.standard_normal((30, width)))
    ref = SP.mlstm_mixer(h, W, "", m, EPS)
    shifted = dict(W)
    shifted["i.b"] = W["i.b"] + 3.0                       # were m the largest gate, this would change nothing
    assert np.abs(SP.mlstm_mixer(h, shifted, "", m, EPS) - ref).max() > 1e-3 * np.abs(ref).max()
    part = state_part("mlstm", m, W, width, "float32")
    for cuts in (([],), ([1] * 30,), ([7, 2, 2],)):
        got = run_part(part, part.cache_need(), [h], cuts, "float32", slots=(2,))[0]
        close(got, ref, "float32", f"mlstm floor {cuts[0][:3]}")


@pytest.mark.parametrize("kind", ["mamba2", "mlstm"])
def test_a_token_far_back_still_counts(kind):
    """520 tokens, the first one huge, heads that forget slowly: 500 in one prompt step, then 20 one by
    one.  The plain recurrence says how much of the end's output is the first token's doing; a state
    lost, cleared or decayed wrongly on the way would miss it by that much."""
    rng = np.random.default_rng(11)
    width = 32
    if kind == "mamba2":
        m = dict(heads=2, groups=1, state=16, vdim=24, conv=2, norm_groups=2)
        W = mixer_weights(rng, kind, m, width)
        W["A_log"][:] = [-8.0, 1.0]
        plain = lambda x: SP.mamba2_mixer(x, W, "", m, EPS)
    else:
        m = dict(heads=2, dim=16, vdim=24, gate_cap=15.0)
        W = mixer_weights(rng, kind, m, width)
        W["f"] *= 0.1
        W["f.b"][:] = [7.0, 0.0]
        W["i"] *= 0.1
        plain = lambda x: SP.mlstm_mixer(x, W, "", m, EPS)
    W = {k: bf(v) for k, v in W.items()}
    h = bf(rng.standard_normal((520, width)))
    h[0] *= 8.0
    ref = plain(h)
    without = h.copy()
    without[0] = 0.0
    share = np.abs(ref[-20:] - plain(without)[-20:]).max()
    assert share > 1e-2 * np.abs(ref[-20:]).max()
    part = state_part(kind, m, W, width, "float32")
    got = run_part(part, part.cache_need(), [h], ([500] + [1] * 20,), "float32", slots=(1,), pages_per_seq=10)[0]
    assert np.abs(got[-20:] - ref[-20:]).max() < 2e-3 * share
    close(got, ref, "float32", f"{kind} over 520 tokens", loose=3.0)


# ----------------------------------------------------------------------------
# the block's norm and token shift, the feed-forwards
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [60, 256, 1000])
def test_norm_and_token_shift_over_steps(width, dtype):
    """h = norm(x) and the mixer's copy h + (h_before - h) mu, the row before taken from the step where
    there is one and from the slot otherwise; slots hold junk beyond what a sequence wrote, and
    the first token of a sequence mixes with zeros whatever its slot held."""
    from gguf2bin_b200 import kernels
    rng = np.random.default_rng(width)
    xs = [rng.standard_normal((n, width)).astype(np.float32) * 3 for n in (29, 8)]
    w, mu = bf(1 + 0.3 * rng.standard_normal(width)), bf(rng.uniform(-0.5, 1.5, width))
    refs = []
    for x in xs:
        h = SP.rms_divide(x.astype(np.float64), EPS) * w[None, :]
        refs.append((h, SP.token_shift(h, mu)))
    tol = 1e-5 if dtype == "float32" else 2e-2
    for cuts in (([], []), ([1] * 29, [1] * 8), ([2] * 15, [2] * 4), ([5, 1, 1, 3, 19], [1, 7])):
        kept = torch.full((6, width), 9.0, dtype=torch.float32, device=DEV)
        slots, done = (4, 2), [0, 0]
        kept[list(slots)] = 0.0
        cuts = [list(c) for c in cuts]
        while any(d < len(x) for d, x in zip(done, xs)):
            live = [b for b in range(2) if done[b] < len(xs[b])]
            sizes = [min(cuts[b].pop(0) if cuts[b] else len(xs[b]), len(xs[b]) - done[b]) for b in live]
            ctx = step_ctx(sizes, [done[b] for b in live], [slots[b] for b in live], dtype,
                           single=all(n == 1 for n in sizes))
            x = torch.cat([dev(xs[b][done[b]:done[b] + n]) for b, n in zip(live, sizes)])
            h = torch.empty(tuple(x.shape), dtype=DTYPES[dtype], device=DEV)
            hs = torch.empty_like(h)
            kernels.norm_shift(x, dev(w), dev(mu), kept, ctx, EPS, h, hs)
            o = 0
            for b, n in zip(live, sizes):
                for got, ref in ((h, refs[b][0]), (hs, refs[b][1])):
                    err = np.abs(got[o:o + n].float().cpu().numpy() - ref[done[b]:done[b] + n]).max()
                    assert err < tol * max(1.0, np.abs(ref).max()), (sizes, b, done[b], err)
                done[b] += n
                o += n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,ff,limit", [(64, 40, 1.0), (60, 28, 4.0), (128, 320, 0.5), (96, 72, 2.5)])
def test_capped_glu_part(width, ff, limit, dtype):
    """Inputs large enough that the gate's cap and both sides of the up value's bite."""
    from gguf2bin_b200.config.sominex import _feed_forward
    from gguf2bin_b200.parts.registry import feed_forward_class
    rng = np.random.default_rng(ff)
    mlp = dict(kind="dense", ff=ff, limit=limit)
    W = {k: bf(v) for k, v in mlp_weights(rng, mlp, width).items()}
    spec = _feed_forward(mlp, "test")
    part = feed_forward_class(spec)(spec, width, DTYPES[dtype], DEV)
    part.bind({"mlp." + k: dev(v, DTYPES[dtype]) for k, v in W.items()})
    h = bf(rng.standard_normal((77, width)) * 1.5)
    g, u = h @ W["gate"].T, h @ W["up"].T
    assert (g > limit).mean() > 0.02 and (u > limit).mean() > 0.02 and (u < -limit).mean() > 0.02
    ref = SP.capped_glu(h, W, "", limit)
    for n in (77, 3, 1):
        y = torch.zeros((n, width), dtype=torch.float32, device=DEV)
        part.forward(dev(h[:n], DTYPES[dtype]), step_ctx([n], [0], [0], dtype), y)
        close(y.cpu().numpy(), ref[:n], dtype, f"capped glu, {n} rows")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,ff,shared,scale,width", [(5, 2, 24, 16, 1.7, 64), (3, 1, 56, None, 1.0, 96),
                                                         (2, 2, 20, 12, 1.2, 60), (16, 4, 64, 128, 2.5, 128)])
def test_routed_experts_with_scale_and_shared_expert(E, top, ff, shared, scale, width, dtype):
    """Softmax over all experts, the largest chosen, their scores times a constant and not renormalised,
    a shared expert for every token; a token's result does not depend on the tokens beside it."""
    from gguf2bin_b200.config.sominex import _feed_forward
    from gguf2bin_b200.parts.registry import feed_forward_class
    rng = np.random.default_rng(E * 7 + top)
    mlp = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=E, top=top, scale=scale))
    if shared:
        mlp["shared"] = dict(ff=shared)
    W = {k: bf(v) for k, v in mlp_weights(rng, mlp, width).items()}
    spec = _feed_forward(mlp, "test")
    part = feed_forward_class(spec)(spec, width, DTYPES[dtype], DEV)
    part.bind({"mlp." + k: dev(v, DTYPES[dtype]) for k, v in W.items()})
    rows = []
    while len(rows) < 77:                                  # rows whose choice is clear
        h = bf(rng.standard_normal((1, width)))
        s = -np.sort(-SP.route(h, W["router"], top, 1.0)[2][0])
        if top == E or (s[top - 1] - s[top]) / s[top - 1] > 0.2:
            rows.append(h[0])
    h = np.stack(rows)
    ref = SP.routed_experts(h, W, "", mlp)
    outs = {}
    for n in (77, 5, 1):
        y = torch.zeros((n, width), dtype=torch.float32, device=DEV)
        part.forward(dev(h[:n], DTYPES[dtype]), step_ctx([n], [0], [0], dtype), y)
        outs[n] = y.cpu().numpy()
        close(outs[n], ref[:n], dtype, f"routed experts, {n} rows")
    assert np.abs(outs[77][:5] - outs[5]).max() < (1e-5 if dtype == "float32" else 2e-2) * max(1.0, np.abs(ref).max())


# ----------------------------------------------------------------------------
# whole models
# ----------------------------------------------------------------------------
CASES = [(n, d) for n in ("p", "q", "r") for d in ("float32", "bfloat16")]
LENGTHS = {"p": [70, 3, 130, 64, 1], "q": [129, 2, 150, 65], "r": [200, 33, 1, 90]}


@pytest.fixture(scope="module")
def engines():
    from gguf2bin_b200.engine import Engine, Model
    made = {}

    def get(name, dtype, max_tokens=4096):
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
                          f"sominex {name}/{dtype} request {i} whole")


@pytest.mark.parametrize("name,dtype", CASES)
def test_token_by_token_and_portions(engines, name, dtype):
    """The same logits however the prompt is cut: every token alone from the first one on; portions
    of two; mixed portions that end on, before and behind page, window and block borders."""
    eng = engines(name, dtype)
    toks = requests_of(name)[2 if name != "r" else 0][:110]
    ref = plain_logits(name, toks)
    whole = run_in_portions(eng, toks, [])
    for what, sizes in [("one by one", [1] * len(toks)), ("twos", [2] * len(toks)), ("mixed", [3, 2, 5, 1, 2, 50, 1, 2, 2]),
                        ("window edge", [19, 1, 1, 4, 1, 6, 1, 1, 36, 1]), ("page edge", [63, 1, 1, 2]), ("page", [64, 2, 2])]:
        got = run_in_portions(eng, toks, sizes)
        assert_rows_close(got, ref, dtype, f"sominex {name}/{dtype} {what}")
        if dtype == "float32":       # the cut changes nothing but the order of a few additions
            assert np.abs(got - whole).max() <= 2e-5 * max(1.0, np.abs(ref).max()), what


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_with_reuse(engines, name, dtype):
    """Batches of up to three requests: prompts (all but the last 6 tokens, at least one) in one step,
    then one token each, shorter requests ending earlier; the cache holds one batch, so every batch
    gets the slots, states, shift rows and pages that the one before gave back."""
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
                              f"sominex {name}/{dtype} batch {bi} request {j}")
    assert eng.cache.table.pages.n_held == 0 and eng.cache.table.slots.n_held == 0


@pytest.mark.parametrize("name,dtype", [("p", "float32"), ("q", "bfloat16"), ("r", "bfloat16"), ("q", "float32")])
def test_long_decoding(engines, name, dtype):
    """A short prompt, then 200 tokens one by one: the window passes over decoded tokens, blocks are
    completed and first seen by decoded tokens, pages begin; beside a second sequence that started
    elsewhere."""
    from gguf2bin_b200.engine import StepEntry
    eng = engines(name, dtype)
    a, b = list(clear_tokens(name, 230, 70)), list(clear_tokens(name, 261, 71))
    sa, sb = eng.open_sequence(), eng.open_sequence()
    out = eng.step([StepEntry(sa, a[:30], range(30)), StepEntry(sb, b[:61], range(61))]).cpu().numpy()
    ga, gb = [out[:30]], [out[30:]]
    for t in range(200):
        out = eng.step([StepEntry(sa, [a[30 + t]], [0]), StepEntry(sb, [b[61 + t]], [0])]).cpu().numpy()
        ga.append(out[:1])
        gb.append(out[1:])
    eng.close_sequence(sa)
    eng.close_sequence(sb)
    assert_rows_close(np.concatenate(ga), plain_logits(name, a), dtype, f"sominex {name}/{dtype} long decoding a")
    assert_rows_close(np.concatenate(gb), plain_logits(name, b), dtype, f"sominex {name}/{dtype} long decoding b")


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
        outs = llm.generate(prompts, n=40, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0)
        for p, o in zip(prompts, outs):
            toks = list(p)
            for t in o.tokens:
                row = plain_logits(name, toks)[-1]
                assert row[t] >= row.max() - 2e-5 * max(1.0, np.abs(row).max())
                toks.append(t)
            assert len(o.tokens) == 40
    a = llm.generate(prompts[:2], n=12, seed=5)
    b = llm.generate(prompts[:2], n=12, seed=5)
    assert [o.tokens for o in a] == [o.tokens for o in b]
    assert llm.engine.cache.table.pages.n_held == 0 and llm.engine.cache.table.slots.n_held == 0


def test_the_programs(tmp_path):
    """info and run of the command line, random weights for the design's config.json, and trace replay."""
    folder = model_folder("p")
    exe = [sys.executable, str(ROOT / "bin" / "gguf2bin_b200")]
    out = subprocess.run(exe + ["info", str(folder)], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "Sominex" in out.stdout + out.stderr, out.stderr[-2000:]
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
    W = SP.read_safetensors(made / "model.safetensors")
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
    ref = SP.forward(CONFIGS["r"], W, toks)
    assert_close(got, ref[[0, 5, 0, 7, 8]], "float32", "sominex trace replay")
