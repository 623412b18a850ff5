"""Runs one part of a model (a mixer, a feed-forward) on the device the way the engine would: steps
packed as the engine packs them, a cache of the part's own need whose storage starts full of junk,
slots that are not 0, 1, ..., sequences cut into portions of any sizes."""
from __future__ import annotations

import numpy as np
import torch

from senotar_helpers import to_bf16_values

DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def bf(a):
    return to_bf16_values(a).astype(np.float64)


def names_of(prefix, keys):
    return tuple((k, prefix + v) for k, v in keys)


def step_ctx(q_lens, pasts, slots, dtype, pages=None, single=False):
    """A step as the engine packs it; ``single``: without the per-sequence table, as a replayed
    decode step is."""
    from gguf2bin_b200.engine import Workspace
    from gguf2bin_b200.parts.base import StepContext
    pos = np.concatenate([np.arange(p, p + n) for p, n in zip(pasts, q_lens)])
    seq = np.concatenate([np.full(n, b) for b, n in enumerate(q_lens)])
    starts = np.cumsum([0] + list(q_lens[:-1]))
    meta = np.array([[s, n, p, sl] for s, n, p, sl in zip(starts, q_lens, pasts, slots)])
    T = int(sum(q_lens))
    table = i32(pages if pages is not None else [[0]] * len(q_lens))
    tiles = {}
    if not single:                                    # the prompt kernels' work lists: tiles of 64 and of 128 rows
        for key, rows in (("attn_tiles", 64), ("attn_tiles_wide", 128)):
            t = [(b, int(s) + r, min(rows, n - r), p + r) for b, (s, n, p) in enumerate(zip(starts, q_lens, pasts))
                 for r in range(0, n, rows)]
            t.sort(key=lambda x: -(x[3] + x[2]))
            tiles[key], tiles["n_" + key] = i32(t), len(t)
    return StepContext(**tiles, n_tokens=T, n_seqs=len(q_lens), tok_ids=i32(np.zeros(T)), tok_pos=i32(pos), tok_seq=i32(seq),
                       page_table=table, page_size=64, workspace=Workspace(DEV), dtype=DTYPES[dtype],
                       q_lens=list(q_lens), past_lens=list(pasts), slots=list(slots),
                       max_kv_len=int(max(p + n for p, n in zip(pasts, q_lens))),
                       seq_meta=None if single else i32(meta), seq_slots=i32(slots))


def run_part(mixer, need, h_seqs, cuts, dtype, slots=(3, 1), n_slots=5, pages_per_seq=8, call=None):
    """Runs a mixer over sequences cut into steps (``cuts``: lists of portion sizes, one list per
    sequence; portions of one token run as replayed decode steps do); returns each sequence's
    output rows.  ``call(h, ctx, view, y)`` replaces ``mixer.forward`` where a part wants more."""
    from gguf2bin_b200.cache.storage import Cache
    cache = Cache([need], 64 * pages_per_seq * len(h_seqs), DTYPES[dtype], DEV, max_seqs=n_slots)
    for g in cache.groups.values():
        g["storage"].fill_(7.0)
        if hasattr(g["need"], "shape"):
            for s in slots:
                g["storage"][:, s].zero_()
    view = cache.view(0)
    pages = [[1 + b * pages_per_seq + j for j in range(pages_per_seq)] for b in range(len(h_seqs))]
    done = [0] * len(h_seqs)
    outs = [[] for _ in h_seqs]
    cuts = [list(c) for c in cuts]
    while any(d < len(h) for d, h in zip(done, h_seqs)):
        live = [b for b in range(len(h_seqs)) if done[b] < len(h_seqs[b])]
        sizes = [min(cuts[b].pop(0) if cuts[b] else len(h_seqs[b]), len(h_seqs[b]) - done[b]) for b in live]
        ctx = step_ctx(sizes, [done[b] for b in live], [slots[b] for b in live], dtype, [pages[b] for b in live],
                       single=all(n == 1 for n in sizes))
        h = torch.cat([dev(h_seqs[b][done[b]:done[b] + n], DTYPES[dtype]) for b, n in zip(live, sizes)])
        y = torch.zeros((h.shape[0], h.shape[1]), dtype=torch.float32, device=DEV)
        (call or mixer.forward)(h, ctx, view, y)
        o = 0
        for b, n in zip(live, sizes):
            outs[b].append(y[o:o + n].cpu().numpy())
            done[b] += n
            o += n
    return [np.concatenate(o) for o in outs]


def close(got, ref, dtype, what, loose=1.0):
    tol = (2e-5 if dtype == "float32" else 3e-2) * loose * max(1.0, float(np.abs(ref).max()))
    err = np.abs(got - ref)
    assert np.isfinite(got).all() and err.max() <= tol, \
        f"{what}: max |diff| {err.max():.3e} > {tol:.3e} at row {err.max(-1).argmax()}"
