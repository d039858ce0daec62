"""Shared workload builders for the tests (seeded, via the library's own generators)."""
from __future__ import annotations

import numpy as np

from cavs_b200 import schedule as S


def make_tree_batch(seed, batch, leaf_lo, leaf_hi, vocab, classes, max_arity=2):
    """Random trees with Zipf leaf tokens (internal vertices use token 0, as the reference's
    zero-filled inputs do) and uniform per-vertex labels, all compact in job order."""
    parents, is_leaf = S.synth_trees(seed, batch, leaf_lo, leaf_hi, max_arity)
    lens = (parents == -1).argmax(1) + 1
    tok_pad = S.synth_zipf(seed + 1, 1.1, vocab, parents.size).reshape(parents.shape) * is_leaf
    tok_job = np.concatenate([tok_pad[i, :lens[i]] for i in range(batch)]).astype(np.int32)
    label_job = S.synth_uniform_int(seed + 2, classes, int(lens.sum()))
    return parents, tok_job, label_job


def make_params(seed, H, E, V, C, scale=0.05, bias_scale=0.0):
    p = dict(Emb=S.synth_uniform_float(seed + 10, scale, (V, E)), W=S.synth_uniform_float(seed + 11, scale, (E * 4 * H,)),
             U=S.synth_uniform_float(seed + 12, scale, (4 * H * H,)), Wc=S.synth_uniform_float(seed + 13, scale, (C, H)))
    if bias_scale:
        p["B"] = S.synth_uniform_float(seed + 14, bias_scale, (4 * H,))
        p["bc"] = S.synth_uniform_float(seed + 15, bias_scale, (C,))
    else:
        p["B"] = np.zeros(4 * H, np.float32)
        p["bc"] = np.zeros(C, np.float32)
    return p


def tables_from_schedule(s, mode=0):
    fg, fs, bg, bs = s.tables(mode)
    t2j, j2t = s.maps()
    return dict(n=s.n_total, n_levels=s.n_levels, level_off=s.level_off, fg=fg, fs=fs, bg=bg, bs=bs, t2j=t2j, j2t=j2t)


def rel_err(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
