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


def chain_to_tree_params(Uc, Wc_rec, b, H):
    """Chain-LSTM parameters in the reference app's layout (apps/paper/seq-lstm-cavs.cc:45-74: U [E,4H] multiplies
    x, W [H,4H] multiplies the child's h, both with column blocks i,f,u,o; bias i,f,u,o) rearranged into the
    child-sum Tree-LSTM layout with one child slot (W [E,4H] blocks i,o,u,f; U = U_iou [H,3H] then U_f [H,H])."""
    Uc = np.asarray(Uc, np.float32).reshape(-1, 4 * H)
    Wr = np.asarray(Wc_rec, np.float32).reshape(H, 4 * H)
    blk = lambda m, k: m[:, k * H:(k + 1) * H]
    W_tree = np.concatenate([blk(Uc, 0), blk(Uc, 3), blk(Uc, 2), blk(Uc, 1)], axis=1)
    U_iou = np.concatenate([blk(Wr, 0), blk(Wr, 3), blk(Wr, 2)], axis=1)
    U_tree = np.concatenate([U_iou.ravel(), blk(Wr, 1).ravel()])
    return W_tree.ravel().copy(), U_tree.copy(), np.asarray(b, np.float32).copy()


def make_chain_batch(seed, batch, len_lo, len_hi, vocab):
    """Ragged chains with Zipf tokens and next-token labels (the last position predicts token 0)."""
    parents = S.synth_chains(seed, batch, len_lo, len_hi)
    lens = (parents == -1).argmax(1) + 1
    n = int(lens.sum())
    tok_job = S.synth_zipf(seed + 1, 1.1, vocab, n)
    label_job = np.empty(n, np.int32)
    off = 0
    for L in lens:
        label_job[off:off + L - 1] = tok_job[off + 1:off + L]
        label_job[off + L - 1] = 0
        off += L
    return parents, tok_job, label_job


def make_gru_params(seed, H, E, V, C, scale=0.05, bias_scale=0.0):
    """Tree-GRU parameters: W [E,3H] (r,z,n), U [3,H,H], B [3H]."""
    p = dict(Emb=S.synth_uniform_float(seed + 10, scale, (V, E)), W=S.synth_uniform_float(seed + 11, scale, (E * 3 * H,)),
             U=S.synth_uniform_float(seed + 12, scale, (3 * H * H,)), Wc=S.synth_uniform_float(seed + 13, scale, (C, H)))
    p["B"] = S.synth_uniform_float(seed + 14, bias_scale, (3 * H,)) if bias_scale else np.zeros(3 * H, np.float32)
    p["bc"] = S.synth_uniform_float(seed + 15, bias_scale, (C,)) if bias_scale else np.zeros(C, np.float32)
    return p


def root_only_labels(parents, label_job):
    """Keeps the label of each sample's root (its last vertex) and sets every other label to -1."""
    lens = (parents == -1).argmax(1) + 1
    out = np.full_like(label_job, -1)
    ends = np.cumsum(lens) - 1
    out[ends] = label_job[ends]
    return out
