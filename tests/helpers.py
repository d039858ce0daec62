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
    """Max-norm relative error of a whole tensor: max|a-b| / max|b|."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def value_err(a, b):
    """Per-value relative error: max over entries of |a-b| / (|b| + rms(b)).  An entry passes a tolerance `tol`
    exactly when |a-b| <= tol*|b| + tol*rms(b), so entries far below the tensor's largest value are checked against
    their own size (plus the tensor's typical size, which absorbs the rounding of sums that cancel to nearly zero).
    rms(b) is taken over b's non-zero entries: the untouched rows of an embedding gradient are exact zeros on both
    sides and say nothing about the size of the others."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    if b.size == 0:
        return 0.0
    nz = b[b != 0.0]
    rms = float(np.sqrt(np.mean(nz * nz))) if nz.size else 0.0
    return float((np.abs(a - b) / (np.abs(b) + max(rms, 1e-30))).max())


def assert_close(got, want, tol, name="", value_tol=None):
    """Both statements of "within tol relative": over the tensor's max norm and value by value."""
    e_norm, e_val = rel_err(got, want), value_err(got, want)
    vt = tol if value_tol is None else value_tol
    assert e_norm < tol and e_val < vt, f"{name}: max-norm error {e_norm:.3e} (tol {tol:g}), per-value error {e_val:.3e} (tol {vt:g})"


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


def make_stack_params(seed, dims, V, C, scale=0.1, bias_scale=0.05):
    """Parameters of a stack of LSTM layers: dims = [(H, E), ...] with E of layer i > 0 equal to H of layer i-1.
    Layer 0 holds Emb, the last layer Wc and bc."""
    layers = []
    for li, (H, E) in enumerate(dims):
        p = dict(W=S.synth_uniform_float(seed + 20 * li + 11, scale, (E * 4 * H,)),
                 U=S.synth_uniform_float(seed + 20 * li + 12, scale, (4 * H * H,)),
                 B=S.synth_uniform_float(seed + 20 * li + 14, bias_scale, (4 * H,)))
        if li == 0:
            p["Emb"] = S.synth_uniform_float(seed + 10, scale, (V, E))
        if li == len(dims) - 1:
            p["Wc"] = S.synth_uniform_float(seed + 13, scale, (C, H))
            p["bc"] = S.synth_uniform_float(seed + 15, bias_scale, (C,))
        layers.append(p)
    return layers


def oracle_stack(oracle, tb, tok, label, layers, dims, V, C, K=1, gemm_bf16=False, loss_rows=0):
    """Runs a layer stack through the oracle's single-layer entry: forward sweeps bottom-up (a forward-only call
    is a call with a zero output gradient), then top-down with each layer's d(input) as the next one's d(h)."""
    n = int(tb["n"])
    kw = dict(K=K, gemm_bf16=gemm_bf16, preact_bf16=gemm_bf16)
    x, fwd = None, []
    for li, (H, E) in enumerate(dims[:-1]):
        r = oracle.treelstm_layer(tb, layers[li], H, E, tok=tok if li == 0 else None, x_dense=x, V=V if li == 0 else 0,
                                  dh_ext=np.zeros((n, H), np.float32), **kw)
        x = np.ascontiguousarray(r["state"][:, :H])
        fwd.append(x)
    outs = [None] * len(dims)
    H, E = dims[-1]
    top = oracle.treelstm_layer(tb, layers[-1], H, E, tok=tok if len(dims) == 1 else None, x_dense=x, label=label, C=C,
                                V=V if len(dims) == 1 else 0, loss_rows=loss_rows, **kw)
    outs[-1] = top
    dh = top["dX"]
    for li in range(len(dims) - 2, -1, -1):
        H, E = dims[li]
        r = oracle.treelstm_layer(tb, layers[li], H, E, tok=tok if li == 0 else None, x_dense=None if li == 0 else fwd[li - 1],
                                  V=V if li == 0 else 0, dh_ext=dh, **kw)
        outs[li] = r
        dh = r["dX"]
    return outs


def loss_head_reference(h, label, Wc, bc, inv_rows):
    """float64 restatement of the reference's loss head: FullyConnected (logits = h Wc^T + bc,
    cavs/backend/op_impl_fullyconnected_cublas.cc:33-85) + SoftmaxEntropyLoss (loss_r = -log softmax(z_r)[y_r],
    cavs/backend/op_impl_softmax_entropy_logits_loss.cu:106-140), and their gradients (:213-250: dz = (softmax - onehot)
    scaled by 1/rows, the upstream gradient ignored; op_impl_fullyconnected_cublas.cc:104-176: dH = dz Wc,
    dWc = dz^T h, dbc = column sums of dz).  A row with label < 0 has no loss term (an extension of this library)."""
    h = np.asarray(h, np.float64); Wc = np.asarray(Wc, np.float64); bc = np.asarray(bc, np.float64)
    label = np.asarray(label)
    z = h @ Wc.T + bc
    z -= z.max(axis=1, keepdims=True)
    p = np.exp(z); p /= p.sum(axis=1, keepdims=True)
    has = label >= 0
    rows = np.arange(h.shape[0])
    loss = np.where(has, -np.log(p[rows, np.maximum(label, 0)]), 0.0)
    dz = p.copy()
    dz[rows, np.maximum(label, 0)] -= 1.0
    dz *= has[:, None] * inv_rows
    return dict(loss=loss, loss_sum=np.array([loss.sum()]), dH=dz @ Wc, dWc=dz.T @ h, dbc=dz.sum(axis=0))
