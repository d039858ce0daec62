"""The C oracle's numerics pinned against float64 PyTorch autograd (live and via the committed
golden file), plus the reference-compatible (shifted-row) mode and the optimizer restatements."""
from pathlib import Path

import numpy as np
import pytest

import oracle
from cavs_b200 import schedule as S
from helpers import assert_close, make_params, make_tree_batch, rel_err, tables_from_schedule
from torch_ref import stacked_lstm_autograd, treegru_autograd, treelstm_autograd

GOLD = Path(__file__).parent / "golden" / "treelstm_small.npz"
KEYS = ("state", "loss", "dEmb", "dW", "dU", "dB", "dWc", "dbc")
TOL = 1e-5   # fp32 contract: 1e-5 relative


def test_golden_file():
    g = np.load(GOLD)
    H, E, V, C = (int(x) for x in g["dims"])
    s = S.Schedule().load(g["parents"])
    tb = tables_from_schedule(s)
    tok, label = g["tok_job"][tb["t2j"]], g["label_job"][tb["t2j"]]
    params = {k: g["p_" + k] for k in ("Emb", "W", "U", "B", "Wc", "bc")}
    o = oracle.treelstm_fwd_bwd(tb, tok, label, params, H, E, V, C)
    for k in KEYS:
        assert rel_err(o[k], g["r_" + k]) < TOL, k


@pytest.mark.parametrize("K,arity", [(1, None), (2, 2), (4, 4)])
def test_against_autograd(K, arity):
    H, E, V, C = 12, 10, 30, 3
    if K == 1:
        parents = S.synth_chains(77, 5, 2, 9)
        lens = (parents == -1).argmax(1) + 1
        tok_job = S.synth_zipf(78, 1.1, V, int(lens.sum()))
        label_job = S.synth_uniform_int(79, C, int(lens.sum()))
    else:
        parents, tok_job, label_job = make_tree_batch(77, 5, 2, 8, V, C, max_arity=arity)
    s = S.Schedule().load(parents, n_slots=K)
    tb = tables_from_schedule(s)
    n = s.n_scheduled
    # single-vertex samples are never scheduled; keep the test on fully scheduled batches
    if n != s.n_total:
        pytest.skip("batch holds a single-vertex sample")
    tok, label = tok_job[tb["t2j"]], label_job[tb["t2j"]]
    params = make_params(5, H, E, V, C, scale=0.4, bias_scale=0.3)
    o = oracle.treelstm_fwd_bwd(tb, tok, label, params, H, E, V, C, K=K)
    r = treelstm_autograd(tb, tok, label, params, H, E, V, C, K=K)
    for k in KEYS:
        assert_close(o[k], r[k], TOL, k)      # max-norm and value by value


def test_root_only_loss_rows():
    H, E, V, C = 8, 8, 20, 2
    parents, tok_job, label_job = make_tree_batch(9, 4, 2, 6, V, C)
    s = S.Schedule().load(parents)
    tb = tables_from_schedule(s)
    tok = tok_job[tb["t2j"]]
    label = np.where(tb["fs"] < 0, label_job[tb["t2j"]], -1)   # roots only
    params = make_params(6, H, E, V, C, scale=0.4)
    o = oracle.treelstm_fwd_bwd(tb, tok, label, params, H, E, V, C, loss_rows=4)
    r = treelstm_autograd(tb, tok, label, params, H, E, V, C, loss_rows=4)
    for k in KEYS:
        assert rel_err(o[k], r[k]) < TOL, k


def test_ref_compat_equals_aligned_on_equal_shapes_and_not_on_skewed():
    H, E, V, C = 8, 8, 20, 3
    params = make_params(3, H, E, V, C, scale=0.4)
    same = np.array([[3, 3, 4, 4, -1]] * 3, np.int32)
    skew = np.array([[2, 2, -1, -1, -1], [3, 3, 4, 4, -1]], np.int32)
    for parents, expect_equal in ((same, True), (skew, False)):
        s = S.Schedule().load(parents)
        n = s.n_total
        tok = S.synth_zipf(1, 1.1, V, n)
        label = S.synth_uniform_int(2, C, n)
        a = oracle.treelstm_fwd_bwd(tables_from_schedule(s, 0), tok, label, params, H, E, V, C)
        r = oracle.treelstm_fwd_bwd(tables_from_schedule(s, 1), tok, label, params, H, E, V, C)
        assert np.array_equal(a["state"], r["state"]) == expect_equal


def test_bf16_rounding_mode_is_close_to_fp32():
    H, E, V, C = 16, 16, 30, 5
    parents, tok_job, label_job = make_tree_batch(11, 6, 2, 9, V, C)
    s = S.Schedule().load(parents)
    tb = tables_from_schedule(s)
    tok, label = tok_job[tb["t2j"]], label_job[tb["t2j"]]
    params = make_params(8, H, E, V, C, scale=0.3)
    a = oracle.treelstm_fwd_bwd(tb, tok, label, params, H, E, V, C)
    b = oracle.treelstm_fwd_bwd(tb, tok, label, params, H, E, V, C, gemm_bf16=True)
    for k in KEYS:
        assert rel_err(b[k], a[k]) < 2e-2, k     # the bf16-GEMM contract
    assert not np.array_equal(a["state"], b["state"])


def test_row_ops_and_optimizers():
    rng = np.random.default_rng(0)
    inp = rng.standard_normal((9, 6)).astype(np.float32)
    ids = np.array([4, 0, 8, 4], np.int32)
    out = np.zeros((4, 6), np.float32)
    lib = oracle.oracle_lib()
    lib.cavs_oracle_gather_rows(oracle._p(out), oracle._p(inp), oracle._p(ids), 4, 6)
    assert np.array_equal(out, inp[ids])
    dst = np.zeros((9, 6), np.float32)
    ids2 = np.array([7, 2, 5, 0], np.int32)
    lib.cavs_oracle_scatter_rows(oracle._p(dst), oracle._p(ids2), oracle._p(out), 4, 6)
    assert np.array_equal(dst[ids2], out) and not dst[[1, 3, 4, 6, 8]].any()
    w = rng.standard_normal(101).astype(np.float32); g = rng.standard_normal(101).astype(np.float32)
    w0 = w.copy()
    oracle.sgd(w, g, 0.5)
    assert np.allclose(w, w0 - 0.5 * g, rtol=1e-7, atol=0)
    acc = np.zeros(101, np.float32); w1 = w.copy()
    oracle.adagrad(w, acc, g, 0.05, 1e-10)
    assert np.allclose(acc, g * g) and np.allclose(w, w1 - 0.05 * g / (np.abs(g) + 1e-10), rtol=1e-6)


@pytest.mark.parametrize("K,arity,root_only", [(4, 4, True), (2, 2, False)])
def test_treegru_against_autograd(K, arity, root_only):
    """The Tree-GRU restatement (an extension: N-ary trees, label on the root) vs torch autograd in fp64."""
    from helpers import make_gru_params, root_only_labels
    H, E, V, C = 12, 10, 30, 3
    parents, tok_job, label_job = make_tree_batch(21, 6, 2, 9, V, C, max_arity=arity)
    if root_only:
        label_job = root_only_labels(parents, label_job)
    s = S.Schedule().load(parents, n_slots=K)
    tb = tables_from_schedule(s)
    params = make_gru_params(5, H, E, V, C, scale=0.4, bias_scale=0.1)
    rows = parents.shape[0] if root_only else 0
    tok, lab = tok_job[tb["t2j"]], label_job[tb["t2j"]]
    got = oracle.treegru_fwd_bwd(tb, tok, lab, params, H, E, V, C, K=K, loss_rows=rows)
    ref = treegru_autograd(tb, tok, lab, params, H, E, V, C, K=K, loss_rows=rows)
    for k in KEYS:
        assert rel_err(got[k], ref[k]) < 2e-5, k


def test_stacked_chain_lstm_against_autograd():
    """Two stacked LSTM layers over ragged chains (the variable-length chain configuration, scaled down): the
    oracle's single-layer entry chained through dense inputs / external output gradients vs autograd in fp64."""
    from helpers import make_stack_params, oracle_stack
    V, C, dims = 40, 40, [(10, 8), (12, 10)]
    parents = S.synth_chains(31, 6, 3, 9)
    lens = (parents == -1).argmax(1) + 1
    tok_job = S.synth_zipf(32, 1.1, V, int(lens.sum()))
    label_job = S.synth_uniform_int(33, C, int(lens.sum()))
    s = S.Schedule().load(parents, n_slots=1)
    tb = tables_from_schedule(s)
    tok, lab = tok_job[tb["t2j"]], label_job[tb["t2j"]]
    layers = make_stack_params(7, dims, V, C, scale=0.3)
    got = oracle_stack(oracle, tb, tok, lab, layers, dims, V, C)
    ref, ref_loss = stacked_lstm_autograd(tb, tok, lab, layers, dims, V, C)
    assert rel_err(got[-1]["loss"], ref_loss) < 2e-5
    for li in range(2):
        for k in ref[li]:
            assert rel_err(got[li][k], ref[li][k]) < 2e-5, (li, k)
