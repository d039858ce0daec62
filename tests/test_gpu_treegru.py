"""The CUDA Tree-GRU step (a second vertex function over the same scheduler tables) through the C ABI vs the
CPU oracle on identical seeded inputs: N-ary trees, label on the root only.  fp32: 1e-5 relative; bf16-GEMM
mode: 2e-2 relative."""
import numpy as np
import pytest

import oracle
from cavs_b200 import schedule as S
from cavs_b200.treegru import TreeGRU
from helpers import make_gru_params, make_tree_batch, rel_err, root_only_labels, tables_from_schedule

pytestmark = pytest.mark.gpu
KEYS = ("state", "loss", "dEmb", "dW", "dU", "dB", "dWc", "dbc")


def _both(parents, tok_job, label_job, params, H, E, V, C, K, bf16=False, loss_rows=0):
    s = S.Schedule().load(parents, n_slots=K)
    eng = TreeGRU(H, E, V, C, n_slots=K, gemm_bf16=bf16, max_vertices=max(s.n_total, 1), max_level_rows=max(s.max_level_rows, 1))
    eng.set_params(params)
    eng.load_batch(s, tok_job, label_job, loss_rows)
    eng.forward()
    eng.backward()
    loss_sum = eng.read_loss()
    out = dict(state=eng.state(), loss=eng.loss_rows(), **eng.grad_dict())
    tb = tables_from_schedule(s)
    tok, lab = tok_job[tb["t2j"]], label_job[tb["t2j"]]
    ref32 = oracle.treegru_fwd_bwd(tb, tok, lab, params, H, E, V, C, K=K, loss_rows=loss_rows)
    refbf = oracle.treegru_fwd_bwd(tb, tok, lab, params, H, E, V, C, K=K, loss_rows=loss_rows, gemm_bf16=True,
                                   preact_bf16=True) if bf16 else None
    return eng, out, loss_sum, ref32, refbf


@pytest.mark.parametrize("batch,leaf_hi,H,E,V,C,K,arity", [
    (32, 30, 150, 300, 21701, 5, 4, 4),   # N-ary trees, the Tree-LSTM configuration's sizes
    (7, 9, 32, 20, 100, 3, 2, 2),
    (1, 2, 8, 8, 10, 2, 3, 3),
])
def test_fp32_root_label_parity(cuda, batch, leaf_hi, H, E, V, C, K, arity):
    parents, tok_job, label_job = make_tree_batch(300 + batch, batch, 2, leaf_hi, V, C, max_arity=arity)
    label_job = root_only_labels(parents, label_job)
    params = make_gru_params(batch, H, E, V, C, scale=0.05, bias_scale=0.02)
    eng, out, loss_sum, ref, _ = _both(parents, tok_job, label_job, params, H, E, V, C, K, loss_rows=batch)
    for k in KEYS:
        assert rel_err(out[k], ref[k]) < 1e-5, k
    assert abs(loss_sum - ref["loss"].sum()) <= 1e-5 * abs(ref["loss"].sum())
    eng.forward(); eng.backward(); eng.read_loss()
    again = dict(state=eng.state(), loss=eng.loss_rows(), **eng.grad_dict())
    for k in KEYS:
        assert np.array_equal(out[k], again[k]), k   # deterministic


def test_every_vertex_labelled_fp32(cuda):
    H, E, V, C, K = 24, 16, 50, 4, 2
    parents, tok_job, label_job = make_tree_batch(5, 9, 2, 12, V, C)
    params = make_gru_params(4, H, E, V, C, scale=0.3, bias_scale=0.1)
    _, out, _, ref, _ = _both(parents, tok_job, label_job, params, H, E, V, C, K)
    for k in KEYS:
        assert rel_err(out[k], ref[k]) < 1e-5, k


def test_bf16_parity(cuda):
    H, E, V, C, K = 256, 128, 5000, 5, 4
    parents, tok_job, label_job = make_tree_batch(77, 40, 2, 30, V, C, max_arity=4)
    label_job = root_only_labels(parents, label_job)
    params = make_gru_params(9, H, E, V, C, scale=0.05, bias_scale=0.02)
    _, out, _, ref32, refbf = _both(parents, tok_job, label_job, params, H, E, V, C, K, bf16=True, loss_rows=40)
    for k in KEYS:
        assert rel_err(out[k], ref32[k]) < 2e-2, k
        assert rel_err(out[k], refbf[k]) < 5e-3, k


def test_nary_treegru_configuration_dims_bf16(cuda):
    """The N-ary Tree-GRU configuration's dimensions (hidden 1024, embedding 512, vocabulary 32,000, 1-4 children,
    8-128 leaves, 2-class loss on the root) on a batch small enough for the CPU oracle."""
    H, E, V, C, K, batch = 1024, 512, 32000, 2, 4, 6
    parents, tok_job, label_job = make_tree_batch(4040, batch, 8, 128, V, C, max_arity=4)
    label_job = root_only_labels(parents, label_job)
    params = make_gru_params(17, H, E, V, C, scale=0.03, bias_scale=0.02)
    _, out, _, ref32, refbf = _both(parents, tok_job, label_job, params, H, E, V, C, K, bf16=True, loss_rows=batch)
    for k in KEYS:
        assert rel_err(out[k], ref32[k]) < 2e-2, k
        assert rel_err(out[k], refbf[k]) < 5e-3, k
