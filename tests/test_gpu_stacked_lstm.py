"""Two stacked LSTM layers over ragged chains (the variable-length chain configuration: batch of sequences of
different lengths scheduled as a ragged graph, no padding, next-token cross-entropy) through two engines:
layer 0 with an embedding table and no loss head, layer 1 with dense inputs (layer 0's h) and the loss head.
Checked against the CPU oracle's layer entry, chained the same way."""
import numpy as np
import pytest

import oracle
from cavs_b200 import schedule as S
from cavs_b200.treelstm import TreeLSTM
from helpers import make_stack_params, oracle_stack, rel_err, tables_from_schedule

pytestmark = pytest.mark.gpu


def _run_stack(parents, tok_job, label_job, layers, dims, V, C, bf16):
    s = S.Schedule().load(parents, n_slots=1)
    n = s.n_total
    (H0, E0), (H1, E1) = dims
    assert E1 == H0
    cap = dict(n_slots=1, gemm_bf16=bf16, max_vertices=n, max_level_rows=s.max_level_rows)
    l0 = TreeLSTM(H0, E0, V, 0, **cap)       # embedding in, d(h) from above
    l1 = TreeLSTM(H1, E1, 0, C, **cap)       # dense in, loss head
    l0.set_params(layers[0])
    l1.set_params(layers[1])
    l0.load_batch(s, tok_job, None)
    l1.load_batch(s, None, label_job)
    l0.forward()
    l1.set_dense_input(l0.device_view(0, (n, 2 * H0))[:, :H0])
    l1.forward()
    l1.backward()
    l0.set_output_grad(l1.device_view(5, (n, E1)))
    l0.backward()
    loss_sum = l1.read_loss()
    out0 = dict(state=l0.state(), **l0.grad_dict())
    out1 = dict(state=l1.state(), loss=l1.loss_rows(), **l1.grad_dict())
    return s, out0, out1, loss_sum


def _case(seed, batch, len_lo, len_hi, V):
    parents = S.synth_chains(seed, batch, len_lo, len_hi)
    lens = (parents == -1).argmax(1) + 1
    tok_job = S.synth_zipf(seed + 1, 1.1, V, int(lens.sum()))
    label_job = S.synth_zipf(seed + 2, 1.1, V, int(lens.sum()))   # next-token targets: a class per vocabulary entry
    return parents, tok_job, label_job


@pytest.mark.parametrize("bf16,H,batch,len_hi,V,tol", [
    (False, 48, 12, 30, 200, 1e-5),
    (False, 64, 5, 9, 5, 1e-5),         # fused loss head on the top layer (<= 8 classes)
    (True, 512, 16, 40, 1000, 2e-2),    # the configuration's layer width, bf16 GEMMs
])
def test_two_layer_chain_lstm(cuda, bf16, H, batch, len_hi, V, tol):
    dims = [(H, H), (H, H)]
    parents, tok_job, label_job = _case(900 + H, batch, 3, len_hi, V)
    layers = make_stack_params(H, dims, V, V, scale=0.08)
    s, out0, out1, loss_sum = _run_stack(parents, tok_job, label_job, layers, dims, V, V, bf16)
    tb = tables_from_schedule(s)
    tok, lab = tok_job[tb["t2j"]], label_job[tb["t2j"]]
    ref = oracle_stack(oracle, tb, tok, lab, layers, dims, V, V)
    assert rel_err(out1["loss"], ref[1]["loss"]) < tol
    assert abs(loss_sum - ref[1]["loss"].sum()) <= tol * abs(ref[1]["loss"].sum())
    for k in ("state", "dW", "dU", "dB", "dWc", "dbc"):
        assert rel_err(out1[k], ref[1][k]) < tol, ("layer 1", k)
    for k in ("state", "dEmb", "dW", "dU", "dB"):
        assert rel_err(out0[k], ref[0][k]) < tol, ("layer 0", k)
    if bf16:
        refbf = oracle_stack(oracle, tb, tok, lab, layers, dims, V, V, gemm_bf16=True)
        for k in ("state", "dEmb", "dW", "dU", "dB"):
            assert rel_err(out0[k], refbf[0][k]) < 5e-3, ("layer 0 vs bf16 oracle", k)
