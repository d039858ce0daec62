"""Chain-LSTM language model (the reference's apps/paper/seq-lstm-cavs.cc vertex function: one child slot,
vocabulary-sized softmax) on the CUDA path vs the CPU oracle, fp32, 1e-5 relative; SGD(lr=1.0) step included."""
import numpy as np
import pytest

import oracle
from cavs_b200 import schedule as S
from cavs_b200.treelstm import TreeLSTM
from helpers import chain_to_tree_params, make_chain_batch, rel_err, tables_from_schedule

pytestmark = pytest.mark.gpu
KEYS = ("state", "loss", "dEmb", "dW", "dU", "dB", "dWc", "dbc")


def _params(seed, H, E, V, scale):
    U_x = S.synth_uniform_float(seed, scale, (E, 4 * H))          # multiplies x
    W_h = S.synth_uniform_float(seed + 1, scale, (H, 4 * H))      # multiplies the child's h
    b = S.synth_uniform_float(seed + 2, scale, (4 * H,))
    W, U, B = chain_to_tree_params(U_x, W_h, b, H)
    return dict(Emb=S.synth_uniform_float(seed + 3, scale, (V, E)), W=W, U=U, B=B,
                Wc=S.synth_uniform_float(seed + 4, scale, (V, H)), bc=np.zeros(V, np.float32))


def _check(cuda, parents, tok_job, label_job, params, H, E, V, bf16=False, tol=1e-5):
    s = S.Schedule().load(parents, n_slots=1)
    eng = TreeLSTM(H, E, V, V, n_slots=1, gemm_bf16=bf16, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    eng.set_params(params)
    eng.load_batch(s, tok_job, label_job)
    eng.forward()
    eng.backward()
    loss_sum = eng.read_loss()
    got = dict(state=eng.state(), loss=eng.loss_rows(), **eng.grad_dict())
    tb = tables_from_schedule(s)
    ref = oracle.treelstm_fwd_bwd(tb, tok_job[tb["t2j"]], label_job[tb["t2j"]], params, H, E, V, V, K=1, gemm_bf16=bf16,
                                  preact_bf16=bf16)
    for k in KEYS:
        assert rel_err(got[k], ref[k]) < tol, k
    assert abs(loss_sum - float(ref["loss"].sum())) < 10 * tol * abs(float(ref["loss"].sum()))
    return eng, ref


def test_fixed_length_chain_lm_fp32(cuda):
    # batch 20, length 20, vocabulary 10000, embedding = hidden = 200, uniform +-0.1 weights, SGD lr 1.0
    H = E = 200
    V = 10000
    parents, tok_job, label_job = make_chain_batch(11, 20, 20, 20, V)
    params = _params(5, H, E, V, 0.1)
    eng, ref = _check(cuda, parents, tok_job, label_job, params, H, E, V)
    w0 = eng.params.cpu().numpy().copy()
    g0 = eng.grads.cpu().numpy().copy()
    eng.sgd(1.0)
    oracle.sgd(w0, g0, 1.0)
    assert rel_err(eng.params.cpu().numpy(), w0) < 1e-6


def test_ragged_chain_lm_fp32(cuda):
    # variable-length chains scheduled as a ragged graph (no padding): lengths 10..100
    H = E = 64
    V = 1000
    parents, tok_job, label_job = make_chain_batch(21, 32, 10, 100, V)
    _check(cuda, parents, tok_job, label_job, _params(6, H, E, V, 0.1), H, E, V)


def test_chain_lm_bf16(cuda):
    H = E = 128
    V = 2048
    parents, tok_job, label_job = make_chain_batch(31, 24, 5, 40, V)
    _check(cuda, parents, tok_job, label_job, _params(7, H, E, V, 0.1), H, E, V, bf16=True, tol=2e-2)
