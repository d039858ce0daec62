"""The CUDA Tree-LSTM step (forward, loss, backward, update) through the C ABI vs the CPU oracle
on identical seeded inputs.  fp32 configurations: 1e-5 relative; bf16-GEMM configurations: 2e-2
relative (and tighter against the oracle run with bf16-rounded GEMM operands).  "Relative" is checked
twice (helpers.assert_close): over each tensor's max norm at the stated tolerance, and value by value
(|a-b| <= tol*|b| + tol*rms(b)) at VALUE_FACTOR times it -- two fp32 evaluations that sum in different
orders each sit up to 5e-6 per value from the exact result (measured: the fp32 oracle against float64
autograd; entries that are sums of hundreds of cancelling terms carry the rounding of the terms, not of
the small result), so value by value they can be more than 1e-5 apart from one another (measured on the
binary Tree-LSTM configuration: 1e-5 on the embedding gradient); against float64 results the per-value
bound is the stated tolerance itself."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from cavs_b200 import schedule as S
from cavs_b200.treelstm import TreeLSTM
from helpers import assert_close, make_params, make_tree_batch, rel_err, tables_from_schedule

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def level_one_by_token(monkeypatch):
    # Small test batches have fewer level-1 rows than distinct tokens, where the engine would choose the per-vertex
    # form of level 1 by itself: force the per-token form so that every bf16 case below runs it.
    monkeypatch.setenv("CAVS_LEVEL1_BY_TOKEN", "1")
KEYS = ("state", "loss", "dEmb", "dW", "dU", "dB", "dWc", "dbc")
VALUE_FACTOR = 4.0
GOLD = Path(__file__).parent / "golden" / "treelstm_small.npz"


def _run(cuda, parents, tok_job, label_job, params, H, E, V, C, K=2, bf16=False):
    s = S.Schedule().load(parents, n_slots=K)
    eng = TreeLSTM(H, E, V, C, n_slots=K, gemm_bf16=bf16, max_vertices=max(s.n_total, 1), max_level_rows=max(s.max_level_rows, 1))
    eng.set_params(params)
    eng.load_batch(s, tok_job, label_job)
    eng.forward()
    eng.backward()
    loss_sum = eng.read_loss()
    out = dict(state=eng.state(), loss=eng.loss_rows(), **eng.grad_dict())
    return s, eng, out, loss_sum


def _oracle(s, tok_job, label_job, params, H, E, V, C, K=2, bf16=False):
    tb = tables_from_schedule(s)
    # in bf16 mode the product rounds the GEMM operands and the stored gate pre-activations to bf16
    return oracle.treelstm_fwd_bwd(tb, tok_job[tb["t2j"]], label_job[tb["t2j"]], params, H, E, V, C, K=K, gemm_bf16=bf16,
                                   preact_bf16=bf16)


def test_golden_fp32(cuda):
    g = np.load(GOLD)
    H, E, V, C = (int(x) for x in g["dims"])
    params = {k: g["p_" + k] for k in ("Emb", "W", "U", "B", "Wc", "bc")}
    s, eng, out, loss_sum = _run(cuda, g["parents"], g["tok_job"], g["label_job"], params, H, E, V, C)
    for k in KEYS:
        assert_close(out[k], g["r_" + k], 1e-5, k)        # the golden values are float64 autograd results
    assert abs(loss_sum - g["r_loss"].sum()) < 1e-5 * abs(g["r_loss"].sum())


@pytest.mark.parametrize("batch,leaf_hi,H,E,V,C", [
    (64, 50, 150, 300, 21701, 5),   # the binary Tree-LSTM configuration (fp32)
    (7, 9, 32, 20, 100, 3),
    (1, 2, 8, 8, 10, 2),            # one tree of two leaves
])
def test_fp32_parity_with_oracle(cuda, batch, leaf_hi, H, E, V, C):
    parents, tok_job, label_job = make_tree_batch(100 + batch, batch, 2, leaf_hi, V, C)
    params = make_params(batch, H, E, V, C, scale=0.05, bias_scale=0.02)
    s, eng, out, loss_sum = _run(cuda, parents, tok_job, label_job, params, H, E, V, C)
    ref = _oracle(s, tok_job, label_job, params, H, E, V, C)
    for k in KEYS:
        assert_close(out[k], ref[k], 1e-5, k, value_tol=VALUE_FACTOR * 1e-5)
    # determinism: a second run is bit-identical
    eng.forward(); eng.backward(); eng.read_loss()
    again = dict(state=eng.state(), loss=eng.loss_rows(), **eng.grad_dict())
    for k in KEYS:
        assert np.array_equal(out[k], again[k]), k


def test_bf16_parity_with_oracle(cuda):
    H, E, V, C = 256, 128, 5000, 5
    parents, tok_job, label_job = make_tree_batch(321, 48, 2, 40, V, C)
    params = make_params(9, H, E, V, C, scale=0.05, bias_scale=0.02)
    s, eng, out, _ = _run(cuda, parents, tok_job, label_job, params, H, E, V, C, bf16=True)
    ref32 = _oracle(s, tok_job, label_job, params, H, E, V, C)
    refbf = _oracle(s, tok_job, label_job, params, H, E, V, C, bf16=True)
    for k in KEYS:
        assert_close(out[k], ref32[k], 2e-2, k, value_tol=VALUE_FACTOR * 2e-2)      # the bf16-GEMM contract
        assert rel_err(out[k], refbf[k]) < 5e-3, k      # same rounding points as the oracle's bf16 mode


@pytest.mark.parametrize("H,K", [(512, 2), (1024, 2), (512, 3), (512, 1), (512, 4)])
def test_bf16_wide_hidden_parity_with_oracle(cuda, H, K):
    # Hidden sizes of 512 and more: the internal levels' cell gradient and the by-token level's forward cell run as the
    # streaming kernels (rows staged in shared memory by bulk copies); roots, missing children (K = 3 over binary
    # trees), chains (K = 1), four-ary trees and ragged levels included.
    E, V, C = 64, 200, 5
    if K == 1:
        parents = S.synth_chains(77 + H, 10, 2, 14)
        lens = (parents == -1).argmax(1) + 1
        tok_job = S.synth_zipf(78 + H, 1.1, V, int(lens.sum()))
        label_job = S.synth_uniform_int(79 + H, C, int(lens.sum()))
    else:
        parents, tok_job, label_job = make_tree_batch(77 + H + K, 10, 2, 12, V, C, max_arity=4 if K == 4 else 2)
    params = make_params(13, H, E, V, C, scale=0.04, bias_scale=0.02)
    s, eng, out, _ = _run(cuda, parents, tok_job, label_job, params, H, E, V, C, K=K, bf16=True)
    refbf = _oracle(s, tok_job, label_job, params, H, E, V, C, K=K, bf16=True)
    for k in KEYS:
        assert rel_err(out[k], refbf[k]) < 5e-3, k
    s2, eng2, again, _ = _run(cuda, parents, tok_job, label_job, params, H, E, V, C, K=K, bf16=True)
    for k in KEYS:
        assert np.array_equal(out[k], again[k]), k          # deterministic


@pytest.mark.parametrize("K,arity", [(1, None), (4, 4)])
def test_other_slot_counts_fp32(cuda, K, arity):
    H, E, V, C = 24, 16, 50, 4
    if K == 1:
        parents = S.synth_chains(5, 9, 2, 12)
        lens = (parents == -1).argmax(1) + 1
        tok_job = S.synth_zipf(6, 1.1, V, int(lens.sum()))
        label_job = S.synth_uniform_int(7, C, int(lens.sum()))
    else:
        parents, tok_job, label_job = make_tree_batch(5, 9, 2, 12, V, C, max_arity=arity)
    params = make_params(4, H, E, V, C, scale=0.3, bias_scale=0.1)
    s, eng, out, _ = _run(cuda, parents, tok_job, label_job, params, H, E, V, C, K=K)
    ref = _oracle(s, tok_job, label_job, params, H, E, V, C, K=K)
    for k in KEYS:
        assert_close(out[k], ref[k], 1e-5, k, value_tol=VALUE_FACTOR * 1e-5)


def test_updates_match_oracle(cuda):
    H, E, V, C = 16, 16, 40, 3
    parents, tok_job, label_job = make_tree_batch(55, 5, 2, 6, V, C)
    params = make_params(2, H, E, V, C, scale=0.3)
    s, eng, out, _ = _run(cuda, parents, tok_job, label_job, params, H, E, V, C)
    flat_w = eng.params.cpu().numpy().copy()
    flat_g = eng.grads.cpu().numpy().copy()
    eng.sgd(0.5)
    w = flat_w.copy(); oracle.sgd(w, flat_g, 0.5)
    assert rel_err(eng.params.cpu().numpy(), w) < 1e-6
    acc = torch.zeros_like(eng.params)
    acc_h = np.zeros_like(flat_w)
    w2 = eng.params.cpu().numpy().copy()
    eng.adagrad(acc, 0.05)
    oracle.adagrad(w2, acc_h, flat_g, 0.05, 1e-10)
    assert rel_err(eng.params.cpu().numpy(), w2) < 1e-6 and rel_err(acc.cpu().numpy(), acc_h) < 1e-6


def test_capacity_errors(cuda):
    from cavs_b200 import CavsError
    parents, tok_job, label_job = make_tree_batch(1, 4, 2, 6, 20, 2)
    s = S.Schedule().load(parents)
    eng = TreeLSTM(8, 8, 20, 2, max_vertices=4, max_level_rows=4)
    with pytest.raises(CavsError) as e:
        eng.load_batch(s, tok_job, label_job)
    assert e.value.status == 3


def test_embedding_gradient_is_announced_before_the_weight_gradients(cuda):
    """A second stream that waits on cavs_treelstm_wait_embed_grad sees the finished embedding-gradient block
    (the data-parallel caller starts its all-reduce there while backward continues)."""
    H, E, V, C = 64, 32, 300, 5
    parents, tok_job, label_job = make_tree_batch(77, 24, 2, 30, V, C)
    params = make_params(3, H, E, V, C, scale=0.1, bias_scale=0.05)
    s = S.Schedule().load(parents)
    eng = TreeLSTM(H, E, V, C, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    eng.set_params(params)
    eng.load_batch(s, tok_job, label_job)
    side = torch.cuda.Stream()
    for _ in range(3):
        eng.grads.fill_(7.0)          # stale values a too-early reader would see
        eng.forward()
        eng.backward()
        eng.wait_embed_grad(side)
        with torch.cuda.stream(side):
            early = eng.grads[:V * E].clone()
        torch.cuda.synchronize()
        assert torch.equal(early, eng.grads[:V * E])
    ref = _oracle(s, tok_job, label_job, params, H, E, V, C)
    assert rel_err(early.cpu().numpy(), ref["dEmb"]) < 1e-5


@pytest.mark.parametrize("bf16", [False, True])
def test_training_reduces_the_loss(cuda, bf16):
    """Forward + backward + Adagrad on one fixed batch: the loss falls step after step at a small learning rate
    (the whole step loop, not one gradient)."""
    H, E, V, C = 64, 64, 200, 5
    parents, tok_job, label_job = make_tree_batch(31, 32, 2, 20, V, C)
    params = make_params(8, H, E, V, C, scale=0.1)
    s = S.Schedule().load(parents)
    eng = TreeLSTM(H, E, V, C, gemm_bf16=bf16, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    eng.set_params(params)
    acc = torch.zeros_like(eng.params)
    losses = []
    for _ in range(40):
        eng.load_batch(s, tok_job, label_job)
        eng.forward()
        eng.backward()
        losses.append(eng.read_loss() / s.n_total)
        eng.adagrad(acc, 0.01)
    assert all(b < a for a, b in zip(losses[:5], losses[1:6])), losses
    assert losses[-1] < 0.97 * losses[0], losses


@pytest.mark.parametrize("bf16,K,arity", [(False, 2, 2), (True, 4, 4)])
def test_root_only_labels(cuda, bf16, K, arity):
    """Only the root of every tree carries a label (the other vertices have -1, no loss term), the loss is normalised by
    the number of trees: leaves contribute nothing to the loss head, their token rows must come out as zeros."""
    from helpers import root_only_labels
    H, E, V, C = (128, 64, 300, 5) if bf16 else (40, 24, 120, 3)
    batch = 20
    parents, tok_job, label_job = make_tree_batch(47, batch, 2, 16, V, C, max_arity=arity)
    label_job = root_only_labels(parents, label_job)
    params = make_params(6, H, E, V, C, scale=0.2 if not bf16 else 0.08, bias_scale=0.05)
    s = S.Schedule().load(parents, n_slots=K)
    eng = TreeLSTM(H, E, V, C, n_slots=K, gemm_bf16=bf16, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    eng.set_params(params)
    eng.load_batch(s, tok_job, label_job, loss_rows=batch)
    eng.forward()
    eng.backward()
    loss_sum = eng.read_loss()
    out = dict(state=eng.state(), loss=eng.loss_rows(), **eng.grad_dict())
    tb = tables_from_schedule(s)
    ref = oracle.treelstm_fwd_bwd(tb, tok_job[tb["t2j"]], label_job[tb["t2j"]], params, H, E, V, C, K=K, gemm_bf16=bf16,
                                  preact_bf16=bf16, loss_rows=batch)
    tol = 5e-3 if bf16 else 1e-5
    for k in KEYS:
        assert rel_err(out[k], ref[k]) < tol, k
    assert abs(loss_sum - ref["loss"].sum()) <= tol * abs(ref["loss"].sum())
    assert np.count_nonzero(out["loss"]) == batch


@pytest.mark.parametrize("bf16", [False, True])
def test_one_vertex_per_round_schedule_gives_the_same_step(cuda, bf16):
    # The reference's serial scheduling (a Session without OPT_BATCHING) as a schedule of one-row levels:
    # the engine runs it unchanged and must reproduce the batched step -- against the oracle on the same
    # tables, and against the batched engine run job for job.
    H, E, V, C = (64, 48, 300, 5) if bf16 else (32, 20, 100, 3)
    parents, tok_job, label_job = make_tree_batch(77, 6, 2, 8, V, C)
    params = make_params(5, H, E, V, C, scale=0.05, bias_scale=0.02)
    s = S.Schedule().set_order(S.UNBATCHED).load(parents)
    assert s.n_levels == s.n_scheduled and s.max_level_rows == 1
    eng = TreeLSTM(H, E, V, C, gemm_bf16=bf16, max_vertices=s.n_total, max_level_rows=1)
    eng.set_params(params)
    eng.load_batch(s, tok_job, label_job)
    eng.forward()
    eng.backward()
    eng.read_loss()
    out = dict(state=eng.state(), loss=eng.loss_rows(), **eng.grad_dict())
    ref = _oracle(s, tok_job, label_job, params, H, E, V, C, bf16=bf16)
    tol = 5e-3 if bf16 else 1e-5
    for k in KEYS:
        assert rel_err(out[k], ref[k]) < tol, k
    sb, _, outb, _ = _run(cuda, parents, tok_job, label_job, params, H, E, V, C, bf16=bf16)
    t2j, _ = s.maps()
    _, bj2t = sb.maps()
    tol = 2e-2 if bf16 else 1e-5
    assert rel_err(out["state"][: s.n_scheduled], outb["state"][bj2t[t2j[: s.n_scheduled]]]) < tol
    for k in KEYS[2:]:
        assert rel_err(out[k], outb[k]) < tol, k


def test_single_vertex_samples_never_execute(cuda):
    # graph_scheduler.cc:180: a sample of one vertex is never scheduled.  Its vertex keeps a tensor-id-less
    # slot, contributes no loss and no gradient; the rest of the batch is unaffected.
    H, E, V, C = 32, 24, 50, 3
    parents, tok_job, label_job = make_tree_batch(91, 5, 2, 7, V, C)
    lens = (parents == -1).argmax(1) + 1
    holes = np.full((2, parents.shape[1]), -1, np.int32)
    mixed = np.concatenate([parents[:2], holes[:1], parents[2:], holes[1:]])
    cut = int(lens[:2].sum())
    tok_mixed = np.concatenate([tok_job[:cut], [7], tok_job[cut:], [9]]).astype(np.int32)
    lab_mixed = np.concatenate([label_job[:cut], [1], label_job[cut:], [2]]).astype(np.int32)
    params = make_params(4, H, E, V, C, scale=0.1, bias_scale=0.05)
    s = S.Schedule().load(mixed)
    assert s.n_total == int(lens.sum()) + 2 and s.n_scheduled == int(lens.sum())
    eng = TreeLSTM(H, E, V, C, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    eng.set_params(params)
    eng.load_batch(s, tok_mixed, lab_mixed)
    eng.forward(); eng.backward()
    loss_sum = eng.read_loss()
    got = eng.grad_dict()
    _, _, want, want_loss = _run(cuda, parents, tok_job, label_job, params, H, E, V, C)
    assert abs(loss_sum - want_loss) <= 1e-6 * abs(want_loss)
    for k in KEYS[2:]:
        assert np.array_equal(got[k], want[k]), k
    assert np.array_equal(eng.state()[: s.n_scheduled], want["state"][: s.n_scheduled])


def test_batch_of_nothing_but_single_vertices(cuda):
    H, E, V, C = 16, 16, 20, 2
    parents = np.full((3, 4), -1, np.int32)
    s = S.Schedule().load(parents)
    assert (s.n_total, s.n_scheduled, s.n_levels) == (3, 0, 0)
    eng = TreeLSTM(H, E, V, C, max_vertices=8, max_level_rows=8)
    eng.set_params(make_params(1, H, E, V, C))
    eng.load_batch(s, np.zeros(3, np.int32), np.zeros(3, np.int32))
    eng.forward(); eng.backward()
    assert eng.read_loss() == 0.0
    assert all(not g.any() for g in eng.grad_dict().values())


@pytest.mark.parametrize("bf16", [False, True])
def test_one_engine_many_batches(cuda, bf16):
    # An engine sized for the largest batch steps through batches of different shapes (its two table slots
    # alternate) and reproduces, bit for bit, what a fresh engine computes for each of them.
    H, E, V, C = (64, 64, 400, 5) if bf16 else (24, 16, 60, 4)
    params = make_params(8, H, E, V, C, scale=0.08, bias_scale=0.03)
    batches = [make_tree_batch(300 + i, b, 2, hi, V, C) for i, (b, hi) in enumerate([(9, 12), (2, 3), (14, 20), (1, 2), (9, 12)])]
    scheds = [S.Schedule().load(p) for p, _, _ in batches]
    eng = TreeLSTM(H, E, V, C, gemm_bf16=bf16, max_vertices=max(s.n_total for s in scheds),
                   max_level_rows=max(s.max_level_rows for s in scheds))
    eng.set_params(params)
    for (parents, tok_job, label_job), s in zip(batches, scheds):
        eng.load_batch(s, tok_job, label_job)
        eng.forward(); eng.backward()
        loss_sum = eng.read_loss()
        got = dict(state=eng.state()[: s.n_total], loss=eng.loss_rows()[: s.n_total], **eng.grad_dict())
        _, _, want, want_loss = _run(cuda, parents, tok_job, label_job, params, H, E, V, C, bf16=bf16)
        assert loss_sum == want_loss
        for k in KEYS:
            assert np.array_equal(got[k], want[k][: len(got[k])] if k in ("state", "loss") else want[k]), k


def test_level_one_by_token_with_few_distinct_tokens(cuda, monkeypatch):
    # A tiny vocabulary makes every token own hundreds of leaves and of level-1 links, so the per-token link sums and
    # the per-token gradient sums run through their multi-chunk paths; the result must match the oracle and the
    # per-vertex form of level 1 (CAVS_LEVEL1_BY_TOKEN=0, read when an engine is created).
    H, E, V, C = 64, 32, 7, 5
    parents, tok_job, label_job = make_tree_batch(808, 64, 2, 40, V, C)
    params = make_params(12, H, E, V, C, scale=0.05, bias_scale=0.02)
    s, eng, out, loss_sum = _run(cuda, parents, tok_job, label_job, params, H, E, V, C, bf16=True)
    counts = np.bincount(tok_job[s.maps()[0][: s.level_off[1]]], minlength=V)
    assert counts.max() > 256                                   # more than one chunk for the most frequent token
    ref32 = _oracle(s, tok_job, label_job, params, H, E, V, C)
    refbf = _oracle(s, tok_job, label_job, params, H, E, V, C, bf16=True)
    for k in KEYS:
        assert rel_err(out[k], ref32[k]) < 2e-2, k
        assert rel_err(out[k], refbf[k]) < 5e-3, k
    monkeypatch.setenv("CAVS_LEVEL1_BY_TOKEN", "0")
    _, _, per_vertex, loss_pv = _run(cuda, parents, tok_job, label_job, params, H, E, V, C, bf16=True)
    monkeypatch.setenv("CAVS_LEVEL1_BY_TOKEN", "1")
    assert abs(loss_sum - loss_pv) < 2e-3 * abs(loss_pv)
    for k in KEYS:
        assert rel_err(out[k], per_vertex[k]) < 5e-3, k


@pytest.mark.parametrize("bf16,H,C", [(False, 2048, 5), (True, 1280, 8)])
def test_loss_head_that_stores_the_hidden_gradient(cuda, bf16, H, C):
    # classes * hidden above 8192: the cell gradient cannot rebuild d(h) from the d(logits) row, so the loss head
    # writes d(h) for every vertex and the backward cell reads it -- the engine branch no other case reaches.
    E, V = 32, 60
    parents, tok_job, label_job = make_tree_batch(404, 6, 2, 7, V, C)
    params = make_params(13, H, E, V, C, scale=0.03, bias_scale=0.02)
    s, eng, out, loss_sum = _run(cuda, parents, tok_job, label_job, params, H, E, V, C, bf16=bf16)
    ref = _oracle(s, tok_job, label_job, params, H, E, V, C, bf16=bf16)
    tol = 5e-3 if bf16 else 1e-5
    for k in KEYS:
        assert_close(out[k], ref[k], tol, k, value_tol=VALUE_FACTOR * tol * (4 if bf16 else 1))
    assert abs(loss_sum - ref["loss"].sum()) <= tol * abs(ref["loss"].sum())
    # and the stored d(h) itself: (softmax - onehot) / rows . Wc, row by row
    from helpers import loss_head_reference
    tb = tables_from_schedule(s)
    dh = eng.peek(2, (s.n_scheduled, H))
    want = loss_head_reference(ref["state"][:, :H], label_job[tb["t2j"]], params["Wc"], params["bc"], 1.0 / s.n_scheduled)
    assert_close(dh, want["dH"], tol, "dH", value_tol=VALUE_FACTOR * tol * (4 if bf16 else 1))


def test_peek_returns_every_array_with_its_size(cuda):
    import ctypes
    from cavs_b200 import CavsError, check, lib
    H, E, V, C, K = 64, 32, 40, 12, 2      # 12 classes: the wide head, which materialises d(h) (array 2)
    parents, tok_job, label_job = make_tree_batch(3, 4, 2, 6, V, C)
    s = S.Schedule().load(parents)
    n = s.n_scheduled
    eng = TreeLSTM(H, E, V, C, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    eng.set_params(make_params(1, H, E, V, C))
    eng.load_batch(s, tok_job, label_job)
    eng.forward(); eng.backward(); eng.read_loss()
    lo, hi = eng.workspace.data_ptr(), eng.workspace.data_ptr() + eng.workspace.numel()
    want = {0: n * 2 * H * 4, 1: n * 4, 2: n * H * 4, 3: n * 2 * H * 4, 4: n * (3 + K) * H * 4, 6: 8}
    seen = {}
    for what, nbytes in want.items():
        p, b = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().cavs_treelstm_peek(eng._h, what, ctypes.byref(p), ctypes.byref(b)))
        assert b.value == nbytes, what
        assert lo <= p.value and p.value + nbytes <= hi, what
        seen[what] = p.value
    assert len(set(seen.values())) == len(seen)          # six different arrays
    with pytest.raises(CavsError):                         # d(x) exists only with dense inputs
        eng.peek(5, (n, E))
    with pytest.raises(CavsError):
        eng.peek(7, (1,))
    # the saved gates of an internal vertex are what the forward pass computed: i, o in (0,1), u in (-1,1)
    gates = eng.peek(4, (n, (3 + K) * H))
    first_internal = int(s.level_off[1])
    g = gates[first_internal:]
    assert (g[:, :2 * H] > 0).all() and (g[:, :2 * H] < 1).all() and (np.abs(g[:, 2 * H:3 * H]) < 1).all()
    # bf16 mode with the gate epilogue: the arena is split at its capacity, G3 [cap, 3H] then GF [cap, K, H], in half
    cap = s.n_total + 7
    engb = TreeLSTM(H, E, V, 5, gemm_bf16=True, max_vertices=cap, max_level_rows=s.max_level_rows)
    engb.set_params(make_params(1, H, E, V, 5))
    engb.load_batch(s, tok_job, label_job % 5)
    engb.forward()
    p, b = ctypes.c_void_p(), ctypes.c_size_t()
    check(lib().cavs_treelstm_peek(engb._h, 4, ctypes.byref(p), ctypes.byref(b)))
    assert b.value == cap * (3 + K) * H * 2
    off = p.value - engb.workspace.data_ptr()
    arena = engb.workspace[off:off + b.value].view(torch.float16).cpu().numpy().astype(np.float32)
    g3, gf = arena[:cap * 3 * H].reshape(cap, 3 * H), arena[cap * 3 * H:].reshape(cap, K, H)
    assert (g3[first_internal:n, :2 * H] > 0).all() and (g3[first_internal:n, :2 * H] < 1).all()
    assert (np.abs(g3[first_internal:n, 2 * H:]) <= 1).all()
    assert (gf[first_internal:n] > 0).all() and (gf[first_internal:n] < 1).all()
    # fused head: d(h) is not materialised and peek says so
    eng5 = TreeLSTM(H, E, V, 5, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    with pytest.raises(CavsError) as e:
        eng5.peek(2, (n, H))
    assert e.value.status == 6


@pytest.mark.parametrize("bf16", [False, True])
def test_forward_only_caller_may_reload_while_a_forward_is_in_flight(cuda, bf16):
    # forward, load, forward, load, ... without any backward: the table slot of a forward pass still running must
    # not be overwritten by the upload of the batch after next.
    H, E, V, C = (64, 64, 300, 5) if bf16 else (32, 24, 80, 4)
    params = make_params(21, H, E, V, C, scale=0.08, bias_scale=0.03)
    batches = [make_tree_batch(500 + i, b, 2, hi, V, C) for i, (b, hi) in enumerate([(30, 40), (3, 4), (25, 40), (2, 3), (30, 30)])]
    scheds = [S.Schedule().load(p) for p, _, _ in batches]
    eng = TreeLSTM(H, E, V, C, gemm_bf16=bf16, max_vertices=max(x.n_total for x in scheds),
                   max_level_rows=max(x.max_level_rows for x in scheds))
    eng.set_params(params)
    states = []
    eng.load_batch(scheds[0], batches[0][1], batches[0][2])
    for i in range(len(batches)):
        eng.forward()
        if i + 1 < len(batches):
            eng.load_batch(scheds[i + 1], batches[i + 1][1], batches[i + 1][2])   # stages the next batch at once
            eng.load_batch(scheds[i + 1], batches[i + 1][1], batches[i + 1][2])   # and once more: same staged slot
        eng.n = scheds[i].n_scheduled
        states.append(torch.from_numpy(eng.state()[: scheds[i].n_scheduled].copy()))
    for (parents, tok_job, label_job), s, got in zip(batches, scheds, states):
        ref = _oracle(s, tok_job, label_job, params, H, E, V, C, bf16=bf16)
        assert rel_err(got.numpy(), ref["state"][: s.n_scheduled]) < (5e-3 if bf16 else 1e-5)


def test_expired_device_wait_surfaces_as_timeout(cuda):
    # Every wait inside the tensor-core GEMM is bounded.  The self-test entry runs that kernel with its operand
    # loads withheld and a short poll limit: all of its waits run out, it must raise the status word, release its
    # tensor memory and return; the engine whose status word it was then reports CAVS_ERR_TIMEOUT from read_loss,
    # and the context keeps working (an ordinary GEMM right after gives the right product).
    import ctypes
    from cavs_b200 import CavsError, check, lib
    L = lib()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ll = ctypes.c_longlong
    m, n, k = 300, 384, 256
    a = torch.randn((m, k), device=cuda).to(torch.bfloat16)
    b = torch.randn((k, n), device=cuda).to(torch.bfloat16)
    c = torch.full((m, n), 7.0, device=cuda)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    # a stand-alone status word first
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    check(L.cavs_gemm_bf16_wait_selftest(vp(c), ll(n), vp(a), ll(k), vp(b), ll(n), m, n, k, vp(status), st))
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert bool((c == 7.0).all())                     # nothing was written
    # the same through an engine's status word
    H, E, V, C = 64, 64, 50, 5
    parents, tok_job, label_job = make_tree_batch(5, 4, 2, 6, V, C)
    s = S.Schedule().load(parents)
    eng = TreeLSTM(H, E, V, C, gemm_bf16=True, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    eng.set_params(make_params(2, H, E, V, C))
    eng.load_batch(s, tok_job, label_job)
    eng.forward(); eng.backward()
    assert eng.read_loss() > 0
    tail = eng.device_view(6, (2,))
    check(L.cavs_gemm_bf16_wait_selftest(vp(c), ll(n), vp(a), ll(k), vp(b), ll(n), m, n, k, ctypes.c_void_p(tail.data_ptr() + 4), st))
    with pytest.raises(CavsError) as e:
        eng.read_loss()
    assert e.value.status == 4
    # the context is intact: same kernel, loads no longer withheld
    check(L.cavs_gemm_bf16(vp(c), ll(n), 0, vp(a), ll(k), 0, vp(b), ll(n), 1, m, n, k, 1, ctypes.c_void_p(0), ctypes.c_size_t(0),
                           vp(status), st))
    torch.cuda.synchronize()
    want = a.float() @ b.float()
    assert float((c - want).abs().max() / want.abs().max()) < 1e-5


def test_staging_on_the_helper_thread_gives_the_same_steps(cuda):
    # stage_async schedules and packs batch i+1 on the engine's helper thread while this thread enqueues step i; the
    # results must be those of the synchronous sequence, bit for bit, and a malformed batch must surface at the wait.
    from cavs_b200 import CavsError
    H, E, V, C = 64, 64, 300, 5
    params = make_params(31, H, E, V, C, scale=0.08, bias_scale=0.03)
    batches = [make_tree_batch(700 + i, b, 2, hi, V, C) for i, (b, hi) in enumerate([(20, 30), (3, 4), (25, 40), (9, 12)])]
    cap = dict(gemm_bf16=True, max_vertices=4096, max_level_rows=4096)

    def run(mode):
        eng = TreeLSTM(H, E, V, C, **cap)
        eng.set_params(params)
        s = S.Schedule()
        keep = [(np.ascontiguousarray(p), np.ascontiguousarray(t), np.ascontiguousarray(l)) for p, t, l in batches]
        out = []
        if mode != "sync":
            eng.stage_async(s, *keep[0])
        for i in range(len(keep)):
            if mode == "sync":
                eng.stage(s, *keep[i])
            if mode == "promote":
                # explicit promotion: batch i becomes current, batch i+1 is staged WHILE step i is being enqueued
                eng.promote()
                if i + 1 < len(keep):
                    eng.stage_async(s, *keep[i + 1])
            eng.step(None, eng.OPT_SGD, None, 0.05)        # "async": waits for the pending request, promotes, runs the step
            if mode == "async" and i + 1 < len(keep):
                eng.stage_async(s, *keep[i + 1])
            out.append((eng.read_loss(), eng.grads.cpu().numpy().copy()))
        return out

    want = run("sync")
    for mode in ("async", "promote"):
        for (la, ga), (lb, gb) in zip(run(mode), want):
            assert la == lb and np.array_equal(ga, gb), mode

    # the caller schedules on a thread of its own (two schedule objects alternate) and hands the engine a loaded
    # schedule: only the packing runs on the helper thread
    import threading
    eng = TreeLSTM(H, E, V, C, **cap)
    eng.set_params(params)
    keep = [(np.ascontiguousarray(p), np.ascontiguousarray(t), np.ascontiguousarray(l)) for p, t, l in batches]
    scheds = [S.Schedule(), S.Schedule()]
    scheds[0].load(keep[0][0])
    eng.stage_async(scheds[0], None, keep[0][1], keep[0][2])
    worker = threading.Thread(target=scheds[1].load, args=(keep[1][0],))
    worker.start()
    for i in range(len(keep)):
        eng.promote()
        if i + 1 < len(keep):
            worker.join()
            eng.stage_async(scheds[(i + 1) % 2], None, keep[i + 1][1], keep[i + 1][2])
            if i + 2 < len(keep):
                worker = threading.Thread(target=scheds[i % 2].load, args=(keep[i + 2][0],))
                worker.start()
        eng.step(None, eng.OPT_SGD, None, 0.05)
        assert eng.read_loss() == want[i][0] and np.array_equal(eng.grads.cpu().numpy(), want[i][1]), i
    eng = TreeLSTM(H, E, V, C, **cap)
    eng.set_params(params)
    bad = np.array([[5, 5, -1, -1]], np.int32)             # parent index out of range
    eng.stage_async(S.Schedule(), bad, np.zeros(4, np.int32), np.zeros(4, np.int32))
    with pytest.raises(CavsError) as e:
        eng.stage_wait()
    assert e.value.status == 2


@pytest.mark.parametrize("bf16", [False, True])
def test_exchange_rows_give_the_dense_update(cuda, bf16):
    # With a list of exchange rows the embedding block of the gradient buffer is compact (one row per listed row) and
    # step() updates only the listed rows: the parameters after Adagrad steps must equal the dense path's bit for bit,
    # whether the list is exactly the batch's tokens or a superset of them.
    from cavs_b200 import CavsError
    H, E, V, C = 64, 64, 500, 5
    params = make_params(41, H, E, V, C, scale=0.08, bias_scale=0.03)
    batches = [make_tree_batch(900 + i, 12, 2, 20, V, C) for i in range(3)]
    cap = dict(gemm_bf16=bf16, max_vertices=2048, max_level_rows=2048)

    def run(mode):
        eng = TreeLSTM(H, E, V, C, **cap)
        eng.set_params(params)
        acc = torch.zeros_like(eng.params)
        s = S.Schedule()
        emb_grads = []
        for p, t, l in batches:
            rows = None
            if mode == "exact":
                rows = np.unique(t)
            elif mode == "superset":
                rows = np.union1d(np.unique(t), np.arange(0, V, 7))
            eng.stage(s, np.ascontiguousarray(p), t, l, exchange_rows=rows)
            eng.step(None, eng.OPT_ADAGRAD, acc, 0.05)
            g = eng.grads.cpu().numpy()
            if rows is not None:
                dense = np.zeros((V, E), np.float32)
                dense[rows] = g[:rows.size * E].reshape(rows.size, E)
                g = np.concatenate([dense.reshape(-1), g[V * E:]])
            emb_grads.append(g)
        return eng.params.cpu().numpy(), acc.cpu().numpy(), emb_grads

    want = run("dense")
    for mode in ("exact", "superset"):
        got = run(mode)
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]), mode
        for a, b in zip(got[2], want[2]):
            assert np.array_equal(a, b), mode

    # the pipelined loop (explicit promotion, next batch staged on the helper thread while this step is enqueued, no
    # host synchronisation between steps): the row update of step i reads its row list from tables that the upload of
    # batch i+2 must not overwrite before it has run
    eng = TreeLSTM(H, E, V, C, **cap)
    eng.set_params(params)
    acc = torch.zeros_like(eng.params)
    s = S.Schedule()
    keep = [(np.ascontiguousarray(p), np.ascontiguousarray(t), np.ascontiguousarray(l)) for p, t, l in batches]
    eng.stage_async(s, *keep[0], exchange_rows=np.unique(keep[0][1]))
    for i in range(len(keep)):
        eng.promote()
        if i + 1 < len(keep):
            eng.stage_async(s, *keep[i + 1], exchange_rows=np.unique(keep[i + 1][1]))
        eng.step(None, eng.OPT_ADAGRAD, acc, 0.05)
    torch.cuda.synchronize()
    assert np.array_equal(eng.params.cpu().numpy(), want[0]) and np.array_equal(acc.cpu().numpy(), want[1])
    # the list is consumed by one load: the next batch is dense again
    eng = TreeLSTM(H, E, V, C, **cap)
    eng.set_params(params)
    s = S.Schedule()
    p, t, l = batches[0]
    eng.stage(s, np.ascontiguousarray(p), t, l, exchange_rows=np.unique(t))
    eng.stage(s, np.ascontiguousarray(p), t, l)
    eng.step(None, eng.OPT_NONE)
    assert np.array_equal(eng.grads.cpu().numpy(), want[2][0])
    # a token of the batch missing from the list, or a list out of order, is an argument error at load time
    with pytest.raises(CavsError) as e:
        eng.stage(s, np.ascontiguousarray(p), t, l, exchange_rows=np.unique(t)[1:])
    assert e.value.status == 1
    with pytest.raises(CavsError) as e:
        eng.set_exchange_rows(np.array([5, 3], np.int32))
    assert e.value.status == 1
