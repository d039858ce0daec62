"""The CUDA Tree-LSTM step (forward, loss, backward, update) through the C ABI vs the CPU oracle
on identical seeded inputs.  fp32 configurations: 1e-5 relative; bf16-GEMM configurations: 2e-2
relative (and tighter against the oracle run with bf16-rounded GEMM operands)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from cavs_b200 import schedule as S
from cavs_b200.treelstm import TreeLSTM
from helpers import make_params, make_tree_batch, rel_err, tables_from_schedule

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def level_one_by_token(monkeypatch):
    # Small test batches have fewer level-1 rows than distinct tokens, where the engine would choose the per-vertex
    # form of level 1 by itself: force the per-token form so that every bf16 case below runs it.
    monkeypatch.setenv("CAVS_LEVEL1_BY_TOKEN", "1")
KEYS = ("state", "loss", "dEmb", "dW", "dU", "dB", "dWc", "dbc")
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
        assert rel_err(out[k], g["r_" + k]) < 1e-5, k
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
        assert rel_err(out[k], ref[k]) < 1e-5, k
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
        assert rel_err(out[k], ref32[k]) < 2e-2, k      # the bf16-GEMM contract
        assert rel_err(out[k], refbf[k]) < 5e-3, k      # same rounding points as the oracle's bf16 mode


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
        assert rel_err(out[k], ref[k]) < 1e-5, k


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
