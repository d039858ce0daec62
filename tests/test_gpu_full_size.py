"""The data-parallel Tree-LSTM configuration at its full size (4096 random binary trees with 2..128 leaves, hidden =
embedding = 1024, vocabulary 50,000, 5 classes, bf16 GEMMs), checked through properties that do not need the CPU
oracle to run the whole batch:
  * reruns are bit-identical;
  * shard additivity, the data-parallel contract: with the loss normalised by the global vertex count, the gradients
    of the two halves of the batch add up to the gradients of the whole batch;
  * a sample against the oracle: with labels kept only on the first trees, the gradients of the whole batch are the
    gradients of those trees alone, and their vertices' states do not depend on the rest of the batch -- both are
    compared with the oracle run on the sample by itself."""
import numpy as np
import pytest

import bench
import oracle
from cavs_b200 import schedule as S
from cavs_b200.treelstm import TreeLSTM
from helpers import rel_err, tables_from_schedule

pytestmark = pytest.mark.gpu
KEYS = ("dEmb", "dW", "dU", "dB", "dWc", "dbc")


def _step(eng, sched, tok, lab, loss_rows):
    eng.load_batch(sched, tok, lab, loss_rows=loss_rows)
    eng.forward()
    eng.backward()
    return eng.read_loss(), eng.grad_dict()


def test_data_parallel_treelstm_at_full_size(cuda):
    wl = bench.WORKLOADS["dp_treelstm"]
    H, E, V, C = wl["hidden"], wl["embed"], wl["vocab"], wl["classes"]
    parents, tok, lab, total = bench.make_batch(wl, 0, 0, 1)
    s = S.Schedule().load(parents)
    assert s.n_total == total
    eng = TreeLSTM(H, E, V, C, gemm_bf16=True, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    params = bench.make_params(wl)
    eng.set_params(params)

    loss, g = _step(eng, s, tok, lab, total)
    assert np.isfinite(loss) and all(np.isfinite(v).all() for v in g.values())
    loss2, g2 = _step(eng, s, tok, lab, total)
    assert loss2 == loss and all(np.array_equal(g[k], g2[k]) for k in KEYS)           # deterministic

    # shard additivity
    acc, loss_sum = {k: np.zeros_like(g[k], np.float64) for k in KEYS}, 0.0
    for r in range(2):
        p_r, tok_r, lab_r, _ = bench.make_batch(wl, 0, r, 2)
        s_r = S.Schedule().load(p_r)
        l_r, g_r = _step(eng, s_r, tok_r, lab_r, total)
        loss_sum += l_r
        for k in KEYS:
            acc[k] += g_r[k]
    assert abs(loss_sum - loss) <= 1e-4 * abs(loss)
    for k in KEYS:
        # the per-token gradient sums are rounded to bf16 (GEMM operands) per shard instead of once: ~2^-9 relative
        assert rel_err(acc[k], g[k]) < 1e-2, k

    # a sample against the oracle: labels only on the first trees
    n_sample = 6
    lens = (parents == -1).argmax(1) + 1
    n_keep = int(lens[:n_sample].sum())
    lab_masked = lab.copy()
    lab_masked[n_keep:] = -1
    _, g_m = _step(eng, s, tok, lab_masked, n_keep)
    state = eng.state()
    s_small = S.Schedule().load(parents[:n_sample])
    tb = tables_from_schedule(s_small)
    ref = oracle.treelstm_fwd_bwd(tb, tok[:n_keep][tb["t2j"]], lab[:n_keep][tb["t2j"]], params, H, E, V, C, gemm_bf16=True,
                                  preact_bf16=True, loss_rows=n_keep)
    for k in KEYS:
        assert rel_err(g_m[k], ref[k]) < 5e-3, k
    # states of the sample's vertices: job id j of the sample is job id j of the whole batch
    _, j2t_full = s.maps()
    _, j2t_small = s_small.maps()
    got = state[j2t_full[:n_keep]]
    want = ref["state"][j2t_small[:n_keep]]
    assert rel_err(got, want) < 5e-3
