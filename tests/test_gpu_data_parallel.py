"""Two GPUs, one process each: cavs_treelstm_step with the library's own NCCL communicator gives every rank the
gradient of the GLOBAL batch -- equal to what one GPU computes for the whole batch -- and, after identical SGD
updates (linear in the gradient, so the comparison keeps its tolerance), the same parameters.  Skipped where fewer than two GPUs are visible.  The ranks are child processes;
the communicator id travels through a file (no torch.distributed involved), NVLS is off (plain ring / tree kernels).
With `sparse` the ranks exchange only the embedding rows the global batch touches (cavs_treelstm_set_exchange_rows): same
gradients, same parameters."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu

WORKER = r'''
import sys
rank, world, id_file, out_file, bf16, root = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], int(sys.argv[5]), sys.argv[6]
sparse = int(sys.argv[7])
sys.path.insert(0, root); sys.path.insert(0, root + "/tests")
import numpy as np, torch
from cavs_b200 import schedule as S
from cavs_b200.comm import Comm
from cavs_b200.treelstm import TreeLSTM
from helpers import make_params, make_tree_batch
torch.cuda.set_device(rank)
H, E, V, C = (128, 64, 300, 5) if bf16 else (48, 32, 120, 4)
parents, tok_job, label_job = make_tree_batch(77, 16, 2, 24, V, C)
params = make_params(4, H, E, V, C, scale=0.1, bias_scale=0.05)
lens = (parents == -1).argmax(1) + 1
starts = np.concatenate([[0], np.cumsum(lens)])
per = parents.shape[0] // world
lo, hi = rank * per, (rank + 1) * per
comm = Comm.from_file(id_file, rank, world)
s = S.Schedule()
eng = TreeLSTM(H, E, V, C, gemm_bf16=bool(bf16), max_vertices=int(lens.sum()), max_level_rows=int(lens.sum()), device=f"cuda:{rank}")
eng.set_params(params)
shard = np.ascontiguousarray(parents[lo:hi])
tok, lab = np.ascontiguousarray(tok_job[starts[lo]:starts[hi]]), np.ascontiguousarray(label_job[starts[lo]:starts[hi]])
out = {}
# sparse exchange: the table rows any rank touches -- the distinct tokens of the GLOBAL batch, the same list on every rank
rows = np.unique(tok_job).astype(np.int32) if sparse else None
eng.stage(s, shard, tok, lab, loss_rows=int(lens.sum()), exchange_rows=rows)
eng.step(comm, eng.OPT_NONE)                       # gradients only: summed over the ranks
g = eng.grads.cpu().numpy()
if sparse:                                         # one gradient row per listed row -> back to table layout for the comparison
    dense = np.zeros(V * E, np.float32).reshape(V, E)
    dense[rows] = g[:rows.size * E].reshape(rows.size, E)
    g = np.concatenate([dense.reshape(-1), g[V * E:]])
out["grads"] = g
out["loss"] = np.array([eng.read_loss()])
for _ in range(3):                                 # three full training steps
    eng.stage(s, shard, tok, lab, loss_rows=int(lens.sum()), exchange_rows=rows)
    eng.step(comm, eng.OPT_SGD, None, 0.1)
torch.cuda.synchronize()
out["params"] = eng.params.cpu().numpy()
if rank == 0:                                       # the same thing on one GPU over the whole batch
    one = TreeLSTM(H, E, V, C, gemm_bf16=bool(bf16), max_vertices=int(lens.sum()), max_level_rows=int(lens.sum()), device="cuda:0")
    one.set_params(params)
    s1 = S.Schedule()
    one.stage(s1, parents, tok_job, label_job)
    one.step(None, one.OPT_NONE)
    out["grads_one"] = one.grads.cpu().numpy()
    out["loss_one"] = np.array([one.read_loss()])
    for _ in range(3):
        one.stage(s1, parents, tok_job, label_job)
        one.step(None, one.OPT_SGD, None, 0.1)
    torch.cuda.synchronize()
    out["params_one"] = one.params.cpu().numpy()
np.savez(out_file + f".{rank}.npz", **out)
comm.close()
'''


@pytest.mark.parametrize("bf16,sparse", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_two_ranks_compute_the_single_gpu_step(cuda, tmp_path, bf16, sparse):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import rel_err
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    id_file, out_file = str(tmp_path / "comm_id"), str(tmp_path / "out")
    procs = [subprocess.Popen([sys.executable, "-c", WORKER, str(r), "2", id_file, out_file, str(bf16), str(ROOT), str(sparse)], env=env)
             for r in range(2)]
    for p in procs:
        assert p.wait(timeout=600) == 0
    r0, r1 = np.load(out_file + ".0.npz"), np.load(out_file + ".1.npz")
    tol = 5e-3 if bf16 else 1e-5
    assert np.array_equal(r0["grads"], r1["grads"])            # every rank holds the same sum
    assert rel_err(r0["grads"], r0["grads_one"]) < tol
    assert abs(float(r0["loss"][0] + r1["loss"][0]) - float(r0["loss_one"][0])) < tol * abs(float(r0["loss_one"][0]))
    assert np.array_equal(r0["params"], r1["params"])          # and stays in step after the updates
    assert rel_err(r0["params"], r0["params_one"]) < tol
