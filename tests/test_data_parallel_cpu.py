"""Data-parallel path on CPU ranks (gloo, world_size 2): trees are sharded by instance, every rank
normalises its loss by the GLOBAL vertex count, and one all-reduce of the flat gradient gives the
single-process gradient.  The compute on each rank is the CPU oracle (the CUDA engine needs a GPU);
what is under test is the host-side sharding / normalisation / reduction logic that bench.py uses."""
import os
import sys
from pathlib import Path

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
KEYS = ("dEmb", "dW", "dU", "dB", "dWc", "dbc")
H, E, V, C = 12, 10, 40, 3


def _shard_grads(rank, world, parents, tok_job, label_job, params):
    import oracle
    from cavs_b200 import schedule as S
    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import tables_from_schedule
    lens = (parents == -1).argmax(1) + 1
    per = parents.shape[0] // world
    lo, hi = rank * per, (rank + 1) * per
    starts = np.concatenate([[0], np.cumsum(lens)])
    s = S.Schedule().load(parents[lo:hi])
    tb = tables_from_schedule(s)
    tok, lab = tok_job[starts[lo]:starts[hi]], label_job[starts[lo]:starts[hi]]
    out = oracle.treelstm_fwd_bwd(tb, tok[tb["t2j"]], lab[tb["t2j"]], params, H, E, V, C, loss_rows=int(lens.sum()))
    return out


def _worker(rank, world, port, payload, result_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, str(ROOT))
    import torch
    dist.init_process_group("gloo", rank=rank, world_size=world)
    parents, tok_job, label_job, params = payload
    out = _shard_grads(rank, world, parents, tok_job, label_job, params)
    flat = torch.from_numpy(np.concatenate([out[k].ravel() for k in KEYS]).astype(np.float32))
    dist.all_reduce(flat)                         # the one collective of a step
    loss = torch.tensor([float(out["loss"].sum())])
    dist.all_reduce(loss)
    if rank == 0:
        np.savez(result_path, flat=flat.numpy(), loss=loss.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradient_equals_single_process(tmp_path):
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle
    from cavs_b200 import schedule as S
    from helpers import make_params, make_tree_batch, rel_err, tables_from_schedule
    parents, tok_job, label_job = make_tree_batch(31, 8, 2, 7, V, C)
    params = make_params(5, H, E, V, C, scale=0.4, bias_scale=0.2)
    s = S.Schedule().load(parents)
    tb = tables_from_schedule(s)
    ref = oracle.treelstm_fwd_bwd(tb, tok_job[tb["t2j"]], label_job[tb["t2j"]], params, H, E, V, C)
    want = np.concatenate([ref[k].ravel() for k in KEYS])
    result = tmp_path / "dp.npz"
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, (parents, tok_job, label_job, params), str(result)), nprocs=2, join=True)
    got = np.load(result)
    assert rel_err(got["flat"], want) < 1e-5
    assert abs(float(got["loss"][0]) - float(ref["loss"].sum())) < 1e-4 * abs(float(ref["loss"].sum()))
