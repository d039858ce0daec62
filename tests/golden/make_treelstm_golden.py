"""Generates tests/golden/treelstm_small.npz: inputs and float64 PyTorch-autograd results of the
child-sum Tree-LSTM step (tests/torch_ref.py) on a small seeded batch.  The C oracle and the CUDA
path are both checked against this file.

    python tests/golden/make_treelstm_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
from cavs_b200 import schedule as S  # noqa: E402
from helpers import make_params, make_tree_batch, tables_from_schedule  # noqa: E402
from torch_ref import treelstm_autograd  # noqa: E402

H, E, V, C = 16, 24, 40, 5
parents, tok_job, label_job = make_tree_batch(4242, 6, 2, 7, V, C)
s = S.Schedule().load(parents)
tb = tables_from_schedule(s)
tok, label = tok_job[tb["t2j"]], label_job[tb["t2j"]]
params = make_params(4242, H, E, V, C, scale=0.3, bias_scale=0.2)
ref = treelstm_autograd(tb, tok, label, params, H, E, V, C)
np.savez_compressed(Path(__file__).parent / "treelstm_small.npz", parents=parents, tok_job=tok_job, label_job=label_job,
                    dims=np.array([H, E, V, C]), **{"p_" + k: v for k, v in params.items()},
                    **{"r_" + k: v.astype(np.float64) for k, v in ref.items()})
print("vertices", s.n_total, "levels", s.n_levels)
