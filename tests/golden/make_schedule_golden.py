"""Generates tests/golden/schedule_streams.json by running the reference's own graph scheduler
(cavs/midend/graph_scheduler.{h,cc}, compiled by oracle/Makefile into oracle/_ref/) on a fixed
set of small graphs.  Run where the reference checkout is present:

    make -C oracle && python tests/golden/make_schedule_golden.py
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402
from cavs_b200 import schedule as S  # noqa: E402

cases = [
    ("two_leaf_tree", [[2, 2, -1]]),
    ("three_leaf_left", [[3, 3, 4, 4, -1]]),
    ("three_leaf_right", [[4, 3, 3, 4, -1]]),
    ("tree_plus_chain", [[3, 3, 4, 4, -1, -1], [1, 2, -1, -1, -1, -1]]),
    ("skewed_pair", [[2, 2, -1, -1, -1], [3, 3, 4, 4, -1]]),
    ("ragged_chains_short_first", [[1, -1, -1, -1], [1, 2, 3, -1]]),
    ("ragged_chains_long_first", [[1, 2, 3, -1], [1, -1, -1, -1]]),
    ("single_vertex_sample", [[-1, -1], [1, -1]]),
    ("unary_over_binary", [[2, 2, 3, -1]]),
    ("fixed_chains", [[1, 2, 3, -1]] * 3),
]
out = []
for name, p in cases:
    out.append(dict(name=name, parents=p, stream=oracle.ref_schedule_stream(np.array(p, np.int32)).tolist()))
for seed in range(12):
    p = S.synth_trees(1000 + seed, 3 + seed % 4, 1 + seed % 3, 3 + seed)[0]
    out.append(dict(name=f"random_trees_{seed}", parents=p.tolist(), stream=oracle.ref_schedule_stream(p).tolist()))
for seed in range(4):
    p = S.synth_chains(2000 + seed, 4, 1, 6 + seed)
    out.append(dict(name=f"random_chains_{seed}", parents=p.tolist(), stream=oracle.ref_schedule_stream(p).tolist()))
(Path(__file__).parent / "schedule_streams.json").write_text(json.dumps(out, separators=(",", ":")))
print(len(out), "cases")
