"""Generates tests/golden/schedule_streams.json by running the reference's own graph schedulers
(cavs/midend/graph_scheduler.{h,cc}, compiled by oracle/Makefile into oracle/_ref/) on a fixed
set of small graphs: `stream` is BatchGraphScheduler's forward + backward sweep, `serial`
SerialGraphScheduler's (layouts: oracle/refsched_driver.cc).  Run where the reference checkout is present:

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
    ("single_vertex_sample_in_the_middle", [[2, 2, -1, -1, -1], [-1, -1, -1, -1, -1], [3, 3, 4, 4, -1]]),
    ("single_vertex_sample_last", [[1, 2, -1], [-1, -1, -1]]),
]


def record(name, p):
    p = np.array(p, np.int32)
    return dict(name=name, parents=p.tolist(), stream=oracle.ref_schedule_stream(p).tolist(),
                serial=oracle.ref_serial_stream(p).tolist())


out = []
for name, p in cases:
    out.append(record(name, p))
for seed in range(12):
    p = S.synth_trees(1000 + seed, 3 + seed % 4, 1 + seed % 3, 3 + seed)[0]
    out.append(record(f"random_trees_{seed}", p))
for seed in range(4):
    p = S.synth_chains(2000 + seed, 4, 1, 6 + seed)
    out.append(record(f"random_chains_{seed}", p))
(Path(__file__).parent / "schedule_streams.json").write_text(json.dumps(out, separators=(",", ":")))
print(len(out), "cases")
