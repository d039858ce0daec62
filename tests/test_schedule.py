"""Level schedules and index tables: product scheduler vs the reference's own scheduler
(compiled from the reference sources as an oracle, when it was built on this machine),
vs the plain-C restatement, and vs committed golden streams."""
import json
from pathlib import Path

import numpy as np
import pytest

import oracle
from cavs_b200 import CavsError, schedule as S

GOLDEN = Path(__file__).parent / "golden" / "schedule_streams.json"


def _random_graph(seed):
    rng = np.random.default_rng(seed)
    b = int(rng.integers(1, 12))
    lo = int(rng.integers(1, 4))
    hi = lo + int(rng.integers(0, 12))
    if seed % 3 == 0:
        return S.synth_chains(seed, b, lo, hi)
    return S.synth_trees(seed, b, lo, hi)[0]


def test_golden_streams_match_oracle_and_product():
    cases = json.loads(GOLDEN.read_text())
    assert len(cases) >= 20
    for case in cases:
        parents = np.array(case["parents"], np.int32)
        want = np.array(case["stream"], np.int32)
        assert np.array_equal(oracle.schedule_stream(parents), want), case["name"]
        assert np.array_equal(S.Schedule().load(parents).ref_stream(), want), case["name"]
        # one vertex per round (SerialGraphScheduler)
        want = np.array(case["serial"], np.int32)
        assert np.array_equal(oracle.serial_stream(parents), want), case["name"]
        assert np.array_equal(S.Schedule().load(parents).ref_serial_stream(), want), case["name"]


@pytest.mark.skipif(oracle.refsched_lib() is None, reason="reference scheduler was not compiled on this machine")
def test_reference_scheduler_agrees_on_random_graphs():
    for seed in range(150):
        parents = _random_graph(seed)
        ref = oracle.ref_schedule_stream(parents)
        assert np.array_equal(oracle.schedule_stream(parents), ref), seed
        assert np.array_equal(S.Schedule().load(parents).ref_stream(), ref), seed
        ref = oracle.ref_serial_stream(parents)
        assert np.array_equal(oracle.serial_stream(parents), ref), seed
        assert np.array_equal(S.Schedule().load(parents).ref_serial_stream(), ref), seed


def test_tables_match_oracle_both_modes():
    for seed in range(60):
        parents = _random_graph(seed)
        s = S.Schedule().load(parents)
        for mode in (S.ALIGNED, S.REF_COMPAT):
            t = oracle.tables(parents, 2, mode)
            fg, fs, bg, bs = s.tables(mode)
            assert np.array_equal(t["fg"], fg) and np.array_equal(t["bs"], bs)
            assert np.array_equal(t["fs"], fs) and np.array_equal(t["bg"], bg)
            assert np.array_equal(t["level_off"], s.level_off)
            t2j, j2t = s.maps()
            assert np.array_equal(t["t2j"], t2j) and np.array_equal(t["j2t"], j2t)


def test_ref_compat_differs_from_aligned_only_on_skewed_batches():
    # Tree A (2 leaves) + tree B (3 leaves): level 1 holds A's root and B's inner vertex, and the
    # reference's scatter list for that level has one entry -> rows shift (the reference's
    # "we loose this constraint" comments, op_impl_graphop.cu:57-61,140-143).
    parents = np.array([[2, 2, -1, -1, -1], [3, 3, 4, 4, -1]], np.int32)
    s = S.Schedule().load(parents)
    a = s.tables(S.ALIGNED)
    r = s.tables(S.REF_COMPAT)
    assert not np.array_equal(a[1], r[1])
    # Equal-shape batch: identical.
    parents = np.array([[2, 2, -1], [2, 2, -1]], np.int32)
    s = S.Schedule().load(parents)
    for x, y in zip(s.tables(S.ALIGNED), s.tables(S.REF_COMPAT)):
        assert np.array_equal(x, y)


def test_n_ary_tables_extension():
    parents, _ = S.synth_trees(5, 16, 2, 20, max_arity=4)
    s = S.Schedule().load(parents, n_slots=4)
    t = oracle.tables(parents, 4, 0)
    fg, fs, bg, bs = s.tables(0)
    assert np.array_equal(t["fg"], fg) and np.array_equal(t["fs"], fs)
    # every non-root is gathered exactly once
    gathered = fg[fg >= 0]
    assert len(np.unique(gathered)) == len(gathered) == s.n_total - parents.shape[0]


def test_unbatched_order_runs_one_vertex_per_round():
    # The execution order of the serial scheduler as a schedule the engines can run: tensor ids follow
    # execution, every level holds one row, the tables stay consistent with the batched ones.
    for seed in range(40):
        parents = _random_graph(seed)
        s = S.Schedule().set_order(S.UNBATCHED).load(parents)
        b = S.Schedule().load(parents)
        assert s.n_scheduled == b.n_scheduled and s.n_levels == s.n_scheduled
        assert np.array_equal(s.level_off, np.arange(s.n_scheduled + 1))
        t2j, j2t = s.maps()
        fg, fs, bg, bs = s.tables(0)
        bt2j, bj2t = b.maps()
        bfg = b.tables(0)[0]
        n = s.n_scheduled
        for c in range(2):
            m = fg[c][:n] >= 0
            assert (fg[c][:n][m] < np.arange(n)[m]).all()              # children run strictly earlier
            # same children, job for job
            want = np.where(bfg[c][bj2t[t2j[:n]]] >= 0, bt2j[np.maximum(bfg[c][bj2t[t2j[:n]]], 0)], -1)
            got = np.where(fg[c][:n] >= 0, t2j[np.maximum(fg[c][:n], 0)], -1)
            assert np.array_equal(want, got)
        # without single-vertex samples the order is the reference's serial forward sweep
        lens = [list(row).index(-1) + 1 for row in parents]
        if 1 not in lens:
            assert np.array_equal(t2j[:n], s.serial_rounds()[0])
        # samples run one after another
        sample_of = np.searchsorted(np.cumsum(lens), t2j[:n], side="right")
        assert (np.diff(sample_of) >= 0).all()
        parent, child = s.adjacency()
        assert ((parent >= 0).sum() == s.n_total - len(lens)) and child.shape == (2, s.n_total)


def test_level_properties_full_size():
    # config-5-sized shard (512 trees, leaves in [2,128]): size-independent invariants.
    parents, _ = S.synth_trees(123, 512, 2, 128)
    s = S.Schedule().load(parents)
    fg, fs, bg, bs = s.tables(0)
    lo = s.level_off
    level_of = np.repeat(np.arange(s.n_levels), np.diff(lo))
    for c in range(2):
        m = fg[c] >= 0
        assert (level_of[fg[c][m]] < level_of[m]).all()          # children execute strictly earlier
    assert (fg[:, :lo[1]] == -1).all()                            # level 0 = leaves
    t2j, j2t = s.maps()
    assert np.array_equal(np.sort(t2j), np.arange(s.n_total))     # a permutation
    assert np.array_equal(j2t[t2j], np.arange(s.n_total))
    assert (fs >= 0).sum() == s.n_total - 512                     # every non-root scatters once


def test_edge_cases():
    # single-vertex samples never execute (graph_scheduler.cc:180)
    s = S.Schedule().load(np.array([[-1, -1], [1, -1]], np.int32))
    assert (s.n_total, s.n_scheduled, s.n_levels) == (3, 2, 2)
    # empty batch
    s = S.Schedule().load(np.zeros((0, 4), np.int32))
    assert (s.n_total, s.n_levels) == (0, 0)
    # chain of length 2
    s = S.Schedule().load(np.array([[1, -1]], np.int32), n_slots=1)
    assert s.level_off.tolist() == [0, 1, 2]


@pytest.mark.parametrize("parents,why", [
    ([[1, 2, 0, 5]], "no terminator"),
    ([[7, -1, -1]], "parent out of range"),
    ([[0, -1, -1]], "self parent"),
    ([[3, 3, 3, -1]], "three children in two slots"),
    ([[1, 0, 3, -1]], "cycle"),
])
def test_malformed_graphs_return_bad_graph(parents, why):
    with pytest.raises(CavsError) as e:
        S.Schedule().load(np.array(parents, np.int32))
    assert e.value.status == 2, why
