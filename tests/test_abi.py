"""The C ABI library loads and exports every entry point include/cavs_b200.h declares
(no device work here), and host-side argument checks return error codes."""
import ctypes

import numpy as np

import cavs_b200
from cavs_b200 import lib
from cavs_b200 import schedule as S


def test_every_declared_symbol_is_exported():
    L = lib()
    names = cavs_b200.declared_symbols()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_build_info_names_the_architecture():
    assert b"sm_100a" in lib().cavs_build_info()


def test_status_strings():
    L = lib()
    assert L.cavs_status_string(0) == b"ok"
    assert L.cavs_status_string(2) == b"malformed graph"


def test_synthetic_generators_are_deterministic_and_in_range():
    a, leaf = S.synth_trees(1, 8, 2, 50)
    b, _ = S.synth_trees(1, 8, 2, 50)
    assert np.array_equal(a, b)
    lens = (a == -1).argmax(1) + 1
    n_leaf = np.array([leaf[i, :lens[i]].sum() for i in range(8)])
    assert ((n_leaf >= 2) & (n_leaf <= 50)).all() and (lens == 2 * n_leaf - 1).all()
    z = S.synth_zipf(3, 1.1, 21701, 20000)
    assert z.min() >= 0 and z.max() < 21701 and (z == 0).mean() > 0.05   # head-heavy
    f = S.synth_uniform_float(4, 0.05, (1000,))
    assert np.abs(f).max() <= 0.05 and abs(f.mean()) < 0.01
    c = S.synth_chains(5, 16, 10, 100)
    cl = (c == -1).argmax(1) + 1
    assert ((cl >= 10) & (cl <= 100)).all()
    p4, _ = S.synth_trees(6, 8, 8, 128, max_arity=4)
    S.Schedule().load(p4, n_slots=4)


def test_engine_rejects_bad_configs_without_a_gpu():
    L = lib()
    L.cavs_treelstm_workspace_bytes.restype = ctypes.c_size_t
    from cavs_b200.treelstm import Config
    bad = Config(150, 300, 100, 5, 2, 1, 1000, 1000)      # bf16 path needs multiples of 8
    assert L.cavs_treelstm_workspace_bytes(ctypes.byref(bad)) == 0
    assert b"multiples of 8" in L.cavs_last_error()
    ok = Config(150, 300, 100, 5, 2, 0, 1000, 1000)
    assert L.cavs_treelstm_workspace_bytes(ctypes.byref(ok)) > 0
