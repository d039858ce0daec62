"""Host-side level scheduler and synthetic workloads (thin wrappers over the C ABI)."""
from __future__ import annotations

import ctypes

import numpy as np

from ._abi import check, lib, ptr

ALIGNED, REF_COMPAT = 0, 1
BATCHED, UNBATCHED = 0, 1


class Schedule:
    """One batch's level schedule.  Mirrors what the reference's graph ops read from
    GraphSchedulerBase (cavs/midend/graph_scheduler.h:20-77), computed for all levels at once."""

    def __init__(self):
        self._h = ctypes.c_void_p()
        check(lib().cavs_sched_create(ctypes.byref(self._h)))
        self.n_total = self.n_scheduled = self.n_levels = self.max_level_rows = 0
        self.n_slots = 2

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and lib is not None:  # `lib` is cleared during interpreter shutdown
            try:
                lib().cavs_sched_destroy(h)
            except Exception:
                pass

    def set_order(self, order: int) -> "Schedule":
        """Round order of the next load(): BATCHED (one round per level) or UNBATCHED (one vertex per
        round, the reference's serial scheduling, cavs/midend/graph_scheduler.cc:83-167)."""
        check(lib().cavs_sched_set_order(self._h, order))
        return self

    def load(self, parents: np.ndarray, n_slots: int = 2) -> "Schedule":
        parents = np.ascontiguousarray(parents, dtype=np.int32)
        assert parents.ndim == 2
        check(lib().cavs_sched_load(self._h, ptr(parents), parents.shape[0], parents.shape[1], n_slots))
        self.n_slots = n_slots
        return self._refresh()

    def _refresh(self) -> "Schedule":
        """Re-reads the counts after the handle was loaded by another entry point (cavs_treelstm_stage)."""
        a, b, c, d = (ctypes.c_int() for _ in range(4))
        check(lib().cavs_sched_counts(self._h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), ctypes.byref(d)))
        self.n_total, self.n_scheduled, self.n_levels, self.max_level_rows = a.value, b.value, c.value, d.value
        return self

    @property
    def level_off(self) -> np.ndarray:
        out = np.empty(self.n_levels + 1, np.int32)
        check(lib().cavs_sched_level_offsets(self._h, ptr(out), out.size))
        return out

    def maps(self):
        t2j = np.empty(self.n_total, np.int32)
        j2t = np.empty(self.n_total, np.int32)
        check(lib().cavs_sched_maps(self._h, ptr(t2j), ptr(j2t), self.n_total))
        return t2j, j2t

    def tables(self, mode: int = ALIGNED):
        n, k = self.n_total, self.n_slots
        fg = np.empty((k, n), np.int32)
        bs = np.empty((k, n), np.int32)
        fs = np.empty(n, np.int32)
        bg = np.empty(n, np.int32)
        check(lib().cavs_sched_tables(self._h, mode, ptr(fg), ptr(fs), ptr(bg), ptr(bs), n))
        return fg, fs, bg, bs

    def ref_gather(self, level: int, slot: int) -> np.ndarray:
        out = np.empty(max(self.max_level_rows, 1), np.int32)
        n = ctypes.c_int()
        check(lib().cavs_sched_ref_gather(self._h, level, slot, ptr(out), out.size, ctypes.byref(n)))
        return out[: n.value].copy()

    def ref_scatter(self, level: int) -> np.ndarray:
        out = np.empty(max(self.max_level_rows, 1), np.int32)
        n = ctypes.c_int()
        check(lib().cavs_sched_ref_scatter(self._h, level, ptr(out), out.size, ctypes.byref(n)))
        return out[: n.value].copy()

    def ref_stream(self) -> np.ndarray:
        cap = 16 + 12 * max(self.n_total, 1) + 16 * max(self.n_levels, 1) + self.n_levels * (self.level_off[1] if self.n_levels else 0) \
            + self.n_levels * self.n_total
        out = np.empty(min(cap, 2**31 - 1), np.int32)
        n = ctypes.c_int()
        check(lib().cavs_sched_ref_stream(self._h, ptr(out), out.size, ctypes.byref(n)))
        return out[: n.value].copy()


    def adjacency(self):
        """(parent_job [N], child_job [slots, N]) in job-id space."""
        n, k = self.n_total, self.n_slots
        parent = np.empty(n, np.int32)
        child = np.empty((k, n), np.int32)
        check(lib().cavs_sched_adjacency(self._h, ptr(parent), ptr(child), n))
        return parent, child

    def serial_rounds(self, backward: bool = False):
        """Job ids in the order the reference's SerialGraphScheduler runs them, and per round the
        entry of its gather-initialisation list (-1 = empty)."""
        jobs = np.empty(max(self.n_total, 1), np.int32)
        init = np.empty(max(self.n_total, 1), np.int32)
        n = ctypes.c_int()
        check(lib().cavs_sched_serial_rounds(self._h, int(backward), ptr(jobs), ptr(init), jobs.size, ctypes.byref(n)))
        return jobs[: n.value].copy(), init[: n.value].copy()

    def ref_serial_stream(self) -> np.ndarray:
        out = np.empty(16 + 24 * max(self.n_total, 1), np.int32)
        n = ctypes.c_int()
        check(lib().cavs_sched_ref_serial_stream(self._h, ptr(out), out.size, ctypes.byref(n)))
        return out[: n.value].copy()


def synth_trees(seed: int, batch: int, leaf_lo: int, leaf_hi: int, max_arity: int = 2, max_len: int | None = None):
    if max_len is None:
        max_len = 2 * leaf_hi - 1 if max_arity == 2 else 4 * leaf_hi - 2
    parents = np.empty((batch, max_len), np.int32)
    is_leaf = np.empty((batch, max_len), np.uint8)
    check(lib().cavs_synth_trees(ctypes.c_uint64(seed), batch, leaf_lo, leaf_hi, max_arity, max_len, ptr(parents), ptr(is_leaf)))
    return parents, is_leaf


def synth_chains(seed: int, batch: int, len_lo: int, len_hi: int, max_len: int | None = None):
    max_len = max_len or len_hi
    parents = np.empty((batch, max_len), np.int32)
    check(lib().cavs_synth_chains(ctypes.c_uint64(seed), batch, len_lo, len_hi, max_len, ptr(parents)))
    return parents


def synth_zipf(seed: int, s: float, vocab: int, count: int) -> np.ndarray:
    out = np.empty(count, np.int32)
    check(lib().cavs_synth_zipf(ctypes.c_uint64(seed), ctypes.c_double(s), vocab, ptr(out), ctypes.c_size_t(count)))
    return out


def synth_uniform_int(seed: int, bound: int, count: int) -> np.ndarray:
    out = np.empty(count, np.int32)
    check(lib().cavs_synth_uniform_int(ctypes.c_uint64(seed), bound, ptr(out), ctypes.c_size_t(count)))
    return out


def synth_uniform_float(seed: int, scale: float, shape) -> np.ndarray:
    out = np.empty(shape, np.float32)
    check(lib().cavs_synth_uniform_float(ctypes.c_uint64(seed), ctypes.c_float(scale), ptr(out), ctypes.c_size_t(out.size)))
    return out
