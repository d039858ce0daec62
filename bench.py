#!/usr/bin/env python
"""Benchmark of the level-batched Tree-LSTM training step (forward + backward + update).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default "dp_treelstm"): global batch of 4096 random binary trees, leaves uniform in
[2,128], hidden 1024, embedding 1024, vocabulary 50000 with Zipf(1.1) leaf tokens, 5-class loss on
every vertex, bf16 gate GEMMs with fp32 accumulation and fp32 cell maths, Adagrad(lr=0.05).  The
global batch is split evenly by tree across the ranks (strong scaling); gradients are summed with
one NCCL all-reduce per step.  Inputs are seeded synthetic stand-ins for the SST / PTB files the
reference's apps read (those are not distributed with it).

Prints ONE JSON line on rank 0.  `value` times steps whose index tables are already resident in
HBM; `e2e` times the whole public-API step from host arrays: host level scheduling, one pinned
host-to-device upload, forward, backward, all-reduce, update and the device-to-host read of the
loss.  `--impl reference` times the CPU oracle (the reference has no CPU implementation of this
path and its CUDA-8 sources do not build here) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (global_batch, leaf_lo, leaf_hi, hidden, embed, vocab, classes, bf16)
    "dp_treelstm": dict(batch=4096, leaf_lo=2, leaf_hi=128, hidden=1024, embed=1024, vocab=50000, classes=5, bf16=True,
                        init_scale=0.05, lr=0.05),
    "sst_treelstm": dict(batch=64, leaf_lo=2, leaf_hi=50, hidden=150, embed=300, vocab=21701, classes=5, bf16=False,
                         init_scale=0.05, lr=0.05),
}
# The other configurations: launch-latency-bound at their sizes (tens of levels of a few hundred rows), so their line
# carries the measured latency floor -- the same engine stepped on a batch with the same number of levels and one
# or two vertices per level -- beside the achieved step time.  One GPU only.
SMALL_WORKLOADS = {
    "chain_lm": dict(kind="chain", batch=20, len_lo=20, len_hi=20, hidden=200, embed=200, vocab=10000, layers=1, bf16=False,
                     init_scale=0.1, optimizer="sgd", lr=1.0, unit="sequences/s"),
    "ragged_chain_2layer": dict(kind="chain", batch=256, len_lo=10, len_hi=100, hidden=512, embed=512, vocab=10000, layers=2, bf16=False,
                                init_scale=0.05, optimizer=None, lr=0.0, unit="sequences/s"),
    "nary_treegru": dict(kind="gru", batch=512, leaf_lo=8, leaf_hi=128, arity=4, hidden=1024, embed=512, vocab=32000, classes=2, bf16=True,
                         init_scale=0.05, optimizer=None, lr=0.0, unit="trees/s"),
}
POOL = 16            # distinct pre-generated batches cycled through by the end-to-end loop
SEED = 0xC0FFEE00


def make_batch(wl, idx, rank, world, with_rows=False):
    """Global batch `idx`, then this rank's shard of it.  Returns (parents, tok_job, label_job, global_vertices) and, with
    `with_rows`, the distinct token ids of the GLOBAL batch in ascending order: the embedding rows any rank touches, which
    every rank's loader knows because it reads the global batch's ids before it takes its shard."""
    from cavs_b200 import schedule as S
    b = wl["batch"]
    parents, is_leaf = S.synth_trees(SEED + 16 * 5 + 1000 * idx, b, wl["leaf_lo"], wl["leaf_hi"])
    lens = (parents == -1).argmax(1) + 1
    tok_pad = S.synth_zipf(SEED + 16 * 5 + 1000 * idx + 1, 1.1, wl["vocab"], parents.size).reshape(parents.shape) * is_leaf
    lab_pad = S.synth_uniform_int(SEED + 16 * 5 + 1000 * idx + 2, wl["classes"], parents.size).reshape(parents.shape)
    per = b // world
    lo, hi = rank * per, (rank + 1) * per
    mask = np.arange(parents.shape[1])[None, :] < lens[lo:hi, None]
    tok_job = np.ascontiguousarray(tok_pad[lo:hi][mask], np.int32)
    label_job = np.ascontiguousarray(lab_pad[lo:hi][mask], np.int32)
    out = (np.ascontiguousarray(parents[lo:hi]), tok_job, label_job, int(lens.sum()))
    if with_rows:
        all_mask = np.arange(parents.shape[1])[None, :] < lens[:, None]
        seen = np.bincount(tok_pad[all_mask].astype(np.int64), minlength=wl["vocab"])
        out += (np.flatnonzero(seen).astype(np.int32),)
    return out


def make_params(wl):
    from cavs_b200 import schedule as S
    H, E, V, C, sc = wl["hidden"], wl["embed"], wl["vocab"], wl["classes"], wl["init_scale"]
    base = SEED + 16 * 5 + 3
    return dict(Emb=S.synth_uniform_float(base, sc, (V, E)), W=S.synth_uniform_float(base + 100, sc, (E * 4 * H,)),
                U=S.synth_uniform_float(base + 200, sc, (4 * H * H,)), B=np.zeros(4 * H, np.float32),
                Wc=S.synth_uniform_float(base + 300, sc, (C, H)), bc=np.zeros(C, np.float32))


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.path = gpu_index, None, f"/tmp/cavs_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for line in Path(self.path).read_text().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(smax), reasons=sorted(reasons), samples=len(sm))
        try:
            os.unlink(self.path)
        except OSError:
            pass
        return out


def gemm_dram_bytes_per_internal_row():
    """DRAM bytes all GEMM launches of a step move per internal vertex, from the committed figures of a profiler capture
    (one rank's shard at 8 GPUs); None if the record is missing."""
    rec = ROOT / "profiles" / "gemm_dram_traffic_shard_512_trees.json"
    if not rec.exists():
        return None
    d = json.loads(rec.read_text())
    return d["dram_bytes_per_step"] / d["internal_vertices"]



def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


def numpy_sample(wl, n_trees, seed=SEED):
    """A sample of the workload generated with numpy alone (the CPU arm does not load the product library): random
    binary trees by recursive uniform split, vertices in post-order (root last), Zipf(1.1) leaf tokens by inverse-CDF
    lookup, token 0 on internal vertices, uniform labels; weights uniform in +-init_scale, zero biases."""
    rng = np.random.default_rng(seed)
    max_len = 2 * wl["leaf_hi"] - 1
    parents = np.full((n_trees, max_len), -1, np.int32)
    toks, labs = [], []
    ranks = np.arange(1, wl["vocab"] + 1, dtype=np.float64) ** -1.1
    cdf = np.cumsum(ranks) / ranks.sum()
    for b in range(n_trees):
        par, leaf = [], []

        def rec(leaves):
            if leaves == 1:
                par.append(-1); leaf.append(True)
                return len(par) - 1
            split = int(rng.integers(1, leaves))
            left, right = rec(split), rec(leaves - split)
            par.append(-1); leaf.append(False)
            par[left] = par[right] = len(par) - 1
            return len(par) - 1

        rec(int(rng.integers(wl["leaf_lo"], wl["leaf_hi"] + 1)))
        parents[b, :len(par)] = par
        is_leaf = np.array(leaf)
        tok = np.minimum(np.searchsorted(cdf, rng.random(len(par))), wl["vocab"] - 1)
        toks.append(np.where(is_leaf, tok, 0).astype(np.int32))
        labs.append(rng.integers(0, wl["classes"], len(par)).astype(np.int32))
    H, E, V, C, sc = wl["hidden"], wl["embed"], wl["vocab"], wl["classes"], wl["init_scale"]
    u = lambda *shape: rng.uniform(-sc, sc, shape).astype(np.float32)
    params = dict(Emb=u(V, E), W=u(E * 4 * H), U=u(4 * H * H), B=np.zeros(4 * H, np.float32), Wc=u(C, H), bc=np.zeros(C, np.float32))
    return parents, np.concatenate(toks), np.concatenate(labs), params


_cpu_state = {}


def cpu_baseline_sample(wl, n_trees):
    """One training step (level scheduling, forward, loss, backward, Adagrad) of the CPU oracle on a numpy-generated
    sample of n_trees trees.  Returns (trees/s, seconds, executed GEMM GFLOP/s).  Nothing of the product runs here:
    tables come from the oracle's own scheduler restatement."""
    import oracle
    H, E, V, C = wl["hidden"], wl["embed"], wl["vocab"], wl["classes"]
    key = (id(wl), n_trees)
    if key not in _cpu_state:
        parents, tok_job, label_job, params = numpy_sample(wl, n_trees)
        _cpu_state.clear()
        _cpu_state[key] = (parents, tok_job, label_job, params, {k: np.zeros_like(v) for k, v in params.items()})
    parents, tok_job, label_job, flat, acc = _cpu_state[key]
    t0 = time.perf_counter()
    tb = oracle.tables(parents, 2, 0)
    out = oracle.treelstm_fwd_bwd(tb, tok_job[tb["t2j"]], label_job[tb["t2j"]], flat, H, E, V, C, gemm_bf16=wl["bf16"])
    for k in flat:
        oracle.adagrad(flat[k].reshape(-1), acc[k].reshape(-1), out["d" + k].reshape(-1), wl["lr"])
    dt = time.perf_counter() - t0
    n, n_int = int(tb["n"]), int(tb["n"] - tb["level_off"][1])
    flops = 3.0 * (2.0 * n * E * 4 * H + n_int * (2.0 * H * 3 * H + 4.0 * H * H))    # the per-vertex form the oracle executes
    return n_trees / dt, dt, flops / dt / 1e9


def run_reference(args, wl, rank, world):
    """The reference arm: the oracle port on the host cores (rank 0 only)."""
    if rank != 0:
        return
    # torchrun pins every rank to one OpenMP thread; this arm is the only work on the host, so it takes all cores.
    if os.environ.get("OMP_NUM_THREADS") == "1" and world > 1:
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    import oracle
    oracle.oracle_lib()
    # One untimed step on a small sample warms the thread pool and measures the host; the timed steps then use the
    # largest sample (at most --sample-trees) that keeps the whole run within about two minutes.
    probe = min(32, args.sample_trees)
    rate = cpu_baseline_sample(wl, probe)[0]
    n_trees = int(max(probe, min(args.sample_trees, rate * 120.0 / max(args.steps, 1))))
    t0 = time.perf_counter()
    gflops = [cpu_baseline_sample(wl, n_trees)[2] for _ in range(args.steps)]
    total = time.perf_counter() - t0
    value = n_trees * args.steps / total
    line = dict(metric="treelstm_train_trees_per_sec", value=value, unit="trees/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1e3 * total / args.steps, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="bf16" if wl["bf16"] else "f32", data="synthetic", impl="reference",
                config=dict(workload=args.workload, global_batch=wl["batch"], hidden=wl["hidden"], embed=wl["embed"],
                            vocab=wl["vocab"], classes=wl["classes"], leaves=[wl["leaf_lo"], wl["leaf_hi"]]),
                cpu_baseline=dict(value=value, unit="trees/s", cores=oracle.num_threads(), kind="port",
                                  gemm_gflops=statistics.median(gflops),
                                  sample=f"{n_trees} trees per step (numpy-generated sample of the workload), level scheduling + "
                                         "fwd + bwd + Adagrad, OpenMP over rows, cache-blocked GEMMs"),
                e2e=dict(value=value, unit="trees/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                note="the reference has no CPU implementation of this path and its CUDA 8 sources do not build here; "
                     "this arm times the CPU oracle port (oracle/cavs_oracle.c) and loads nothing of the product. "
                     "A step of the sample pays the per-step fixed costs (dense embedding-gradient block, full-table "
                     "Adagrad) for fewer trees than a full batch would: trees/s understates the CPU at full batch size "
                     "by the share of those costs; gemm_gflops is the size-independent figure")
    print(json.dumps(line))


def run_small_workload(args, name, wl):
    """Chain LM, two stacked ragged-chain layers, N-ary Tree-GRU: step time, end-to-end time and latency floor on one GPU."""
    import torch
    from cavs_b200 import lib, schedule as S
    from cavs_b200.treegru import TreeGRU
    from cavs_b200.treelstm import TreeLSTM
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(0)
    L = lib()
    L.cavs_launch_count.restype = ctypes.c_ulonglong
    H, E, V, B = wl["hidden"], wl["embed"], wl["vocab"], wl["batch"]
    K = 1 if wl["kind"] == "chain" else wl["arity"]
    pool_n = 8

    def make(idx):
        seed = SEED + 977 * (idx + 1) + (hash(name) & 0xffff)
        if wl["kind"] == "chain":
            parents = S.synth_chains(seed, B, wl["len_lo"], wl["len_hi"])
            lens = (parents == -1).argmax(1) + 1
            n = int(lens.sum())
            tok = S.synth_zipf(seed + 1, 1.1, V, n)
            lab = np.empty(n, np.int32)           # next token; the last position predicts token 0
            off = 0
            for ln in lens:
                lab[off:off + ln - 1] = tok[off + 1:off + ln]; lab[off + ln - 1] = 0; off += ln
            return parents, tok, lab, n
        parents, is_leaf = S.synth_trees(seed, B, wl["leaf_lo"], wl["leaf_hi"], wl["arity"])
        lens = (parents == -1).argmax(1) + 1
        n = int(lens.sum())
        mask = np.arange(parents.shape[1])[None, :] < lens[:, None]
        tok = (S.synth_zipf(seed + 1, 1.1, V, parents.size).reshape(parents.shape) * is_leaf)[mask].astype(np.int32)
        lab = np.full(n, -1, np.int32)            # root-only loss: the root is each sample's last vertex
        lab[np.cumsum(lens) - 1] = S.synth_uniform_int(seed + 2, wl["classes"], B)
        return parents, tok, lab, n

    pool = [make(i) for i in range(pool_n)]
    scheds = [S.Schedule().load(p[0], n_slots=K) for p in pool]
    levels = max(s.n_levels for s in scheds)
    # the floor batch: one sample with as many levels as the deepest batch (a chain, or a tree whose internal vertices
    # each have one leaf child and one internal child)
    if K == 1:
        floor_parents = np.full((1, levels), -1, np.int32); floor_parents[0, :levels - 1] = np.arange(1, levels)
    else:
        m = 2 * levels - 1                        # leaf, leaf, parent, leaf, parent, ... in post-order
        floor_parents = np.full((1, m), -1, np.int32)
        floor_parents[0, 0] = floor_parents[0, 1] = 2
        for v in range(2, m - 1, 2):
            floor_parents[0, v] = v + 2; floor_parents[0, v + 1] = v + 2
    floor_sched = S.Schedule().load(floor_parents, n_slots=K)
    max_n = max(max(s.n_total for s in scheds), floor_sched.n_total)
    max_rows = max(s.max_level_rows for s in scheds)
    sc = wl["init_scale"]
    u = lambda seed, *shape: S.synth_uniform_float(SEED + seed, sc, shape)
    cap = dict(n_slots=K, gemm_bf16=wl["bf16"], max_vertices=max_n, max_level_rows=max_rows)
    if wl["kind"] == "gru":
        C = wl["classes"]
        engines = [TreeGRU(H, E, V, C, **cap)]
        engines[0].set_params(dict(Emb=u(1, V, E), W=u(2, E * 3 * H), U=u(3, 3 * H * H), B=np.zeros(3 * H, np.float32), Wc=u(4, C, H),
                                   bc=np.zeros(C, np.float32)))
    else:
        C = V
        n_layers = wl["layers"]
        engines = []
        for li in range(n_layers):
            eng = TreeLSTM(H, E if li == 0 else H, V if li == 0 else 0, C if li == n_layers - 1 else 0, **cap)
            Ei = E if li == 0 else H
            eng.set_params(dict(Emb=u(10 * li + 1, V, E) if li == 0 else np.zeros(0, np.float32), W=u(10 * li + 2, Ei * 4 * H),
                                U=u(10 * li + 3, 4 * H * H), B=np.zeros(4 * H, np.float32),
                                Wc=u(10 * li + 4, C, H) if li == n_layers - 1 else np.zeros(0, np.float32),
                                bc=np.zeros(C if li == n_layers - 1 else 0, np.float32)))
            engines.append(eng)

    def load(sched, tok, lab, rows):
        for li, eng in enumerate(engines):
            if wl["kind"] == "gru":
                eng.load_batch(sched, tok, lab, loss_rows=rows)
            else:
                eng.load_batch(sched, tok if li == 0 else None, lab if li == len(engines) - 1 else None, loss_rows=rows)

    def step(n_rows):
        if wl["kind"] == "gru":
            engines[0].forward(); engines[0].backward()
            return
        for li, eng in enumerate(engines):       # bottom-up: a layer's h columns feed the next layer
            if li > 0:
                below = engines[li - 1]
                eng.set_dense_input(below.device_view(0, (n_rows, 2 * H))[:, :H])
            eng.forward()
        for li in range(len(engines) - 1, -1, -1):   # top-down: a layer's d(x) is the output gradient of the layer below
            eng = engines[li]
            if li < len(engines) - 1:
                eng.set_output_grad(engines[li + 1].device_view(5, (n_rows, H)))
            eng.backward()
        if wl["optimizer"] == "sgd":
            for eng in engines:
                eng.sgd(wl["lr"])

    def timed_steps(k, n_rows):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        l0 = L.cavs_launch_count()
        a.record()
        for _ in range(k):
            step(n_rows)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / k, (L.cavs_launch_count() - l0) // k

    warm = max(args.warmup, 3)
    # latency floor: same engines, same level count, one or two vertices per level
    n_floor = floor_sched.n_total
    load(floor_sched, np.zeros(n_floor, np.int32), np.zeros(n_floor, np.int32), n_floor)
    for _ in range(warm):
        step(n_floor)
    floor_ms, floor_launches = timed_steps(args.steps, n_floor)
    # device-resident arm (tables of batch 0 in HBM)
    load(scheds[0], pool[0][1], pool[0][2], B if wl["kind"] == "gru" else pool[0][3])
    for _ in range(warm):
        step(scheds[0].n_total)
    sampler = ClockSampler(0)
    sampler.start()
    ms_dev, launches = timed_steps(args.steps, scheds[0].n_total)
    loss_dev = engines[-1].read_loss()
    # end-to-end arm: host scheduling, table upload, step and loss read-back for every batch of the pool
    host = S.Schedule()

    def e2e(k):
        for i in range(k):
            par, tok, lab, n = pool[i % pool_n]
            host.load(par, n_slots=K)
            load(host, tok, lab, B if wl["kind"] == "gru" else n)
            step(host.n_total)
            engines[-1].read_loss()
    e2e(warm)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e(args.steps)
    torch.cuda.synchronize()
    ms_e2e = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop()
    up = engines[0].upload_bytes() if wl["kind"] != "gru" else 0
    n_v = int(scheds[0].n_total)
    line = dict(metric=f"{name}_train_{wl['unit'].split('/')[0]}_per_sec", value=B / (ms_dev * 1e-3), unit=wl["unit"], n_gpus=1, steps=args.steps,
                warmup=warm, ms_per_step=ms_dev, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="bf16" if wl["bf16"] else "f32", data="synthetic",
                config=dict(workload=name, batch=B, hidden=H, embed=E, vocab=V, layers=wl.get("layers", 1), child_slots=K,
                            vertices=n_v, levels=int(scheds[0].n_levels), optimizer=wl["optimizer"] or "none (forward + backward)",
                            l2="per-step working set below L2: the step is bound by its dependent launches, see latency_floor"),
                e2e=dict(value=B / (ms_e2e * 1e-3), unit=wl["unit"], ms_per_step=ms_e2e, h2d_bytes_per_step=int(up), d2h_bytes_per_step=8),
                gpu_launches=int(launches) * args.steps, gpu_launches_per_step=int(launches), loss_sum=loss_dev, clocks=clocks,
                latency_floor=dict(ms_per_step=floor_ms, launches_per_step=int(floor_launches), levels=int(levels),
                                   us_per_level=1e3 * floor_ms / max(levels, 1), frac_of_step=floor_ms / ms_dev,
                                   note="the same engines stepped on one sample with the same number of levels and one or two "
                                        "vertices per level: what the level loop costs before any data moves"),
                roofline=dict(bound="latency", achieved=ms_dev, peak=floor_ms, unit="ms per step (achieved) vs measured latency floor",
                              frac=floor_ms / ms_dev, traffic=None))
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dp_treelstm", choices=sorted(WORKLOADS) + sorted(SMALL_WORKLOADS))
    ap.add_argument("--sample-trees", type=int, default=256, help="trees per CPU-baseline step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--dense-exchange", action="store_true",
                    help="data parallel: all-reduce the whole embedding-gradient block instead of the rows the global batch touches")
    args = ap.parse_args()
    if args.workload in SMALL_WORKLOADS:
        if int(os.environ.get("RANK", "0")) == 0:
            run_small_workload(args, args.workload, SMALL_WORKLOADS[args.workload])
        return
    wl = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, wl, rank, world)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from cavs_b200 import lib, schedule as S
    from cavs_b200.treelstm import TreeLSTM
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    assert wl["batch"] % world == 0

    L = lib()
    L.cavs_launch_count.restype = ctypes.c_ulonglong

    def lib_check(rc):
        if rc != 0:
            raise RuntimeError(L.cavs_last_error().decode())
    # The embedding gradient is kept, exchanged between the ranks and applied for the rows the global batch touches, not
    # for the whole table (at one GPU there is no exchange, but the same compact block and row update).
    sparse = not args.dense_exchange
    pool = [make_batch(wl, i, rank, world, with_rows=True) for i in range(POOL)]
    xrows = [p[4] if sparse else None for p in pool]
    scheds = [S.Schedule().load(p[0]) for p in pool]
    max_n = max(s.n_total for s in scheds)
    max_rows = max(s.max_level_rows for s in scheds)
    eng = TreeLSTM(wl["hidden"], wl["embed"], wl["vocab"], wl["classes"], gemm_bf16=wl["bf16"], max_vertices=max_n,
                   max_level_rows=max_rows, device=dev)
    eng.set_params(make_params(wl))
    acc = torch.zeros_like(eng.params)
    pinned = [tuple(torch.from_numpy(a).pin_memory() for a in p[:3]) for p in pool]
    host_sched = S.Schedule()

    # The library's own communicator (NCCL from C++); torch.distributed only carries its 128-byte id to the ranks
    # and the benchmark's barriers.
    comm = None
    if world > 1:
        from cavs_b200.comm import Comm
        comm = Comm.from_torch()

    def device_step():
        # forward, backward, gradient sum over the ranks (embedding block on a side stream under the weight-gradient
        # products), Adagrad, refresh of the bf16 weights: one call into the library
        eng.step(comm, eng.OPT_ADAGRAD, acc, wl["lr"])

    host_ms = [0.0, 0]   # host scheduling + packing + upload-enqueue ms, calls

    pinned_np = [tuple(t.numpy() for t in p) for p in pinned]

    # Host pipeline of the end-to-end loop, three stations: level scheduling of batch i+2 on a thread of this script
    # (cavs_sched_load releases the interpreter lock), table packing + upload of batch i+1 on the engine's helper thread,
    # enqueueing of step i on this thread.  Two schedule objects alternate: the one being packed from is not written.
    from concurrent.futures import ThreadPoolExecutor
    sched_pool = ThreadPoolExecutor(max_workers=1)
    host_scheds = [host_sched, S.Schedule()]
    sched_job = {}

    def schedule_ahead(i):
        sched_job[i] = sched_pool.submit(host_scheds[i % 2].load, pinned_np[i % POOL][0])

    def stage(i):
        """Packing and pinned upload of batch i's tables on the engine's helper thread, from the schedule the scheduling
        thread has finished (started one step earlier); then batch i+1's scheduling starts.  Both run beside this
        thread's enqueueing of the step in flight."""
        par, tok, lab = pinned_np[i % POOL]
        t0 = time.perf_counter()
        if i not in sched_job:
            schedule_ahead(i)
        sched_job.pop(i).result()
        eng.stage_async(host_scheds[i % 2], None, tok, lab, loss_rows=pool[i % POOL][3], exchange_rows=xrows[i % POOL])
        schedule_ahead(i + 1)
        host_ms[0] += (time.perf_counter() - t0) * 1e3
        host_ms[1] += 1

    def stage_time():
        """What one batch's host scheduling + packing + upload costs when run synchronously (reported, not timed in e2e)."""
        par, tok, lab = pinned_np[0]
        for job in list(sched_job.values()):     # the scheduling thread is idle from here on
            job.result()
        sched_job.clear()
        eng.stage_wait()
        t0 = time.perf_counter()
        eng.stage(host_sched, par, tok, lab, loss_rows=pool[0][3], exchange_rows=xrows[0])
        return (time.perf_counter() - t0) * 1e3

    tail_view = eng.device_view(6, (2,))                       # [loss sum, status word] on the device
    LOSS_LAG = 2                                               # a step's loss is collected this many steps later
    loss_pinned = [torch.zeros(2, dtype=torch.float32).pin_memory() for _ in range(LOSS_LAG + 1)]
    loss_ready = [torch.cuda.Event() for _ in range(LOSS_LAG + 1)]

    pipeline = dict(primed=False, next=0)

    def e2e_loop(steps):
        # Software-pipelined like a data loader: while the GPU runs step i the host schedules batch i+1 and
        # enqueues its upload; every step's tables still cross PCIe inside the timed region, and every step's
        # loss comes back to the host -- through a pinned slot, collected two steps later (all of them before the
        # timed region ends) so that the host never drains the GPU's queue between steps: with a lag of one step the
        # ranks' host loops, each gated by its own GPU, cost 0.5 to 0.9 ms per step at 2 to 8 GPUs.
        losses = []

        def collect(slot):
            loss_ready[slot].synchronize()
            if loss_pinned[slot][1:].view(torch.int32).item() != 0:
                raise RuntimeError("a bounded device-side wait expired during the step")
            losses.append(float(loss_pinned[slot][0]))

        # Steady state: the warm-up call fills the pipeline (stages the first batch), and every call stages the
        # batch of the step after its last one, so a timed call of K steps contains exactly K host schedules,
        # K table uploads, K device steps and K loss read-backs.
        if not pipeline["primed"]:
            stage(pipeline["next"])
            pipeline["next"] += 1
            pipeline["primed"] = True
        pending = []
        for i in range(steps):
            # the batch staged during the previous step becomes current; the helper thread starts on the next one
            # at once, so it works beside this thread's enqueueing of the step (host side = the longer of the two)
            eng.promote()
            stage(pipeline["next"])
            pipeline["next"] += 1
            device_step()
            slot = i % (LOSS_LAG + 1)
            loss_pinned[slot].copy_(tail_view, non_blocking=True)
            loss_ready[slot].record()
            pending.append(slot)
            if len(pending) > LOSS_LAG:
                collect(pending.pop(0))
        while pending:
            collect(pending.pop(0))
        return losses

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        l0 = L.cavs_launch_count()
        e0.record()
        fn(steps)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        launches = L.cavs_launch_count() - l0
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, launches

    # ---- device-resident arm: tables of batch 0 already in HBM ----
    eng.load_batch(scheds[0], pool[0][1], pool[0][2], loss_rows=pool[0][3], exchange_rows=xrows[0])
    for _ in range(args.warmup):
        device_step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_dev, launches = timed(lambda k: [device_step() for _ in range(k)], args.steps)
    loss_dev = eng.read_loss()
    # The loss of the GLOBAL batch: every rank's shard summed.  After the same number of steps it equals the 1-GPU
    # run's loss_sum (same batch, same summed gradient, same updates) up to the rounding of the bf16 products.
    global_loss = loss_dev
    if world > 1:
        t = torch.tensor([loss_dev], device=dev, dtype=torch.float64)
        dist.all_reduce(t)
        global_loss = float(t.item())
    # ---- end-to-end arm: host arrays in, loss out, every step ----
    e2e_loop(args.warmup)
    ms_e2e, _ = timed(e2e_loop, args.steps)
    clocks = sampler.stop() if rank == 0 else {}

    host_stage_sync_ms = stage_time()
    # ---- per-kernel-class timing for the roofline (separate instrumented steps) ----
    L.cavs_treelstm_profile(eng._h, 1)
    prof_steps = 3
    eng.load_batch(scheds[0], pool[0][1], pool[0][2], loss_rows=pool[0][3], exchange_rows=xrows[0])
    eng.promote()     # the end-to-end loop promoted explicitly; the engine has stopped doing it by itself
    for _ in range(prof_steps):
        device_step()
    torch.cuda.synchronize()
    n_cls = 13
    ms_c = (ctypes.c_double * n_cls)(); work_c = (ctypes.c_double * n_cls)(); cnt_c = (ctypes.c_int * n_cls)()
    L.cavs_treelstm_profile_read(eng._h, ms_c, work_c, cnt_c, n_cls)
    L.cavs_treelstm_profile(eng._h, 0)
    names = ["gate_gemm", "cell_fwd", "cell_bwd", "gather_child_h", "scatter_child_grad", "loss_head", "embed_fwd", "embed_bwd",
             "column_sum", "allreduce_embedding", "allreduce_weights", "allreduce_exposed_wait", "optimizer"]
    peaks = measured_peaks()
    classes = {}
    for i, nm in enumerate(names):
        if cnt_c[i] == 0:
            continue
        rate = work_c[i] / (ms_c[i] * 1e-3) if ms_c[i] > 0 else 0.0
        if i == 0:
            classes[nm] = dict(ms_per_step=ms_c[i] / prof_steps, launches_per_step=cnt_c[i] // prof_steps, tflops=rate / 1e12,
                               frac=rate / 1e12 / peaks["tflops"])
        else:
            classes[nm] = dict(ms_per_step=ms_c[i] / prof_steps, launches_per_step=cnt_c[i] // prof_steps, gbs=rate / 1e9,
                               frac=rate / 1e9 / peaks["hbm_gbs"])
    # communication and optimizer time per step: the embedding block's all-reduce runs on a side stream (hidden_ms of
    # it lies under the weight-gradient products), the other blocks' and the wait for the side stream on the compute stream
    ms_of = lambda nm: classes[nm]["ms_per_step"] if nm in classes else 0.0
    comm_info = None
    if world > 1:
        comm_info = dict(allreduce_embedding_ms=ms_of("allreduce_embedding"), allreduce_weights_ms=ms_of("allreduce_weights"),
                         exposed_wait_ms=ms_of("allreduce_exposed_wait"),
                         hidden_ms=max(0.0, ms_of("allreduce_embedding") - ms_of("allreduce_exposed_wait")),
                         on_compute_stream_ms=ms_of("allreduce_weights") + ms_of("allreduce_exposed_wait"),
                         allreduce_bytes_per_step=4 * (int(eng.params.numel()) - (wl["vocab"] - int(np.mean([len(x) for x in xrows]))) * wl["embed"]
                                                       if sparse else int(eng.params.numel())),
                         dense_allreduce_bytes_per_step=4 * int(eng.params.numel()),
                         embedding_exchange=("rows the global batch touches (cavs_treelstm_set_exchange_rows): mean %d of %d table rows"
                                             % (int(np.mean([len(x) for x in xrows])), wl["vocab"])) if sparse else "dense block",
                         nccl_version=comm.nccl_version(),
                         issued_by="cavs_treelstm_step -> cavs_allreduce (ncclAllReduce called from the library)")
    optimizer_ms = ms_of("optimizer")
    for nm in ("allreduce_embedding", "allreduce_weights", "allreduce_exposed_wait", "optimizer"):
        classes.pop(nm, None)      # not kernels of this library's level loop: reported as comm / optimizer_ms
    dominant = max(classes, key=lambda k: classes[k]["ms_per_step"])
    d = classes[dominant]
    if dominant == "gate_gemm":
        # DRAM bytes per GEMM launch: captured with the profiler on one rank's shard at 8 GPUs (all GEMM launches of a
        # step) and scaled by internal vertices, to which every per-level operand and output is proportional: an
        # extrapolation, not a measurement of this run.
        internal_rows = int(scheds[0].n_total - scheds[0].level_off[1]) if scheds[0].n_levels > 1 else 0
        per_row = gemm_dram_bytes_per_internal_row()
        traffic = per_row * internal_rows / max(d["launches_per_step"], 1) if per_row is not None else None
        # `achieved` counts the flops the GEMM launches EXECUTE.  The per-vertex formula of the reference's algorithm
        # (every vertex multiplies its own input and its own children's states: 3 x (2 N E 4H + N_int (2 H 3H + 2 K H H)))
        # is reported beside it: the engine executes fewer flops than that, because products that depend on a vertex only
        # through its token (the input projection, the leaves' states and everything level 1 does with them) run once per
        # distinct token.
        H_, E_, K_ = wl["hidden"], wl["embed"], 2
        n_v = int(scheds[0].n_scheduled)
        formula = 3.0 * (2.0 * n_v * E_ * 4 * H_ + internal_rows * (2.0 * H_ * 3 * H_ + 2.0 * K_ * H_ * H_))
        roofline = dict(bound="tensor", kernel="GemmBf16Kernel (all gate / gradient GEMMs of a step)", achieved=d["tflops"],
                        peak=peaks["tflops"], unit="TFLOP/s", frac=d["frac"], traffic=traffic,
                        traffic_unit="DRAM bytes per launch, extrapolated: profiler capture of a 512-tree shard scaled by internal vertices",
                        peak_source=peaks["source"], flops_executed_per_step=work_c[0] / prof_steps,
                        flops_per_vertex_formula_per_step=formula)
    else:
        roofline = dict(bound="hbm", kernel=dominant, achieved=d["gbs"], peak=peaks["hbm_gbs"], unit="GB/s", frac=d["frac"],
                        traffic=None, peak_source=peaks["source"])

    # ---- the graph-op row kernels on their own (Gather / Scatter of child state rows, the reference's
    # BatchedDynamicSelected*Copy kernels): the widest internal level's gather list of slot 0, rows of h|c ----
    graph_ops = None
    if rank == 0 and scheds[0].n_levels > 1:
        lvl_rows = np.diff(scheds[0].level_off)
        lvl = 1 + int(np.argmax(lvl_rows[1:]))
        ids_h = scheds[0].ref_gather(lvl, 0)
        n_ids, row_bytes = int(ids_h.size), 2 * wl["hidden"] * 4
        ids_d = torch.from_numpy(ids_h).to(dev)
        src = torch.randn((int(scheds[0].n_total), 2 * wl["hidden"]), device=dev)
        dst = torch.empty((n_ids, 2 * wl["hidden"]), device=dev)
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        vp = lambda t: ctypes.c_void_p(t.data_ptr())

        def run_rows(fn, reps=10):
            for _ in range(3):
                fn()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / reps * 1e-3

        work = n_ids * (2 * row_bytes + 4)
        t_g = run_rows(lambda: lib_check(L.cavs_gather_rows(vp(dst), vp(src), vp(ids_d), n_ids, ctypes.c_size_t(row_bytes), st)))
        t_s = run_rows(lambda: lib_check(L.cavs_scatter_rows(vp(src), vp(ids_d), vp(dst), n_ids, ctypes.c_size_t(row_bytes), st)))
        graph_ops = dict(rows=n_ids, row_bytes=row_bytes, level=lvl, gather_gbs=work / t_g / 1e9, scatter_gbs=work / t_s / 1e9,
                         gather_frac=work / t_g / 1e9 / peaks["hbm_gbs"], scatter_frac=work / t_s / 1e9 / peaks["hbm_gbs"],
                         note="cavs_gather_rows / cavs_scatter_rows on the widest internal level's child list; "
                              "bytes = rows x (read + write of a row + its index); source and target exceed L2")
        del src, dst

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    trees = wl["batch"]
    value = trees * args.steps / (ms_dev * 1e-3)
    e2e_value = trees * args.steps / (ms_e2e * 1e-3)
    # tables uploaded per step (child and child-state rows, parent, token, label, order, token row, state row,
    # loss-head rows, the per-token chunk / histogram tables, the link lists of level 1): counted by the engine
    h2d = eng.upload_bytes()
    line = dict(metric="treelstm_train_trees_per_sec", value=value, unit="trees/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                ms_per_step=ms_dev / args.steps, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="bf16" if wl["bf16"] else "f32", data="synthetic",
                config=dict(workload=args.workload, global_batch=trees, trees_per_gpu=trees // world, hidden=wl["hidden"],
                            embed=wl["embed"], vocab=wl["vocab"], classes=wl["classes"], leaves=[wl["leaf_lo"], wl["leaf_hi"]],
                            vertices_per_gpu=int(scheds[0].n_total), levels=int(scheds[0].n_levels), optimizer="adagrad",
                            parallelism=f"dp{world}", l2="working set per step (tens of GB) exceeds L2; no flush needed",
                            embedding_gradient=("rows the global batch touches (mean %d of %d), listed with the batch"
                                                % (int(np.mean([len(x) for x in xrows])), wl["vocab"])) if sparse else "dense block"),
                e2e=dict(value=e2e_value, unit="trees/s", ms_per_step=ms_e2e / args.steps, h2d_bytes_per_step=h2d, d2h_bytes_per_step=8,
                         host_stage_ms=host_stage_sync_ms, host_stage_mode=("three stations: cavs_sched_load of batch i+2 on a thread of the script, packing + upload of batch "
                                          "i+1 on the engine's helper thread (cavs_treelstm_promote, cavs_treelstm_stage_async), "
                                          "enqueueing of step i"),
                         loss_read="every step into a pinned slot, collected two steps later"),
                gpu_launches=int(launches), gpu_launches_per_step=int(launches) // max(args.steps, 1), loss_sum=loss_dev,
                global_loss_sum=global_loss, comm=comm_info, optimizer_ms=optimizer_ms, clocks=clocks, roofline=roofline,
                kernel_classes=classes, graph_ops=graph_ops)
    if not args.no_cpu_baseline and world == 1:   # torchrun pins ranks to one host thread: the CPU arm runs at N=1 only
        rate, secs, gflops = cpu_baseline_sample(wl, args.sample_trees)
        import oracle
        line["cpu_baseline"] = dict(value=rate, unit="trees/s", cores=oracle.num_threads(), kind="port", gemm_gflops=gflops,
                                    sample=f"{args.sample_trees} trees (numpy-generated sample of the workload), one step: level "
                                           f"scheduling + fwd + bwd + Adagrad ({secs:.1f} s)")
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
