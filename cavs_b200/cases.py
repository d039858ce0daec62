"""A profiling harness, not part of the product: the commands recorded with the profiler summaries run it.

Small, self-contained cases of the library's kernels, sized for profiler captures
(inputs larger than L2, a few GB on the device at most, a handful of launches).

    python -m cavs_b200.cases gemm    one per-level gate product: [65536,1024] x [1024,3072], bf16 in / bf16 out
    python -m cavs_b200.cases loss    the fused loss head on 65536 rows of hidden size 1024, 5 classes
    python -m cavs_b200.cases cell    one interior level of 32768 two-child vertices (hidden 1024, 2 slots, bf16 mode):
                                      child-state gather, cell forward, cell backward, child-gradient scatter
    python -m cavs_b200.cases level   three training steps of the Tree-LSTM engine on 32768 two-leaf trees with level 1 run per
                                      vertex (CAVS_LEVEL1_BY_TOKEN=0): one interior level of 32768 rows through exactly the
                                      kernels of the benchmark step's levels from 2 up -- child-state gather, the two gate
                                      products with the gate epilogue, the light forward cell, the backward cell with the
                                      fused loss-head gradient, the two gradient products (hidden 1024, bf16, ~3 GB)
    python -m cavs_b200.cases gru     three forward + backward passes of the Tree-GRU engine on 16384 trees of 2..4 leaves
                                      under one root (hidden 1024, embedding 512, 4 child slots, bf16): one interior level
    python -m cavs_b200.cases rows    the graph ops' row kernels: gather and scatter of 88320 rows of 8 KB (h|c of hidden 1024)
                                      through a random index list, three times each (1.4 GB)
    python -m cavs_b200.cases shard   two training steps of the Tree-LSTM engine on one rank's shard of the
                                      benchmark workload at 8 GPUs (512 trees, ~66 k vertices, ~4 GB);
                                      `shard 50` also times 50 further steps with CUDA events
    python -m cavs_b200.cases unbatched [steps]
                                      what level batching buys: the binary Tree-LSTM configuration (64 trees of 2..50
                                      leaves, hidden 150, embedding 300, fp32) stepped with the level schedule and with the
                                      one-vertex-per-round schedule (the reference's serial scheduler), CUDA-event times
"""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from cavs_b200 import lib, schedule as S  # noqa: E402
from cavs_b200.treelstm import TreeLSTM  # noqa: E402


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _st():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def gemm(iters: int = 3) -> None:
    L, dev, ll = lib(), torch.device("cuda"), ctypes.c_longlong
    m, n, k = 65536, 3072, 1024
    a = torch.randn((m, k), device=dev).to(torch.bfloat16)
    b = torch.randn((k, n), device=dev).to(torch.bfloat16)
    c = torch.empty((m, n), device=dev, dtype=torch.bfloat16)
    for _ in range(iters):
        rc = L.cavs_gemm_bf16(_p(c), ll(n), 2, _p(a), ll(k), 0, _p(b), ll(n), 1, m, n, k, 1, _p(None), ctypes.c_size_t(0), _p(None), _st())
        assert rc == 0, L.cavs_last_error()
    torch.cuda.synchronize()


def loss(iters: int = 3) -> None:
    L, dev, ll = lib(), torch.device("cuda"), ctypes.c_longlong
    L.cavs_fc_softmax_xent_scratch_bytes.restype = ctypes.c_size_t
    rows, H, C = 65536, 1024, 5
    state = torch.randn((rows, 2 * H), device=dev)
    label = torch.randint(0, C, (rows,), device=dev, dtype=torch.int32)
    Wc = torch.randn((C, H), device=dev) * 0.05
    bc = torch.zeros(C, device=dev)
    out = [torch.empty(rows, device=dev), torch.empty(4, device=dev), torch.empty((rows, H), device=dev),
           torch.empty((C, H), device=dev), torch.empty(C, device=dev)]
    scratch = torch.empty(L.cavs_fc_softmax_xent_scratch_bytes(H, C), dtype=torch.uint8, device=dev)
    for _ in range(iters):
        rc = L.cavs_fc_softmax_xent(*map(_p, out), _p(state), ll(2 * H), _p(label), _p(Wc), _p(bc), rows, H, C,
                                    ctypes.c_float(1.0 / rows), _p(scratch), _st())
        assert rc == 0, L.cavs_last_error()
    torch.cuda.synchronize()


def cell(iters: int = 3) -> None:
    L, dev = lib(), torch.device("cuda")
    R, H, K = 32768, 1024, 2
    n = 3 * R                                   # children occupy rows [0, 2R), the level rows [2R, 3R)
    bf, hf = torch.bfloat16, torch.float16
    child = torch.full((K, n), -1, dtype=torch.int32)
    child[0, 2 * R:] = torch.arange(0, 2 * R, 2, dtype=torch.int32)
    child[1, 2 * R:] = torch.arange(1, 2 * R, 2, dtype=torch.int32)
    parent = torch.full((n,), -1, dtype=torch.int32)
    parent[:2 * R] = 2 * R + torch.arange(2 * R, dtype=torch.int32) // 2
    child, parent = child.to(dev), parent.to(dev)
    state = torch.randn((n, 2 * H), device=dev) * 0.5
    gates = torch.empty((n, (3 + K) * H), device=dev, dtype=hf)
    A = (torch.randn((n, 4 * H), device=dev) * 0.5).to(bf)
    P = (torch.randn((R, 3 * H), device=dev) * 0.5).to(bf)
    Q = (torch.randn((R, K, H), device=dev) * 0.5).to(bf)
    bias = torch.zeros(4 * H, device=dev)
    S = torch.empty((R, H), device=dev, dtype=bf)
    HK = torch.empty((R, K, H), device=dev, dtype=bf)
    mailbox = torch.randn((n, 2 * H), device=dev) * 0.1
    dOut = torch.randn((n, H), device=dev) * 0.1
    dA = torch.empty((n, 4 * H), device=dev, dtype=bf)
    ZF = torch.empty((n, K, H), device=dev, dtype=bf)
    ds = torch.randn((R, H), device=dev) * 0.1
    dq = torch.randn((R, K, H), device=dev) * 0.1
    for _ in range(iters):
        for rc in (
            L.cavs_gather_child_h(_p(S), _p(HK), 1, _p(state), _p(child), n, 2 * R, R, H, K, _st()),
            L.cavs_treelstm_cell_fwd(_p(state), _p(gates), _p(A), _p(P), _p(Q), 1, _p(bias), _p(child), _p(None), n, 2 * R, R,
                                     H, K, 0, _st()),
            L.cavs_treelstm_cell_bwd(_p(dA), _p(ZF), 1, _p(mailbox), _p(dOut), _p(gates), _p(state), _p(child), _p(parent), n,
                                     2 * R, R, H, K, 0, _st()),
            L.cavs_scatter_child_grad(_p(mailbox), _p(ds), _p(dq), _p(child), n, 2 * R, R, H, K, _st()),
        ):
            assert rc == 0, L.cavs_last_error()
    torch.cuda.synchronize()


def shard(steps: int = 2) -> None:
    import bench
    wl = bench.WORKLOADS["dp_treelstm"]
    par, tok, lab, _ = bench.make_batch(wl, 0, 0, 8)
    s = S.Schedule().load(par)
    eng = TreeLSTM(wl["hidden"], wl["embed"], wl["vocab"], wl["classes"], gemm_bf16=True, max_vertices=s.n_total,
                   max_level_rows=s.max_level_rows)
    eng.set_params(bench.make_params(wl))
    eng.load_batch(s, tok, lab)
    for _ in range(steps):
        eng.forward()
        eng.backward()
    print("loss", eng.read_loss(), "vertices", s.n_total, "levels", s.n_levels)
    if steps > 2:   # timing run: forward + backward of the resident shard, CUDA events on the launching stream
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            eng.forward()
            eng.backward()
        b.record()
        torch.cuda.synchronize()
        print("ms_per_step", a.elapsed_time(b) / steps)


def rows(iters: int = 3) -> None:
    L, dev = lib(), torch.device("cuda")
    n, n_src, row_bytes = 88320, 176640, 8192
    ids = torch.randperm(n_src, device=dev)[:n].to(torch.int32)
    src = torch.randn((n_src, row_bytes // 4), device=dev)
    dst = torch.empty((n, row_bytes // 4), device=dev)
    for _ in range(iters):
        assert L.cavs_gather_rows(_p(dst), _p(src), _p(ids), n, ctypes.c_size_t(row_bytes), _st()) == 0, L.cavs_last_error()
        assert L.cavs_scatter_rows(_p(src), _p(ids), _p(dst), n, ctypes.c_size_t(row_bytes), _st()) == 0, L.cavs_last_error()
    torch.cuda.synchronize()


def level(steps: int = 3) -> None:
    import os
    import numpy as np
    os.environ["CAVS_LEVEL1_BY_TOKEN"] = "0"
    H, E, V, C, trees = 1024, 1024, 50000, 5, 32768
    parents = np.full((trees, 3), -1, np.int32)
    parents[:, 0] = parents[:, 1] = 2                      # two leaves under one root
    tok = np.zeros((trees, 3), np.int32)
    tok[:, :2] = S.synth_zipf(5, 1.1, V, 2 * trees).reshape(trees, 2)
    lab = S.synth_uniform_int(6, C, 3 * trees)
    s = S.Schedule().load(parents)
    eng = TreeLSTM(H, E, V, C, gemm_bf16=True, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    u = lambda seed, *shape: S.synth_uniform_float(seed, 0.05, shape)
    eng.set_params(dict(Emb=u(1, V, E), W=u(2, E * 4 * H), U=u(3, 4 * H * H), B=np.zeros(4 * H, np.float32), Wc=u(4, C, H),
                        bc=np.zeros(C, np.float32)))
    eng.load_batch(s, tok.reshape(-1), lab)
    for _ in range(steps):
        eng.forward()
        eng.backward()
    print("loss", eng.read_loss(), "vertices", s.n_total, "levels", s.n_levels, "level rows", np.diff(s.level_off).tolist())


def gru(steps: int = 3) -> None:
    import numpy as np
    from cavs_b200.treegru import TreeGRU
    H, E, V, C, trees, K = 1024, 512, 32000, 2, 16384, 4
    leaves = 2 + (np.arange(trees) % 3)                    # 2, 3 or 4 leaves under one root
    parents = np.full((trees, 5), -1, np.int32)
    tok = np.zeros((trees, 5), np.int32)
    for k in (2, 3, 4):
        rows = leaves == k
        parents[rows, :k] = k
        tok[rows, :k] = S.synth_zipf(5 + k, 1.1, V, int(rows.sum()) * k).reshape(-1, k)
    lens = leaves + 1
    mask = np.arange(5)[None, :] < lens[:, None]
    lab = np.full(int(lens.sum()), -1, np.int32)
    lab[np.cumsum(lens) - 1] = S.synth_uniform_int(9, C, trees)
    s = S.Schedule().load(parents, n_slots=K)
    eng = TreeGRU(H, E, V, C, n_slots=K, gemm_bf16=True, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
    u = lambda seed, *shape: S.synth_uniform_float(seed, 0.05, shape)
    eng.set_params(dict(Emb=u(1, V, E), W=u(2, E * 3 * H), U=u(3, 3 * H * H), B=np.zeros(3 * H, np.float32), Wc=u(4, C, H),
                        bc=np.zeros(C, np.float32)))
    eng.load_batch(s, tok[mask].astype(np.int32), lab, loss_rows=trees)
    for _ in range(steps):
        eng.forward()
        eng.backward()
    print("loss", eng.read_loss(), "vertices", s.n_total, "levels", s.n_levels, "level rows", np.diff(s.level_off).tolist())


def unbatched(steps: int = 10) -> None:
    import numpy as np
    H, E, V, C, batch = 150, 300, 21701, 5, 64
    parents, is_leaf = S.synth_trees(2, batch, 2, 50)
    lens = (parents == -1).argmax(1) + 1
    tok_pad = S.synth_zipf(3, 1.1, V, parents.size).reshape(parents.shape) * is_leaf
    tok = np.concatenate([tok_pad[i, :lens[i]] for i in range(batch)]).astype(np.int32)
    lab = S.synth_uniform_int(4, C, int(lens.sum()))
    params = dict(Emb=S.synth_uniform_float(10, 0.05, (V, E)), W=S.synth_uniform_float(11, 0.05, (E * 4 * H,)),
                  U=S.synth_uniform_float(12, 0.05, (4 * H * H,)), Wc=S.synth_uniform_float(13, 0.05, (C, H)),
                  B=np.zeros(4 * H, np.float32), bc=np.zeros(C, np.float32))
    for order, name in ((S.BATCHED, "level schedule"), (S.UNBATCHED, "one vertex per round")):
        s = S.Schedule().set_order(order).load(parents)
        eng = TreeLSTM(H, E, V, C, max_vertices=s.n_total, max_level_rows=s.max_level_rows)
        eng.set_params(params)
        eng.load_batch(s, tok, lab)
        for _ in range(2):
            eng.forward()
            eng.backward()
        loss_sum = eng.read_loss()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            eng.forward()
            eng.backward()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        print(f"{name}: {s.n_levels} rounds, {s.n_total} vertices, loss {loss_sum:.4f}, {ms:.3f} ms per forward+backward, "
              f"{batch / ms * 1e3:.0f} trees/s")


if __name__ == "__main__":
    fn = {"gemm": gemm, "loss": loss, "cell": cell, "shard": shard, "unbatched": unbatched, "level": level, "gru": gru, "rows": rows}[sys.argv[1]]
    fn(*(int(a) for a in sys.argv[2:3]))   # optional iteration / step count
    print("ok", sys.argv[1])
