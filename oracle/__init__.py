"""TEST INFRASTRUCTURE: ctypes loaders for the CPU oracle.

`oracle_lib()` is the plain-C restatement (oracle/cavs_oracle.c); `refsched_lib()` is the
reference's own graph scheduler compiled against stand-in headers (oracle/_ref/, built by
oracle/Makefile where the reference checkout is present, prebuilt elsewhere).  Only tests,
the smoke check and the benchmark's CPU-baseline leg import this package; the product never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_oracle = None
_ref = None


def reference_checkout() -> str:
    """Where the reference project's sources lie: $CAVS_REFERENCE, else a directory named `reference` beside this
    repository; empty if neither exists (the compiled reference scheduler is then kept as prebuilt)."""
    for cand in (os.environ.get("CAVS_REFERENCE", ""), str(HERE.parent.parent / "reference")):
        if cand and (Path(cand) / "cavs" / "midend" / "graph_scheduler.cc").is_file():
            return cand
    return ""


def build(verbose: bool = False) -> None:
    subprocess.run(["make", "-C", str(HERE), "all", f"REF={reference_checkout()}"], check=True, capture_output=not verbose)


def oracle_lib() -> ctypes.CDLL:
    global _oracle
    if _oracle is None:
        p = HERE / "libcavs_oracle.so"
        if not p.exists():
            build()
        _oracle = ctypes.CDLL(str(p))
    return _oracle


def refsched_lib():
    """The compiled reference scheduler, or None if it was never built on this machine."""
    global _ref
    if _ref is None:
        p = HERE / "_ref" / "libcavs_refsched.so"
        if not p.exists():
            return None
        _ref = ctypes.CDLL(str(p))
    return _ref


def _p(a):
    return ctypes.c_void_p(0) if a is None else ctypes.c_void_p(a.ctypes.data)


def _stream(fn, parents: np.ndarray) -> np.ndarray:
    parents = np.ascontiguousarray(parents, np.int32)
    cap = 1 << 16
    while True:
        out = np.empty(cap, np.int32)
        n = fn(_p(parents), parents.shape[0], parents.shape[1], _p(out), cap)
        if n >= 0:
            return out[:n].copy()
        if n <= -1000000 + 10:
            raise ValueError(f"malformed graph (code {n + 1000000})")
        cap = -n


def ref_schedule_stream(parents: np.ndarray) -> np.ndarray:
    lib = refsched_lib()
    if lib is None:
        raise FileNotFoundError("oracle/_ref/libcavs_refsched.so not built")
    return _stream(lib.refsched_stream, parents)


def schedule_stream(parents: np.ndarray) -> np.ndarray:
    return _stream(oracle_lib().cavs_oracle_schedule_stream, parents)


def ref_serial_stream(parents: np.ndarray) -> np.ndarray:
    """The reference's SerialGraphScheduler, driven through one forward and one backward sweep."""
    lib = refsched_lib()
    if lib is None or not hasattr(lib, "refsched_serial_stream"):
        raise FileNotFoundError("oracle/_ref/libcavs_refsched.so not built")
    return _stream(lib.refsched_serial_stream, parents)


def serial_stream(parents: np.ndarray) -> np.ndarray:
    """Restatement of the serial sweep (layout: oracle/refsched_driver.cc)."""
    return _stream(oracle_lib().cavs_oracle_serial_stream, parents)


def tables(parents: np.ndarray, n_slots: int = 2, mode: int = 0):
    parents = np.ascontiguousarray(parents, np.int32)
    b, m = parents.shape
    cap = b * m
    n_total = ctypes.c_int()
    level_off = np.empty(m + 2, np.int32)
    t2j = np.empty(cap, np.int32); j2t = np.empty(cap, np.int32)
    fg = np.empty(cap * n_slots, np.int32); bs = np.empty(cap * n_slots, np.int32)
    fs = np.empty(cap, np.int32); bg = np.empty(cap, np.int32)
    L = oracle_lib().cavs_oracle_tables(_p(parents), b, m, n_slots, mode, ctypes.byref(n_total), _p(level_off), level_off.size,
                                        _p(t2j), _p(j2t), _p(fg), _p(fs), _p(bg), _p(bs))
    if L < 0:
        raise ValueError(f"malformed graph (code {L})")
    n = n_total.value
    return dict(n=n, n_levels=L, level_off=level_off[: L + 1].copy(), t2j=t2j[:n].copy(), j2t=j2t[:n].copy(),
                fg=fg[: n * n_slots].reshape(n_slots, n).copy(), bs=bs[: n * n_slots].reshape(n_slots, n).copy(),
                fs=fs[:n].copy(), bg=bg[:n].copy())


class Cfg(ctypes.Structure):
    _fields_ = [(k, ctypes.c_int) for k in
                ("n", "n_levels", "hidden", "embed", "vocab", "classes", "n_slots", "gemm_bf16", "loss_rows", "preact_bf16")]


def treelstm_fwd_bwd(tb: dict, tok, label, params: dict, H, E, V, C, K=2, gemm_bf16=False, loss_rows=0, want_dstate=False,
                     preact_bf16=False):
    """Runs the oracle's Tree-LSTM forward + loss + backward on index tables `tb`
    (from tables() or from the product scheduler).  Returns a dict of numpy arrays."""
    n = int(tb["n"])
    cfg = Cfg(n, int(tb["n_levels"]), H, E, V, C, K, int(gemm_bf16), int(loss_rows), int(preact_bf16))
    f32 = lambda a: np.ascontiguousarray(a, np.float32)
    i32 = lambda a: np.ascontiguousarray(a, np.int32)
    Emb, W, U, B, Wc, bc = (f32(params[k]) for k in ("Emb", "W", "U", "B", "Wc", "bc"))
    out = dict(state=np.zeros((n, 2 * H), np.float32), loss=np.zeros(n, np.float32), dEmb=np.zeros_like(Emb),
               dW=np.zeros_like(W), dU=np.zeros_like(U), dB=np.zeros_like(B), dWc=np.zeros_like(Wc), dbc=np.zeros_like(bc))
    dstate = np.zeros((n, 2 * H), np.float32) if want_dstate else None
    lo, fg, fs, bg, bs = i32(tb["level_off"]), i32(tb["fg"]), i32(tb["fs"]), i32(tb["bg"]), i32(tb["bs"])
    tok, label = i32(tok), i32(label)
    rc = oracle_lib().cavs_oracle_treelstm_fwd_bwd(
        ctypes.byref(cfg), _p(lo), _p(fg), _p(fs), _p(bg), _p(bs), _p(tok), _p(label), _p(Emb), _p(W), _p(U), _p(B), _p(Wc), _p(bc),
        _p(out["state"]), _p(out["loss"]), _p(out["dEmb"]), _p(out["dW"]), _p(out["dU"]), _p(out["dB"]), _p(out["dWc"]),
        _p(out["dbc"]), _p(dstate))
    assert rc == 0
    if want_dstate:
        out["dstate"] = dstate
    return out


def treelstm_layer(tb: dict, params: dict, H, E, K=1, tok=None, x_dense=None, label=None, dh_ext=None, V=0, C=0,
                   gemm_bf16=False, loss_rows=0, preact_bf16=False):
    """One layer of a stack: inputs are either tokens (Emb lookup) or dense rows x_dense [n,E]; the output
    gradient is either the layer's own loss head (label, Wc, bc) or dh_ext [n,H] from the layer above.
    Returns state, loss, dW, dU, dB, dX ([n,E]) and, where they exist, dEmb, dWc, dbc."""
    n = int(tb["n"])
    cfg = Cfg(n, int(tb["n_levels"]), H, E, max(V, 1), C, K, int(gemm_bf16), int(loss_rows), int(preact_bf16))
    f32 = lambda a: None if a is None else np.ascontiguousarray(a, np.float32)
    i32 = lambda a: None if a is None else np.ascontiguousarray(a, np.int32)
    Emb, W, U, B, Wc, bc = (f32(params.get(k)) for k in ("Emb", "W", "U", "B", "Wc", "bc"))
    assert (tok is None) != (x_dense is None) and (label is None) != (dh_ext is None)
    out = dict(state=np.zeros((n, 2 * H), np.float32), loss=np.zeros(n, np.float32), dW=np.zeros_like(W), dU=np.zeros_like(U),
               dB=np.zeros_like(B), dX=np.zeros((n, E), np.float32))
    if x_dense is None:
        out["dEmb"] = np.zeros_like(Emb)
    if dh_ext is None:
        out["dWc"], out["dbc"] = np.zeros_like(Wc), np.zeros_like(bc)
    lo, fg, fs, bg, bs = (i32(tb[k]) for k in ("level_off", "fg", "fs", "bg", "bs"))
    tok, label, x_dense, dh_ext = i32(tok), i32(label), f32(x_dense), f32(dh_ext)
    rc = oracle_lib().cavs_oracle_treelstm_layer(
        ctypes.byref(cfg), _p(lo), _p(fg), _p(fs), _p(bg), _p(bs), _p(tok), _p(label), _p(Emb), _p(W), _p(U), _p(B), _p(Wc), _p(bc),
        _p(out["state"]), _p(out["loss"]), _p(out.get("dEmb")), _p(out["dW"]), _p(out["dU"]), _p(out["dB"]), _p(out.get("dWc")),
        _p(out.get("dbc")), _p(x_dense), _p(dh_ext), _p(out["dX"]))
    assert rc == 0
    return out


def treegru_fwd_bwd(tb: dict, tok, label, params: dict, H, E, V, C, K=4, gemm_bf16=False, loss_rows=0, preact_bf16=False):
    """Child-sum Tree-GRU forward + loss + backward (an extension defined by the oracle).  params: Emb [V,E],
    W [E*3H] (r,z,n), U [3*H*H] (U_r|U_z|U_n), B [3H], Wc [C,H], bc [C]."""
    n = int(tb["n"])
    cfg = Cfg(n, int(tb["n_levels"]), H, E, V, C, K, int(gemm_bf16), int(loss_rows), int(preact_bf16))
    f32 = lambda a: np.ascontiguousarray(a, np.float32)
    i32 = lambda a: np.ascontiguousarray(a, np.int32)
    Emb, W, U, B, Wc, bc = (f32(params[k]) for k in ("Emb", "W", "U", "B", "Wc", "bc"))
    out = dict(state=np.zeros((n, H), np.float32), loss=np.zeros(n, np.float32), dEmb=np.zeros_like(Emb),
               dW=np.zeros_like(W), dU=np.zeros_like(U), dB=np.zeros_like(B), dWc=np.zeros_like(Wc), dbc=np.zeros_like(bc))
    lo, fg, fs, bg, bs = i32(tb["level_off"]), i32(tb["fg"]), i32(tb["fs"]), i32(tb["bg"]), i32(tb["bs"])
    tok, label = i32(tok), i32(label)
    rc = oracle_lib().cavs_oracle_treegru_fwd_bwd(
        ctypes.byref(cfg), _p(lo), _p(fg), _p(fs), _p(bg), _p(bs), _p(tok), _p(label), _p(Emb), _p(W), _p(U), _p(B), _p(Wc), _p(bc),
        _p(out["state"]), _p(out["loss"]), _p(out["dEmb"]), _p(out["dW"]), _p(out["dU"]), _p(out["dB"]), _p(out["dWc"]),
        _p(out["dbc"]))
    assert rc == 0
    return out


def sgd(w, g, lr):
    oracle_lib().cavs_oracle_sgd(_p(w), _p(g), ctypes.c_size_t(w.size), ctypes.c_float(lr))


def adagrad(w, acc, g, lr, eps=1e-10):
    oracle_lib().cavs_oracle_adagrad(_p(w), _p(acc), _p(g), ctypes.c_size_t(w.size), ctypes.c_float(lr), ctypes.c_float(eps))


def num_threads() -> int:
    return oracle_lib().cavs_oracle_num_threads()
