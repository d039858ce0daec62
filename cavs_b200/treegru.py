"""Tree-GRU engine binding (cavs_treegru_*): same shape as the Tree-LSTM binding, a second vertex function
over the same scheduler tables."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from ._abi import check, lib, ptr
from .schedule import Schedule
from .treelstm import Config, _stream


class TreeGRU:
    """Level-batched child-sum Tree-GRU training step on one GPU."""

    PARAM_NAMES = ("Emb", "W", "U", "B", "Wc", "bc")

    def __init__(self, hidden, embed, vocab, classes, n_slots=2, gemm_bf16=False, max_vertices=1 << 16, max_level_rows=None,
                 device="cuda"):
        L = lib()
        L.cavs_treegru_param_count.restype = ctypes.c_size_t
        L.cavs_treegru_workspace_bytes.restype = ctypes.c_size_t
        self.cfg = Config(hidden, embed, vocab, classes, n_slots, int(gemm_bf16), max_vertices, max_level_rows or max_vertices)
        self.device = torch.device(device)
        n_params = L.cavs_treegru_param_count(ctypes.byref(self.cfg))
        ws = L.cavs_treegru_workspace_bytes(ctypes.byref(self.cfg))
        if n_params == 0 or ws == 0:
            check(1)
        self.params = torch.zeros(n_params, dtype=torch.float32, device=self.device)
        self.grads = torch.zeros(n_params, dtype=torch.float32, device=self.device)
        self.workspace = torch.empty(ws + 256, dtype=torch.uint8, device=self.device)
        base = (self.workspace.data_ptr() + 255) // 256 * 256
        self._h = ctypes.c_void_p()
        check(L.cavs_treegru_create(ctypes.byref(self.cfg), ctypes.c_void_p(base), ctypes.c_size_t(ws), ctypes.byref(self._h)))
        check(L.cavs_treegru_bind(self._h, ctypes.c_void_p(self.params.data_ptr()), ctypes.c_void_p(self.grads.data_ptr())))
        H, E, V, C = hidden, embed, vocab, classes
        sizes = [V * E, E * 3 * H, 3 * H * H, 3 * H, C * H, C]
        self.offsets = dict(zip(self.PARAM_NAMES, np.concatenate([[0], np.cumsum(sizes)[:-1]]).tolist()))
        self.sizes = dict(zip(self.PARAM_NAMES, sizes))
        self.n = 0

    def close(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib().cavs_treegru_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_params(self, params: dict) -> None:
        for k in self.PARAM_NAMES:
            o, s = self.offsets[k], self.sizes[k]
            self.params[o:o + s].copy_(torch.from_numpy(np.ascontiguousarray(params[k], np.float32).ravel()))
        check(lib().cavs_treegru_refresh_weights(self._h, _stream()))

    def load_batch(self, sched: Schedule, tok_job: np.ndarray, label_job: np.ndarray, loss_rows: int = 0) -> None:
        tok_job = np.ascontiguousarray(tok_job, np.int32)
        label_job = np.ascontiguousarray(label_job, np.int32)
        assert tok_job.size >= sched.n_total and label_job.size >= sched.n_total
        check(lib().cavs_treegru_load_batch(self._h, sched._h, ptr(tok_job), ptr(label_job), loss_rows, _stream()))
        self.n = sched.n_scheduled

    def forward(self) -> None:
        check(lib().cavs_treegru_forward(self._h, _stream()))

    def backward(self) -> None:
        check(lib().cavs_treegru_backward(self._h, _stream()))

    def read_loss(self) -> float:
        out, status = ctypes.c_float(), ctypes.c_int()
        check(lib().cavs_treegru_read_loss(self._h, ctypes.byref(out), ctypes.byref(status), _stream()))
        return out.value

    def peek(self, what: int, shape) -> np.ndarray:
        p, nbytes = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().cavs_treegru_peek(self._h, what, ctypes.byref(p), ctypes.byref(nbytes)))
        off = p.value - self.workspace.data_ptr()
        t = self.workspace[off:off + nbytes.value].view(torch.float32)
        torch.cuda.synchronize()
        return t.cpu().numpy().reshape(shape)

    def state(self) -> np.ndarray:
        return self.peek(0, (self.n, self.cfg.hidden))

    def loss_rows(self) -> np.ndarray:
        return self.peek(1, (self.n,))

    def grad_dict(self) -> dict:
        torch.cuda.synchronize()
        g = self.grads.cpu().numpy()
        return {"d" + k: g[self.offsets[k]:self.offsets[k] + self.sizes[k]].copy() for k in self.PARAM_NAMES}
