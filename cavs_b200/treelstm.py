"""Tree-LSTM engine binding: device memory comes from torch, every computation goes
through the C ABI (cavs_treelstm_*).  Used by the tests and the benchmark."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from ._abi import check, lib, ptr
from .schedule import Schedule


class Config(ctypes.Structure):
    _fields_ = [(k, ctypes.c_int) for k in
                ("hidden", "embed", "vocab", "classes", "n_slots", "gemm_bf16", "max_vertices", "max_level_rows")]


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class TreeLSTM:
    """Level-batched child-sum Tree-LSTM training step on one GPU."""

    PARAM_NAMES = ("Emb", "W", "U", "B", "Wc", "bc")

    def __init__(self, hidden, embed, vocab, classes, n_slots=2, gemm_bf16=False, max_vertices=1 << 16, max_level_rows=None,
                 device="cuda"):
        L = lib()
        L.cavs_treelstm_param_count.restype = ctypes.c_size_t
        L.cavs_treelstm_workspace_bytes.restype = ctypes.c_size_t
        self.cfg = Config(hidden, embed, vocab, classes, n_slots, int(gemm_bf16), max_vertices, max_level_rows or max_vertices)
        self.device = torch.device(device)
        n_params = L.cavs_treelstm_param_count(ctypes.byref(self.cfg))
        ws = L.cavs_treelstm_workspace_bytes(ctypes.byref(self.cfg))
        if n_params == 0 or ws == 0:
            check(1 if not L.cavs_last_error() else 1)
        self.params = torch.zeros(n_params, dtype=torch.float32, device=self.device)
        self.grads = torch.zeros(n_params, dtype=torch.float32, device=self.device)
        self.workspace = torch.empty(ws + 256, dtype=torch.uint8, device=self.device)
        base = (self.workspace.data_ptr() + 255) // 256 * 256
        self._h = ctypes.c_void_p()
        check(L.cavs_treelstm_create(ctypes.byref(self.cfg), ctypes.c_void_p(base), ctypes.c_size_t(ws), ctypes.byref(self._h)))
        check(L.cavs_treelstm_bind(self._h, ctypes.c_void_p(self.params.data_ptr()), ctypes.c_void_p(self.grads.data_ptr())))
        H, E, V, C = hidden, embed, vocab, classes
        sizes = [V * E, E * 4 * H, 4 * H * H, 4 * H, C * H, C]
        self.offsets = dict(zip(self.PARAM_NAMES, np.concatenate([[0], np.cumsum(sizes)[:-1]]).tolist()))
        self.sizes = dict(zip(self.PARAM_NAMES, sizes))
        self.n = 0

    def close(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib().cavs_treelstm_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        o, s = self.offsets[name], self.sizes[name]
        return flat[o:o + s]

    def set_params(self, params: dict) -> None:
        for k in self.PARAM_NAMES:
            if self.sizes[k]:
                self.view(self.params, k).copy_(torch.from_numpy(np.ascontiguousarray(params[k], np.float32).ravel()))
        self.refresh_weights()

    def refresh_weights(self) -> None:
        check(lib().cavs_treelstm_refresh_weights(self._h, _stream()))

    def set_exchange_rows(self, rows) -> None:
        """Sparse exchange of the embedding gradient for the NEXT batch loaded or staged: `rows` = ascending table rows
        touched by any rank's shard of it (identical on every rank).  The embedding block of `grads` then holds one row
        per listed row, step() all-reduces and applies only those.  None / empty: dense block."""
        rows = np.ascontiguousarray(rows if rows is not None else [], np.int32)
        check(lib().cavs_treelstm_set_exchange_rows(self._h, ptr(rows) if rows.size else ptr(None), int(rows.size)))

    def load_batch(self, sched: Schedule, tok_job=None, label_job=None, loss_rows: int = 0, exchange_rows=None) -> None:
        # tokens are ignored by a dense-input engine (vocab == 0), labels by a headless one (classes == 0)
        if exchange_rows is not None:
            self.set_exchange_rows(exchange_rows)
        tok_job = np.ascontiguousarray(tok_job, np.int32) if self.cfg.vocab else None
        label_job = np.ascontiguousarray(label_job, np.int32) if self.cfg.classes else None
        assert tok_job is None or tok_job.size >= sched.n_total
        assert label_job is None or label_job.size >= sched.n_total
        check(lib().cavs_treelstm_load_batch(self._h, sched._h, ptr(tok_job), ptr(label_job), loss_rows, _stream()))
        self.n = sched.n_scheduled

    def stage(self, sched: Schedule, parents: np.ndarray, tok_job, label_job, loss_rows: int = 0, exchange_rows=None) -> None:
        """Level scheduling of `parents` into `sched` and the upload of the batch's tables, in one C call."""
        assert parents.dtype == np.int32 and parents.flags.c_contiguous
        if exchange_rows is not None:
            self.set_exchange_rows(exchange_rows)
        check(lib().cavs_treelstm_stage(self._h, sched._h, ptr(parents), parents.shape[0], parents.shape[1],
                                        ptr(tok_job) if self.cfg.vocab else ptr(None), ptr(label_job) if self.cfg.classes else ptr(None),
                                        loss_rows))
        sched._refresh()
        self.n = sched.n_scheduled

    def stage_async(self, sched: Schedule, parents: np.ndarray, tok_job, label_job, loss_rows: int = 0, exchange_rows=None) -> None:
        """stage() on the engine's helper thread: returns at once; the next step() / forward() waits for it.  The arrays
        are kept alive here until then."""
        # parents None: `sched` was loaded by the caller (Schedule.load, possibly on another thread); only the packing runs
        assert parents is None or (parents.dtype == np.int32 and parents.flags.c_contiguous)
        if exchange_rows is not None:
            self.set_exchange_rows(exchange_rows)      # copied by the library before it returns
        self._staging = (sched, parents, tok_job, label_job)
        check(lib().cavs_treelstm_stage_async(self._h, sched._h, ptr(parents), parents.shape[0] if parents is not None else 0,
                                              parents.shape[1] if parents is not None else 0,
                                              ptr(tok_job) if self.cfg.vocab else ptr(None),
                                              ptr(label_job) if self.cfg.classes else ptr(None), loss_rows))

    def promote(self) -> None:
        """Join a staging request in flight and make the staged batch current; from then on forward() / step() run the
        batch last promoted, so the next batch can be staged while this one's step is being enqueued."""
        check(lib().cavs_treelstm_promote(self._h, _stream()))
        if getattr(self, "_staging", None) is not None:
            self._staging[0]._refresh()
            self.n = self._staging[0].n_scheduled

    def stage_wait(self) -> None:
        check(lib().cavs_treelstm_stage_wait(self._h))
        if getattr(self, "_staging", None) is not None:
            self._staging[0]._refresh()
            self.n = self._staging[0].n_scheduled

    OPT_NONE, OPT_SGD, OPT_ADAGRAD = 0, 1, 2

    def step(self, comm=None, optimizer: int = 0, opt_state: torch.Tensor | None = None, lr: float = 0.0, eps: float = 1e-10) -> None:
        """forward + backward + gradient sum over the ranks of `comm` + parameter update, one C call."""
        check(lib().cavs_treelstm_step(self._h, comm._h if comm is not None else ctypes.c_void_p(0), optimizer,
                                       ctypes.c_void_p(opt_state.data_ptr() if opt_state is not None else 0),
                                       ctypes.c_float(lr), ctypes.c_float(eps), _stream()))

    def forward(self) -> None:
        check(lib().cavs_treelstm_forward(self._h, _stream()))

    def backward(self) -> None:
        check(lib().cavs_treelstm_backward(self._h, _stream()))

    def device_view(self, what: int, shape) -> torch.Tensor:
        """A float32 view of one of the engine's arrays (cavs_treelstm_peek) inside its workspace tensor."""
        p, nbytes = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().cavs_treelstm_peek(self._h, what, ctypes.byref(p), ctypes.byref(nbytes)))
        off = p.value - self.workspace.data_ptr()
        return self.workspace[off:off + nbytes.value].view(torch.float32).view(*shape)

    def set_dense_input(self, x: torch.Tensor) -> None:
        """x: float32 device rows [n, embed] (any row pitch), e.g. the h columns of the layer below."""
        assert x.dtype == torch.float32 and x.stride(1) == 1
        self._x_keep = x
        check(lib().cavs_treelstm_set_dense_input(self._h, ctypes.c_void_p(x.data_ptr()), ctypes.c_longlong(x.stride(0))))

    def set_output_grad(self, dh: torch.Tensor) -> None:
        """dh: dense float32 device rows [n, hidden], e.g. d(x) of the layer above."""
        assert dh.dtype == torch.float32 and dh.is_contiguous()
        self._dh_keep = dh
        check(lib().cavs_treelstm_set_output_grad(self._h, ctypes.c_void_p(dh.data_ptr())))

    def upload_bytes(self) -> int:
        """Bytes of index tables the last load_batch() sent to the device."""
        fn = lib().cavs_treelstm_upload_bytes
        fn.restype = ctypes.c_size_t
        return int(fn(self._h))

    def wait_embed_grad(self, stream) -> None:
        """Makes `stream` (a torch.cuda.Stream) wait for the embedding-gradient block of the last backward()."""
        check(lib().cavs_treelstm_wait_embed_grad(self._h, ctypes.c_void_p(stream.cuda_stream)))

    def read_loss(self) -> float:
        out = ctypes.c_float()
        status = ctypes.c_int()
        check(lib().cavs_treelstm_read_loss(self._h, ctypes.byref(out), ctypes.byref(status), _stream()))
        return out.value

    def sgd(self, lr: float) -> None:
        check(lib().cavs_sgd(ctypes.c_void_p(self.params.data_ptr()), ctypes.c_void_p(self.grads.data_ptr()),
                             ctypes.c_size_t(self.params.numel()), ctypes.c_float(lr), _stream()))
        self.refresh_weights()

    def adagrad(self, acc: torch.Tensor, lr: float, eps: float = 1e-10) -> None:
        check(lib().cavs_adagrad(ctypes.c_void_p(self.params.data_ptr()), ctypes.c_void_p(acc.data_ptr()),
                                 ctypes.c_void_p(self.grads.data_ptr()), ctypes.c_size_t(self.params.numel()),
                                 ctypes.c_float(lr), ctypes.c_float(eps), _stream()))
        self.refresh_weights()

    def peek(self, what: int, shape) -> np.ndarray:
        p = ctypes.c_void_p()
        nbytes = ctypes.c_size_t()
        check(lib().cavs_treelstm_peek(self._h, what, ctypes.byref(p), ctypes.byref(nbytes)))
        off = p.value - self.workspace.data_ptr()
        t = self.workspace[off:off + nbytes.value].view(torch.float32)
        torch.cuda.synchronize()
        return t.cpu().numpy().reshape(shape)

    def state(self) -> np.ndarray:
        check(lib().cavs_treelstm_materialize_state(self._h, _stream()))   # leaf rows may live per token
        return self.peek(0, (self.n, 2 * self.cfg.hidden))

    def loss_rows(self) -> np.ndarray:
        check(lib().cavs_treelstm_materialize_state(self._h, _stream()))   # leaf losses may live per token
        return self.peek(1, (self.n,))

    def grad_dict(self) -> dict:
        torch.cuda.synchronize()
        g = self.grads.cpu().numpy()
        return {"d" + k: g[self.offsets[k]:self.offsets[k] + self.sizes[k]].copy() for k in self.PARAM_NAMES}
