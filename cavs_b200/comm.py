"""Communicator binding (cavs_comm_*): one NCCL communicator per process / GPU, created by the library itself.

The 128-byte NCCL id made by rank 0 has to reach every rank through a channel the host program owns.  `Comm.from_torch`
uses an initialised torch.distributed process group for that one broadcast (any backend: gloo works); `Comm.from_file`
uses a file both ranks can see (single node, no torch).  All collectives afterwards go through the C ABI.
"""
from __future__ import annotations

import ctypes
import os
import time

from ._abi import check, lib

ID_BYTES = 128


class Comm:
    def __init__(self, id_bytes: bytes, rank: int, world: int):
        self.rank, self.world = rank, world
        self._h = ctypes.c_void_p()
        buf = (ctypes.c_char * ID_BYTES).from_buffer_copy(id_bytes)
        check(lib().cavs_comm_create(buf, ctypes.c_size_t(ID_BYTES), rank, world, ctypes.byref(self._h)))

    @staticmethod
    def make_id() -> bytes:
        buf = (ctypes.c_char * ID_BYTES)()
        check(lib().cavs_comm_unique_id(buf, ctypes.c_size_t(ID_BYTES)))
        return bytes(buf)

    @classmethod
    def from_torch(cls, device=None):
        """Rank 0's id is broadcast over the default torch.distributed process group (the current CUDA device must
        already be this rank's)."""
        import torch
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        dev = device if device is not None else (torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else "cpu")
        t = torch.zeros(ID_BYTES, dtype=torch.uint8)
        if rank == 0:
            t = torch.frombuffer(bytearray(cls.make_id()), dtype=torch.uint8).clone()
        t = t.to(dev)
        dist.broadcast(t, 0)
        return cls(bytes(t.cpu().numpy().tobytes()), rank, world)

    @classmethod
    def from_file(cls, path: str, rank: int, world: int, timeout_s: float = 60.0):
        if rank == 0:
            tmp = f"{path}.tmp{os.getpid()}"
            with open(tmp, "wb") as f:
                f.write(cls.make_id())
            os.replace(tmp, path)
        t0 = time.time()
        while not os.path.exists(path) or os.path.getsize(path) < ID_BYTES:
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"no communicator id appeared at {path}")
            time.sleep(0.01)
        with open(path, "rb") as f:
            return cls(f.read(ID_BYTES), rank, world)

    def nccl_version(self) -> int:
        v = ctypes.c_int()
        check(lib().cavs_comm_info(self._h, None, None, ctypes.byref(v)))
        return v.value

    def allreduce(self, t, stream=None) -> None:
        """In-place fp32 sum of a torch CUDA tensor across ranks."""
        import torch
        assert t.dtype == torch.float32 and t.is_contiguous()
        st = ctypes.c_void_p((stream or torch.cuda.current_stream()).cuda_stream)
        check(lib().cavs_allreduce(ctypes.c_void_p(t.data_ptr()), ctypes.c_size_t(t.numel()), self._h, st))

    def broadcast(self, t, root: int = 0) -> None:
        import torch
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib().cavs_broadcast(ctypes.c_void_p(t.data_ptr()), ctypes.c_size_t(t.numel() * t.element_size()), root, self._h, st))

    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib().cavs_comm_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
