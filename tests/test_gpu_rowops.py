"""Row gather / scatter / zero through the C ABI vs the oracle's row ops: bit-exact."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from cavs_b200 import check, lib

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _st():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("rows,n_ids,width", [
    (64, 64, 300),        # 1200-byte rows (config 2: 2*150 floats), 16-byte path
    (1000, 777, 2048),    # 8 KB rows (config 5: 2*1024 floats)
    (50, 31, 75),         # 300-byte rows: not a multiple of 16 -> word path
    (5, 1, 4),
    (3, 0, 16),           # empty id list
])
def test_gather_scatter_bit_exact(cuda, rows, n_ids, width):
    rng = np.random.default_rng(rows * 7 + width)
    inp = rng.standard_normal((rows, width)).astype(np.float32)
    ids = rng.integers(0, rows, n_ids).astype(np.int32)
    want = np.zeros((max(n_ids, 1), width), np.float32)
    oracle.oracle_lib().cavs_oracle_gather_rows(oracle._p(want), oracle._p(inp), oracle._p(ids), n_ids, width)
    d_inp, d_ids = _dev(inp, cuda), _dev(ids if n_ids else np.zeros(1, np.int32), cuda)
    d_out = torch.zeros((max(n_ids, 1), width), dtype=torch.float32, device=cuda)
    check(lib().cavs_gather_rows(_p(d_out), _p(d_inp), _p(d_ids), n_ids, ctypes.c_size_t(width * 4), _st()))
    torch.cuda.synchronize()
    assert np.array_equal(d_out.cpu().numpy().view(np.uint32), want.view(np.uint32))

    # scatter: distinct targets (one mailbox row per vertex)
    tgt = rng.permutation(rows)[:n_ids].astype(np.int32)
    src = rng.standard_normal((max(n_ids, 1), width)).astype(np.float32)
    base = rng.standard_normal((rows, width)).astype(np.float32)
    want2 = base.copy()
    oracle.oracle_lib().cavs_oracle_scatter_rows(oracle._p(want2), oracle._p(tgt), oracle._p(src), n_ids, width)
    d_dst, d_src, d_tgt = _dev(base, cuda), _dev(src, cuda), _dev(tgt if n_ids else np.zeros(1, np.int32), cuda)
    check(lib().cavs_scatter_rows(_p(d_dst), _p(d_tgt), _p(d_src), n_ids, ctypes.c_size_t(width * 4), _st()))
    torch.cuda.synchronize()
    assert np.array_equal(d_dst.cpu().numpy().view(np.uint32), want2.view(np.uint32))


def test_negative_ids_extension_and_zero_rows(cuda):
    inp = np.arange(40, dtype=np.float32).reshape(5, 8)
    ids = np.array([3, -1, 0], np.int32)
    d_out = torch.full((3, 8), 7.0, device=cuda)
    d_inp, d_ids = _dev(inp, cuda), _dev(ids, cuda)     # keep the device buffers alive across the launch
    check(lib().cavs_gather_rows(_p(d_out), _p(d_inp), _p(d_ids), 3, ctypes.c_size_t(32), _st()))
    got = d_out.cpu().numpy()
    assert np.array_equal(got[0], inp[3]) and not got[1].any() and np.array_equal(got[2], inp[0])
    d_dst = torch.full((5, 8), 9.0, device=cuda)
    d_src = _dev(inp[:3], cuda)
    check(lib().cavs_scatter_rows(_p(d_dst), _p(d_ids), _p(d_src), 3, ctypes.c_size_t(32), _st()))
    got = d_dst.cpu().numpy()
    assert np.array_equal(got[3], inp[0]) and np.array_equal(got[0], inp[2]) and (got[[1, 2, 4]] == 9.0).all()
    # zero-fill clears the first n rows whatever the ids were (functor_batched_memcpy.cuh:64-75)
    d_z = torch.full((6, 75), 1.0, device=cuda)
    check(lib().cavs_zero_rows(_p(d_z), 4, ctypes.c_size_t(300), _st()))
    got = d_z.cpu().numpy()
    assert not got[:4].any() and (got[4:] == 1.0).all()


def test_full_size_roundtrip_property(cuda):
    # config-5 sized mailbox slice: scatter by a permutation then gather by it is the identity.
    rows, width = 66000, 2048
    g = torch.Generator(device="cpu").manual_seed(1)
    perm = torch.randperm(rows, generator=g).to(torch.int32).to(cuda)
    src = torch.randn((rows, width), device=cuda)
    mail = torch.empty_like(src)
    back = torch.empty_like(src)
    check(lib().cavs_scatter_rows(_p(mail), _p(perm), _p(src), rows, ctypes.c_size_t(width * 4), _st()))
    check(lib().cavs_gather_rows(_p(back), _p(mail), _p(perm), rows, ctypes.c_size_t(width * 4), _st()))
    torch.cuda.synchronize()
    assert torch.equal(back, src)
    assert torch.equal(mail[perm.long()], src)
