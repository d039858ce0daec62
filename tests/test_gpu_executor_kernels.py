"""The kernels the op-by-op executor adds to the C ABI, each against numpy on the same inputs:
strided row copies (bit-exact), |x| sum, fill, axpy, and gradient clipping as Sym::Optimizer(vars, lr, clip) defines it
(cavs/backend/op_impl_clip.cu:25-45, cavs/midend/graph_util.cc:209-225)."""
import ctypes

import numpy as np
import pytest
import torch

from cavs_b200 import check, lib

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _st():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("rows,width,dst_pitch,src_pitch", [
    (257, 64, 256, 64),      # Concat: narrow source into a column range of wider rows
    (257, 64, 64, 256),      # Slice: column range of wider rows into a dense array
    (1000, 150, 600, 150),   # config-2 sized, width not a multiple of 4 floats -> scalar path
    (33, 1, 7, 3),           # one float per row, odd pitches
    (0, 16, 16, 16),         # empty level
])
@pytest.mark.parametrize("accumulate", [0, 1])
def test_copy_rows_2d_views_bit_exact(cuda, rows, width, dst_pitch, src_pitch, accumulate):
    rng = np.random.default_rng(rows * 31 + width + accumulate)
    n_dst, n_src = max(rows, 1) + 5, max(rows, 1) + 3
    dst = rng.standard_normal((n_dst, dst_pitch)).astype(np.float32)
    src = rng.standard_normal((n_src, src_pitch)).astype(np.float32)
    dcol, scol = dst_pitch - width, (src_pitch - width) // 2     # views that start inside the row
    dst_ids = rng.permutation(n_dst)[:rows].astype(np.int32)       # distinct targets
    src_ids = rng.integers(0, n_src, rows).astype(np.int32)
    if rows > 4:
        src_ids[1] = -1       # a negative source row reads zeros
        dst_ids[3] = -1       # a negative target row is skipped
    want = dst.copy()
    for b in range(rows):
        if dst_ids[b] < 0:
            continue
        row = src[src_ids[b], scol:scol + width] if src_ids[b] >= 0 else np.zeros(width, np.float32)
        if accumulate:
            want[dst_ids[b], dcol:dcol + width] += row
        else:
            want[dst_ids[b], dcol:dcol + width] = row
    d_dst, d_src = _dev(dst, cuda), _dev(src, cuda)
    d_di = _dev(dst_ids if rows else np.zeros(1, np.int32), cuda)
    d_si = _dev(src_ids if rows else np.zeros(1, np.int32), cuda)
    check(lib().cavs_copy_rows_2d(
        ctypes.c_void_p(d_dst.data_ptr() + 4 * dcol), ctypes.c_longlong(dst_pitch), _p(d_di),
        ctypes.c_void_p(d_src.data_ptr() + 4 * scol), ctypes.c_longlong(src_pitch), _p(d_si),
        rows, width, accumulate, _st()))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(d_dst.cpu().numpy()), _bits(want))


def test_copy_rows_2d_null_index_lists_mean_identity(cuda):
    rng = np.random.default_rng(5)
    src = rng.standard_normal((40, 96)).astype(np.float32)
    d_src = _dev(src, cuda)
    d_dst = torch.zeros((40, 32), dtype=torch.float32, device=cuda)
    check(lib().cavs_copy_rows_2d(_p(d_dst), ctypes.c_longlong(32), _p(None),
                                  ctypes.c_void_p(d_src.data_ptr() + 4 * 32), ctypes.c_longlong(96), _p(None),
                                  40, 32, 0, _st()))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(d_dst.cpu().numpy()), _bits(src[:, 32:64]))


@pytest.mark.parametrize("count", [1, 1023, 1024, 150 * 1000 + 7, 5_000_000])
def test_abs_sum_fill_axpy(cuda, count):
    rng = np.random.default_rng(count)
    x = rng.standard_normal(count).astype(np.float32)
    d_x = _dev(x, cuda)
    d_out = torch.zeros(1, dtype=torch.float32, device=cuda)
    d_scr = torch.empty(1024, dtype=torch.float32, device=cuda)
    got = []
    for _ in range(2):          # fixed reduction order: two launches give the same bits
        check(lib().cavs_abs_sum(_p(d_out), _p(d_x), ctypes.c_size_t(count), _p(d_scr), _st()))
        got.append(float(d_out.cpu()[0]))
    assert got[0] == got[1]
    want = float(np.abs(x.astype(np.float64)).sum())
    assert abs(got[0] - want) <= 2e-6 * want

    check(lib().cavs_fill(_p(d_x), ctypes.c_size_t(count), ctypes.c_float(1.0), _st()))
    assert (d_x.cpu().numpy() == 1.0).all()

    y = rng.standard_normal(count).astype(np.float32)
    d_y, d_x2 = _dev(y, cuda), _dev(x, cuda)
    check(lib().cavs_axpy(_p(d_y), _p(d_x2), ctypes.c_size_t(count), ctypes.c_float(-0.25), _st()))
    # -0.25 * x is exact, so one rounding per element: the same bits as numpy's fp32 arithmetic
    assert np.array_equal(_bits(d_y.cpu().numpy()), _bits(y + np.float32(-0.25) * x))


@pytest.mark.parametrize("scale,clip", [(1.0, 5.0), (0.001, 5.0), (3.0, 0.5)])
def test_clip_gradients_sum_of_block_norms(cuda, scale, clip):
    rng = np.random.default_rng(11)
    sizes = [150 * 600, 600, 1, 300 * 600, 5, 21701 * 8]
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.uint64)
    g = (rng.standard_normal(int(offs[-1])) * scale).astype(np.float32)
    s = sum(float(np.sqrt((g[int(a):int(b)].astype(np.float64) ** 2).sum())) for a, b in zip(offs[:-1], offs[1:]))
    factor = clip / max(s, clip)
    want = g.astype(np.float64) * factor
    d_g = _dev(g, cuda)
    lib().cavs_clip_gradients_scratch_bytes.restype = ctypes.c_size_t
    nbytes = lib().cavs_clip_gradients_scratch_bytes(len(sizes))
    assert nbytes > 0
    d_scr = torch.empty((nbytes + 7) // 8, dtype=torch.float64, device=cuda)     # 8-byte aligned
    check(lib().cavs_clip_gradients(_p(d_g), offs.ctypes.data_as(ctypes.c_void_p), len(sizes), ctypes.c_float(clip),
                                    _p(d_scr), _st()))
    torch.cuda.synchronize()
    got = d_g.cpu().numpy().astype(np.float64)
    if s <= clip:
        assert np.array_equal(_bits(d_g.cpu().numpy()), _bits(g))      # factor is exactly 1
    else:
        assert np.abs(got - want).max() <= 4e-6 * np.abs(want).max()
    # the clipped gradient's own norm sum is at most clip (up to rounding)
    s2 = sum(float(np.sqrt((got[int(a):int(b)] ** 2).sum())) for a, b in zip(offs[:-1], offs[1:]))
    assert s2 <= clip * (1 + 1e-5)
