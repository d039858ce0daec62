"""The allocation-free loss head (cavs_fc_softmax_xent_static) against the regular entry point.

Some callers of this library must not allocate device memory at all: a host that has handed the
whole GPU to its own pool, or a step loop where cudaMalloc / cudaFree are off limits because they
stall the device.  For them the loss head keeps its partial-sum buffer inside the library.  This
test calls it through the C ABI twice in a row (the buffer is shared between calls and keeps the
previous call's contents) and compares every output with cavs_fc_softmax_xent given caller scratch,
and the second call's outputs also with a float64 restatement of the reference's loss head, so that a
fault shared by both entry points cannot pass.
Collected last so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

from cavs_b200 import CavsError, check, lib
from helpers import assert_close, loss_head_reference

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _run(cuda, entry, rows, H, C, seed, with_scratch):
    g = torch.Generator(device="cpu").manual_seed(seed)
    state = torch.randn((rows, 2 * H), generator=g).to(cuda)                  # h is the first half of each row
    label = torch.randint(-1, C, (rows,), generator=g, dtype=torch.int32).to(cuda)   # -1: row without a loss term
    Wc = (torch.randn((C, H), generator=g) * 0.1).to(cuda)
    bc = (torch.randn((C,), generator=g) * 0.1).to(cuda)
    out = dict(loss=torch.full((rows,), 7.0, device=cuda), loss_sum=torch.full((4,), 7.0, device=cuda),
               dH=torch.full((rows, H), 7.0, device=cuda), dWc=torch.full((C, H), 7.0, device=cuda),
               dbc=torch.full((C,), 7.0, device=cuda))
    L = lib()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [_p(out["loss"]), _p(out["loss_sum"]), _p(out["dH"]), _p(out["dWc"]), _p(out["dbc"]), _p(state),
            ctypes.c_longlong(2 * H), _p(label), _p(Wc), _p(bc), rows, H, C, ctypes.c_float(1.0 / rows)]
    if with_scratch:
        L.cavs_fc_softmax_xent_scratch_bytes.restype = ctypes.c_size_t
        scratch = torch.empty(L.cavs_fc_softmax_xent_scratch_bytes(H, C), dtype=torch.uint8, device=cuda)
        args.append(_p(scratch))
    check(getattr(L, entry)(*args, st))
    torch.cuda.synchronize()
    out["loss_sum"] = out["loss_sum"][:1]
    ref = loss_head_reference(state[:, :H].cpu().numpy(), label.cpu().numpy(), Wc.cpu().numpy(), bc.cpu().numpy(), 1.0 / rows)
    return {k: v.cpu() for k, v in out.items()}, ref


@pytest.mark.parametrize("rows,H,C", [(3000, 1024, 5), (777, 152, 3)])
def test_static_scratch_matches_caller_scratch_twice_in_a_row(cuda, rows, H, C):
    for call in range(2):                       # second call sees the first call's leftovers in the array
        seed = 100 * call + rows
        want, _ = _run(cuda, "cavs_fc_softmax_xent", rows, H, C, seed, with_scratch=True)
        got, ref = _run(cuda, "cavs_fc_softmax_xent_static", rows, H, C, seed, with_scratch=False)
        for k in ref:
            assert_close(got[k].numpy(), ref[k], 1e-5, f"call {call}: {k} against float64")
        for k in want:
            # same kernel, same grid, same reduction order: the tolerance of the other loss-head
            # checks (1e-5 relative) is kept although the results are expected to be identical
            scale = want[k].abs().max().clamp(min=1e-30)
            assert ((got[k] - want[k]).abs().max() / scale).item() <= 1e-5, (call, k)


def test_static_scratch_rejects_shapes_beyond_its_capacity(cuda):
    with pytest.raises(CavsError) as e:
        _run(cuda, "cavs_fc_softmax_xent_static", 64, 2048, 8, 1, with_scratch=False)
    assert e.value.status == 3 and "exceeds the built-in scratch" in str(e.value)
