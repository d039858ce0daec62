"""The loss head's C-ABI entries that write d(hidden) -- cavs_fc_softmax_xent (caller scratch) and
cavs_fc_softmax_xent_static (scratch inside the library) -- against a float64 restatement of the reference's
FullyConnected + SoftmaxEntropyLoss and their gradients (helpers.loss_head_reference), 1e-5 relative, checked over
each tensor's max norm and value by value.  Shapes cover all three kernels: the streaming form (hidden a multiple
of 4, at most 1024), the generic form with 128-bit accesses (hidden 2048) and its scalar form (hidden 150, and a
hidden row pitch that breaks 16-byte alignment); a fifth of the rows carries label -1 (no loss term).  The engine
tests elsewhere only use the form that hands d(logits) rows to the cell gradient."""
import ctypes

import numpy as np
import pytest
import torch

from cavs_b200 import check, lib
from helpers import assert_close, loss_head_reference

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _call(cuda, entry, h, pitch, label, Wc, bc, rows, H, C, inv_rows):
    out = dict(loss=torch.full((rows,), 7.0, device=cuda), loss_sum=torch.full((4,), 7.0, device=cuda),
               dH=torch.full((rows, H), 7.0, device=cuda), dWc=torch.full((C, H), 7.0, device=cuda),
               dbc=torch.full((C,), 7.0, device=cuda))
    L = lib()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [_p(out["loss"]), _p(out["loss_sum"]), _p(out["dH"]), _p(out["dWc"]), _p(out["dbc"]), _p(h), ctypes.c_longlong(pitch),
            _p(label), _p(Wc), _p(bc), rows, H, C, ctypes.c_float(inv_rows)]
    if entry == "cavs_fc_softmax_xent":
        L.cavs_fc_softmax_xent_scratch_bytes.restype = ctypes.c_size_t
        scratch = torch.empty(L.cavs_fc_softmax_xent_scratch_bytes(H, C), dtype=torch.uint8, device=cuda)
        args.append(_p(scratch))
    check(getattr(L, entry)(*args, st))
    torch.cuda.synchronize()
    out["loss_sum"] = out["loss_sum"][:1]
    return {k: v.cpu().numpy() for k, v in out.items()}


CASES = [
    # rows, hidden, classes, row pitch of h (floats)
    (3000, 1024, 5, 2048),     # streaming form, h = first half of h|c rows (the engine's layout)
    (777, 152, 3, 304),        # streaming form, small hidden, partial last batch
    (513, 2048, 5, 2048),      # generic form (hidden above 1024), 128-bit accesses
    (333, 150, 4, 150),        # generic form, scalar accesses (hidden not a multiple of 4)
    (200, 64, 8, 65),          # a pitch that is not a multiple of 4 floats: scalar accesses
    (1, 16, 2, 16),            # a single row
]


@pytest.mark.parametrize("rows,H,C,pitch", CASES)
@pytest.mark.parametrize("entry", ["cavs_fc_softmax_xent", "cavs_fc_softmax_xent_static"])
def test_loss_head_with_hidden_gradient_against_float64(cuda, entry, rows, H, C, pitch):
    if entry.endswith("_static") and C * H + C + 1 > 10240:
        pytest.skip("beyond the built-in scratch (rejected: see test_zz_no_alloc.py)")
    g = torch.Generator(device="cpu").manual_seed(rows * 7 + H)
    store = torch.randn((rows, pitch), generator=g)
    label = torch.randint(0, C, (rows,), generator=g, dtype=torch.int32)
    label[torch.rand(rows, generator=g) < 0.2] = -1
    Wc = torch.randn((C, H), generator=g) * 0.1
    bc = torch.randn((C,), generator=g) * 0.1
    inv_rows = 1.0 / max(int((label >= 0).sum()), 1)
    got = _call(cuda, entry, store.to(cuda), pitch, label.to(cuda), Wc.to(cuda), bc.to(cuda), rows, H, C, inv_rows)
    want = loss_head_reference(store[:, :H].numpy(), label.numpy(), Wc.numpy(), bc.numpy(), inv_rows)
    for k in want:
        assert_close(got[k], want[k], 1e-5, f"{entry} {k}")
    # rows without a label: no loss, no gradient
    none = (label < 0).numpy()
    assert not got["loss"][none].any() and not got["dH"][none].any()


def test_loss_head_is_deterministic(cuda):
    rows, H, C = 5000, 512, 5
    g = torch.Generator(device="cpu").manual_seed(3)
    h = torch.randn((rows, H), generator=g).to(cuda)
    label = torch.randint(0, C, (rows,), generator=g, dtype=torch.int32).to(cuda)
    Wc = (torch.randn((C, H), generator=g) * 0.1).to(cuda)
    bc = torch.zeros(C).to(cuda)
    a = _call(cuda, "cavs_fc_softmax_xent", h, H, label, Wc, bc, rows, H, C, 1.0 / rows)
    b = _call(cuda, "cavs_fc_softmax_xent", h, H, label, Wc, bc, rows, H, C, 1.0 / rows)
    for k in a:
        assert np.array_equal(a[k], b[k]), k
