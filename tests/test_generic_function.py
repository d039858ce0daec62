"""Vertex functions other than the fused LSTM forms (the reference's Tree-FC app, a Tree-FC with inputs, a gated cell on
tokens) declared through Sym / GraphSupport::Node() and run by Session::Run operator by operator, with their elementwise
groups compiled at run time.  The C++ executable runs them on the device and writes everything to a file; this test
recomputes outputs, losses and gradients with float64 PyTorch autograd -- the reference's loss semantics included: a
Reduce_sum loss is a sum of absolute values whose gradient is a fill with ones, the cross-entropy gradient is divided by
the row count, clipping scales by clip / max(sum of the per-variable L2 norms, clip) -- and compares at 1e-5 relative."""
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest

BIN = Path(__file__).parent / "cpp" / "bin" / "generic_fn_test"


def _exe():
    if not BIN.exists():
        import __graft_entry__ as g
        g.build()
    return BIN


def test_planning_and_runtime_compilation_cpu():
    """Plans both vertex functions and compiles their generated kernels for sm_100a (needs no GPU)."""
    r = subprocess.run([str(_exe()), "cpu"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ok" in r.stdout


def _read(path):
    out = {}
    raw = Path(path).read_bytes()
    pos = 0
    while pos < len(raw):
        kind = raw[pos:pos + 1].decode(); pos += 1
        (ln,) = struct.unpack_from("<i", raw, pos); pos += 4
        name = raw[pos:pos + ln].decode(); pos += ln
        (cnt,) = struct.unpack_from("<Q", raw, pos); pos += 8
        out[name] = np.frombuffer(raw, dtype=np.float32 if kind == "f" else np.int32, count=cnt, offset=pos).copy()
        pos += 4 * cnt
    return out


@pytest.mark.gpu
def test_generic_vertex_functions_against_autograd(cuda, tmp_path):
    import torch
    import oracle
    from helpers import assert_close
    path = tmp_path / "generic.bin"
    r = subprocess.run([str(_exe()), "gpu", str(path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    d = _read(path)
    B, L, H, E, V, C = (int(x) for x in d["dims"])
    parents = d["parents"].reshape(B, L)
    tb = oracle.tables(parents, 2, 0)
    n, fg, t2j, lo = int(tb["n"]), tb["fg"], tb["t2j"], tb["level_off"]
    f64 = lambda a, *shape: torch.tensor(np.asarray(a, np.float64).reshape(*shape), requires_grad=True)

    # ---- Tree-FC with inputs ----
    W, Wx, b = f64(d["fc.W"], 2 * H, H), f64(d["fc.Wx"], E, H), f64(d["fc.b"], H)
    half = torch.tensor([0.5], dtype=torch.float64, requires_grad=True)
    x = torch.tensor(d["fc.x"].astype(np.float64).reshape(n, E))
    res = [None] * n
    zero = torch.zeros(H, dtype=torch.float64)
    for t in range(n):
        left = res[fg[0][t]] if fg[0][t] >= 0 else zero
        right = res[fg[1][t]] if fg[1][t] >= 0 else zero
        res[t] = torch.relu(torch.cat([left, right]) @ W + x[t2j[t]] @ Wx + b) - (left * right) * half
    out = torch.stack(res)
    out.sum().backward()                                      # the gradient of Reduce_sum is a fill with ones
    lr, clip = (float(v) for v in d["fc.lr_clip"])
    grads = [W.grad, Wx.grad, b.grad, half.grad]
    scale = clip / max(sum(float(g.norm()) for g in grads), clip)
    got_out = d["fc.out"].reshape(n, H)
    want_out = np.zeros((n, H))
    want_out[t2j] = out.detach().numpy()                      # fetched in job order
    assert_close(got_out, want_out, 1e-5, "Tree-FC output")
    want_loss = float(out.detach().abs().sum())
    assert abs(float(d["fc.loss"][0]) - want_loss) <= 1e-5 * want_loss
    for name, g in zip(("fc.gW", "fc.gWx", "fc.gb", "fc.ghalf"), grads):
        assert_close(d[name], (scale * g).numpy().ravel(), 1e-5, name)
    for name, w, g in (("fc.W1", W, W.grad), ("fc.Wx1", Wx, Wx.grad), ("fc.b1", b, b.grad)):
        assert_close(d[name], (w - lr * scale * g).detach().numpy().ravel(), 1e-5, name)

    # ---- gated cell on tokens with a softmax head ----
    table, Wx, Wh = f64(d["gc.table"], V, E), f64(d["gc.Wx"], E, 3 * H), f64(d["gc.Wh"], H, 3 * H)
    bias, wc, bc = f64(d["gc.bias"], 3 * H), f64(d["gc.wc"], C, H), f64(d["gc.bc"], C)
    tok, lab = d["gc.tok"].astype(np.int64), d["gc.lab"].astype(np.int64)
    hs, cs = [None] * n, [None] * n
    for t in range(n):
        hl, cl = (hs[fg[0][t]], cs[fg[0][t]]) if fg[0][t] >= 0 else (zero, zero)
        hr, cr = (hs[fg[1][t]], cs[fg[1][t]]) if fg[1][t] >= 0 else (zero, zero)
        pre = table[tok[t2j[t]]] @ Wx + (hl + hr) @ Wh + bias
        z, g, u = torch.sigmoid(pre[:H]), torch.sigmoid(pre[H:2 * H]), torch.tanh(pre[2 * H:])
        cs[t] = z * u + g * (cl + cr)
        hs[t] = torch.tanh(cs[t]) * z
    hout = torch.stack(hs)
    logp = torch.log_softmax(hout @ wc.t() + bc, dim=1)
    loss_rows = -logp[torch.arange(n), torch.tensor(lab[t2j])]
    (loss_rows.sum() / n).backward()
    want = np.zeros(n); want[t2j] = loss_rows.detach().numpy()
    assert_close(d["gc.loss"], want, 1e-5, "gated cell loss")
    want_h = np.zeros((n, H)); want_h[t2j] = hout.detach().numpy()
    assert_close(d["gc.out"].reshape(n, H), want_h, 1e-5, "gated cell output")
    for name, p in (("gc.gtable", table), ("gc.gWx", Wx), ("gc.gWh", Wh), ("gc.gbias", bias), ("gc.gwc", wc), ("gc.gbc", bc)):
        assert_close(d[name], p.grad.numpy().ravel(), 1e-5, name)
