"""PyTorch-CPU restatement of the child-sum Tree-LSTM vertex function with autograd,
used only to cross-check the C oracle (secondary oracle; float64 capable)."""
from __future__ import annotations

import numpy as np
import torch


def treelstm_autograd(tb, tok, label, params, H, E, V, C, K=2, dtype=torch.float64, loss_rows=0):
    """Aligned tables only.  Returns dict with state, loss and gradients as numpy arrays."""
    n = int(tb["n"])
    P = {k: torch.tensor(np.asarray(v), dtype=dtype, requires_grad=True) for k, v in params.items()}
    Emb, W, U, B, Wc, bc = (P[k] for k in ("Emb", "W", "U", "B", "Wc", "bc"))
    U_iou = U[: 3 * H * H].reshape(H, 3 * H)
    U_f = U[3 * H * H:].reshape(H, H)
    b_i, b_f, b_u, b_o = B[:H], B[H:2 * H], B[2 * H:3 * H], B[3 * H:]
    tok_t = torch.tensor(np.asarray(tok), dtype=torch.long)
    x = Emb[tok_t]
    a = x @ W.reshape(E, 4 * H)
    hs = [None] * n
    cs = [None] * n
    zero = torch.zeros(H, dtype=dtype)
    lo = tb["level_off"]
    fg = tb["fg"]
    for l in range(int(tb["n_levels"])):
        for t in range(int(lo[l]), int(lo[l + 1])):
            hk = [hs[int(fg[c][t])] if fg[c][t] >= 0 else zero for c in range(K)]
            ck = [cs[int(fg[c][t])] if fg[c][t] >= 0 else zero for c in range(K)]
            s = sum(hk[1:], hk[0])
            p = s @ U_iou
            i = torch.sigmoid(a[t, :H] + p[:H] + b_i)
            o = torch.sigmoid(a[t, H:2 * H] + p[H:2 * H] + b_o)
            u = torch.tanh(a[t, 2 * H:3 * H] + p[2 * H:] + b_u)
            c_new = i * u
            for c in range(K):
                f = torch.sigmoid(a[t, 3 * H:] + hk[c] @ U_f + b_f)
                c_new = c_new + f * ck[c]
            hs[t] = o * torch.tanh(c_new)
            cs[t] = c_new
    Hout = torch.stack(hs)
    z = Hout @ Wc.t() + bc
    lab = torch.tensor(np.asarray(label), dtype=torch.long)
    mask = lab >= 0
    logp = torch.log_softmax(z, dim=1)
    loss_rows_v = -logp[torch.arange(n), lab.clamp(min=0)] * mask
    rows = loss_rows if loss_rows > 0 else n
    (loss_rows_v.sum() / rows).backward()
    out = dict(state=torch.cat([Hout, torch.stack(cs)], dim=1).detach().numpy(), loss=loss_rows_v.detach().numpy())
    for k in ("Emb", "W", "U", "B", "Wc", "bc"):
        g = P[k].grad
        out["d" + k] = (g if g is not None else torch.zeros_like(P[k])).numpy()
    return out


def treegru_autograd(tb, tok, label, params, H, E, V, C, K=4, dtype=torch.float64, loss_rows=0):
    """Child-sum Tree-GRU (r_k per child, update gate on the child sum) with autograd; aligned tables only."""
    n = int(tb["n"])
    P = {k: torch.tensor(np.asarray(v), dtype=dtype, requires_grad=True) for k, v in params.items()}
    Emb, W, U, B, Wc, bc = (P[k] for k in ("Emb", "W", "U", "B", "Wc", "bc"))
    U_r, U_z, U_n = (U[i * H * H:(i + 1) * H * H].reshape(H, H) for i in range(3))
    b_r, b_z, b_n = B[:H], B[H:2 * H], B[2 * H:]
    a = Emb[torch.tensor(np.asarray(tok), dtype=torch.long)] @ W.reshape(E, 3 * H)
    hs = [None] * n
    zero = torch.zeros(H, dtype=dtype)
    lo, fg = tb["level_off"], tb["fg"]
    for l in range(int(tb["n_levels"])):
        for t in range(int(lo[l]), int(lo[l + 1])):
            hk = [hs[int(fg[c][t])] if fg[c][t] >= 0 else zero for c in range(K)]
            ht = sum(hk[1:], hk[0])
            m = sum(torch.sigmoid(a[t, :H] + h @ U_r + b_r) * h for h in hk)
            z = torch.sigmoid(a[t, H:2 * H] + ht @ U_z + b_z)
            g = torch.tanh(a[t, 2 * H:] + m @ U_n + b_n)
            hs[t] = (1 - z) * ht + z * g
    Hout = torch.stack(hs)
    logits = Hout @ Wc.t() + bc
    lab = torch.tensor(np.asarray(label), dtype=torch.long)
    mask = lab >= 0
    logp = torch.log_softmax(logits, dim=1)
    loss_rows_v = -logp[torch.arange(n), lab.clamp(min=0)] * mask
    rows = loss_rows if loss_rows > 0 else n
    (loss_rows_v.sum() / rows).backward()
    out = dict(state=Hout.detach().numpy(), loss=loss_rows_v.detach().numpy())
    for k in ("Emb", "W", "U", "B", "Wc", "bc"):
        g_ = P[k].grad
        out["d" + k] = (g_ if g_ is not None else torch.zeros_like(P[k])).numpy()
    return out


def stacked_lstm_autograd(tb, tok, label, layers, dims, V, C, K=1, dtype=torch.float64, loss_rows=0):
    """A stack of child-sum LSTM layers over one graph: layer 0 reads Emb[tok], layer i > 0 reads the h of
    layer i-1, the loss head sits on the last layer.  layers: list of parameter dicts (layer 0 holds Emb, the
    last one Wc and bc); dims: list of (H, E) per layer.  Returns per-layer dicts of state and gradients, and
    the per-vertex loss."""
    n = int(tb["n"])
    P = [{k: torch.tensor(np.asarray(v), dtype=dtype, requires_grad=True) for k, v in lp.items()} for lp in layers]
    lo, fg = tb["level_off"], tb["fg"]
    x = P[0]["Emb"][torch.tensor(np.asarray(tok), dtype=torch.long)]
    states = []
    for li, (H, E) in enumerate(dims):
        W, U, B = P[li]["W"], P[li]["U"], P[li]["B"]
        U_iou, U_f = U[: 3 * H * H].reshape(H, 3 * H), U[3 * H * H:].reshape(H, H)
        b_i, b_f, b_u, b_o = B[:H], B[H:2 * H], B[2 * H:3 * H], B[3 * H:]
        a = x @ W.reshape(E, 4 * H)
        hs, cs, zero = [None] * n, [None] * n, torch.zeros(H, dtype=dtype)
        for l in range(int(tb["n_levels"])):
            for t in range(int(lo[l]), int(lo[l + 1])):
                hk = [hs[int(fg[c][t])] if fg[c][t] >= 0 else zero for c in range(K)]
                ck = [cs[int(fg[c][t])] if fg[c][t] >= 0 else zero for c in range(K)]
                p = sum(hk[1:], hk[0]) @ U_iou
                i = torch.sigmoid(a[t, :H] + p[:H] + b_i)
                o = torch.sigmoid(a[t, H:2 * H] + p[H:2 * H] + b_o)
                u = torch.tanh(a[t, 2 * H:3 * H] + p[2 * H:] + b_u)
                c_new = i * u
                for c in range(K):
                    c_new = c_new + torch.sigmoid(a[t, 3 * H:] + hk[c] @ U_f + b_f) * ck[c]
                hs[t], cs[t] = o * torch.tanh(c_new), c_new
        x = torch.stack(hs)
        states.append(torch.cat([x, torch.stack(cs)], dim=1))
    z = x @ P[-1]["Wc"].t() + P[-1]["bc"]
    lab = torch.tensor(np.asarray(label), dtype=torch.long)
    logp = torch.log_softmax(z, dim=1)
    loss_v = -logp[torch.arange(n), lab.clamp(min=0)] * (lab >= 0)
    (loss_v.sum() / (loss_rows if loss_rows > 0 else n)).backward()
    outs = []
    for li in range(len(dims)):
        o = dict(state=states[li].detach().numpy())
        for k, v in P[li].items():
            o["d" + k] = (v.grad if v.grad is not None else torch.zeros_like(v)).numpy()
        outs.append(o)
    return outs, loss_v.detach().numpy()
