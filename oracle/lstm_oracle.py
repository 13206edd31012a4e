"""CPU oracle for the single-layer LSTM hot path (TEST INFRASTRUCTURE ONLY).

This file is a checker, not a product path: only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it.  The shipped
library never falls back to it.

It restates, in plain numpy, the algorithm of the reference project
oleicht/FastLSTM:

* forward cell      -> fastlstm/lstm.py:1087-1105  (naive_lstm_cell_fwd)
* forward sequence  -> fastlstm/lstm.py:1108-1137  (naive_lstm_fwd) and the
                       Triton kernel fastlstm/kernels.py:532-661
* backward cell     -> fastlstm/lstm.py:1140-1192  (naive_lstm_cell_bwd) and the
                       Triton kernel fastlstm/kernels.py:1270-1390
* backward sequence -> fastlstm/lstm.py:1195-1223  (naive_lstm_bwd)
* weight gradients  -> fastlstm/lstm.py:494-501    (Wgrad), :294 (d_x)
* layer stacking    -> fastlstm/lstm.py:664-698    (FastLSTM.forward)

Parity pin: tests/golden/*.npz hold inputs and outputs produced by running
the reference's own pure-PyTorch path (NaiveLSTMfn / naive_lstm_fwd /
naive_lstm_bwd) and torch.nn.LSTM on CPU (generator: tests/golden/make_golden.py);
tests/test_oracle.py checks this restatement against them.

Layout conventions (all row-major):
  x    [T, B, I]      Wx [4H, I]   bx, bh [4H]
  out  [T+1, B, H]    (slot 0 = h0)            Wh [4H, H]
  cell [T+1, B, H]    (slot 0 = c0)
  ifgo [T, B, 4H]     pre-activations, gate order i | f | g | o along 4H
The reference's naive path stores ifgo as [T,B,H,4]; the persistent kernels
store [T,B,4H] (kernels.py:533-536), which is the layout used here.
"""
from __future__ import annotations

import numpy as np


def _sigmoid(v):
    # numerically stable logistic in the array's own dtype
    out = np.empty_like(v)
    pos = v >= 0
    out[pos] = 1.0 / (1.0 + np.exp(-v[pos]))
    e = np.exp(v[~pos])
    out[~pos] = e / (1.0 + e)
    return out


def lstm_cell_fwd(pre, c0):
    """Gate math of one step given the summed pre-activations [B,4H].

    Follows fastlstm/lstm.py:1101-1104 (kernels.py:647-648)."""
    H = c0.shape[-1]
    pi, pf, pg, po = (pre[..., k * H:(k + 1) * H] for k in range(4))
    c1 = _sigmoid(pf) * c0 + _sigmoid(pi) * np.tanh(pg)
    h1 = _sigmoid(po) * np.tanh(c1)
    return h1, c1


def lstm_fwd(x, h0, c0, Wx, bx, Wh, bh):
    """Forward over a sequence; returns (out[T+1], cell[T+1], ifgo[T]).

    Follows fastlstm/lstm.py:31-146 (host) / kernels.py:532-661 (device):
    ifgo~ = x Wx^T + (bx + bh) for all t at once (lstm.py:66-68), then per step
    pre = ifgo~[t] + h[t] Wh^T, stored back as ifgo[t] (kernels.py:631-640)."""
    dt = x.dtype
    T, B, _ = x.shape
    H = Wh.shape[1]
    bias = np.zeros(4 * H, dt)
    if bx is not None:
        bias = bias + bx
    if bh is not None:
        bias = bias + bh
    ifgo = (x.reshape(T * B, -1) @ Wx.T + bias).reshape(T, B, 4 * H).astype(dt)
    out = np.zeros((T + 1, B, H), dt)
    cell = np.zeros((T + 1, B, H), dt)
    if h0 is not None:
        out[0] = h0
        cell[0] = c0
    for t in range(T):
        ifgo[t] += out[t] @ Wh.T
        out[t + 1], cell[t + 1] = lstm_cell_fwd(ifgo[t], cell[t])
    return out, cell, ifgo


def lstm_bwd(dout, dh_n, dc_n, x, out, cell, ifgo, Wx, Wh):
    """Backward over a sequence.

    dout [T,B,H] is the gradient w.r.t. out[1:], dh_n/dc_n [B,H] (or None) the
    gradients w.r.t. the final states.  Returns
    (dx[T,B,I], dh0[B,H], dc0[B,H], dWx[4H,I], dWh[4H,H], db[4H]).
    Per-step equations: fastlstm/kernels.py:1291-1316; recurrent product
    kernels.py:1362-1383; tail GEMMs lstm.py:294,494-501."""
    dt = x.dtype
    T, B, _ = x.shape
    H = Wh.shape[1]
    d_ifgo = np.zeros((T, B, 4 * H), dt)
    dh_carry = np.zeros((B, H), dt) if dh_n is None else dh_n.astype(dt).copy()
    dc = np.zeros((B, H), dt) if dc_n is None else dc_n.astype(dt).copy()
    for t in range(T - 1, -1, -1):
        pi, pf, pg, po = (ifgo[t][:, k * H:(k + 1) * H] for k in range(4))
        c0, c1 = cell[t], cell[t + 1]
        si, sf, so = _sigmoid(pi), _sigmoid(pf), _sigmoid(po)
        tg, tc = np.tanh(pg), np.tanh(c1)
        dh = dout[t] + dh_carry
        dc = dc + dh * so * (1.0 - tc * tc)
        d_ifgo[t][:, 0 * H:1 * H] = dc * tg * si * (1.0 - si)
        d_ifgo[t][:, 1 * H:2 * H] = dc * c0 * sf * (1.0 - sf)
        d_ifgo[t][:, 2 * H:3 * H] = dc * si * (1.0 - tg * tg)
        d_ifgo[t][:, 3 * H:4 * H] = dh * tc * so * (1.0 - so)
        dc = dc * sf
        dh_carry = d_ifgo[t] @ Wh
    dg2 = d_ifgo.reshape(T * B, 4 * H)
    dx = (dg2 @ Wx).reshape(T, B, -1)
    dWx = dg2.T @ x.reshape(T * B, -1)
    dWh = dg2.T @ out[:-1].reshape(T * B, H)
    db = dg2.sum(axis=0)
    return dx, dh_carry, dc, dWx, dWh, db


def stacked_fwd_bwd(x, h0, c0, params, dout=None, dh_n=None, dc_n=None):
    """Multi-layer forward (+ backward when dout is given).

    params: list of (Wx, Wh, bx, bh) per layer; h0/c0 [L,B,H] or None;
    dh_n/dc_n [L,B,H] or None.  Mirrors the sequential layer loop of
    fastlstm/lstm.py:685-698.  Returns a dict of arrays."""
    L = len(params)
    saved = []
    inp = x
    hn, cn = [], []
    for l, (Wx, Wh, bx, bh) in enumerate(params):
        out, cell, ifgo = lstm_fwd(inp, None if h0 is None else h0[l],
                                   None if c0 is None else c0[l], Wx, bx, Wh, bh)
        saved.append((inp, out, cell, ifgo))
        inp = out[1:]
        hn.append(out[-1])
        cn.append(cell[-1])
    res = {"out": inp, "h_n": np.stack(hn), "c_n": np.stack(cn)}
    if dout is None:
        return res
    g = dout
    dh0s, dc0s, grads = [None] * L, [None] * L, [None] * L
    for l in range(L - 1, -1, -1):
        Wx, Wh, bx, bh = params[l]
        xin, out, cell, ifgo = saved[l]
        g, dh0s[l], dc0s[l], dWx, dWh, db = lstm_bwd(
            g, None if dh_n is None else dh_n[l], None if dc_n is None else dc_n[l],
            xin, out, cell, ifgo, Wx, Wh)
        grads[l] = (dWx, dWh, db)
    res.update({"dx": g, "dh0": np.stack(dh0s), "dc0": np.stack(dc0s), "grads": grads})
    return res
