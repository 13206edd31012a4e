"""torch.nn.LSTM on the host cores (TEST INFRASTRUCTURE / CPU BASELINE ONLY).

torch.nn.LSTM in fp32 on CPU is what every test of the reference project
compares against (tests/test_lstm.py:53,120,196 of oleicht/FastLSTM), so it is
used here as the second oracle and as the timed CPU baseline.  Nothing in the
shipped package imports this file.
"""
from __future__ import annotations

import os
import time

import torch
import torch.nn as nn


def make_nn_lstm(params, bias=True, batch_first=False, dtype=torch.float32):
    """Build a CPU nn.LSTM whose weights are the given per-layer tensors.

    params: list of (Wx[4H,I], Wh[4H,H], bx[4H]|None, bh[4H]|None)."""
    Wx0, Wh0 = params[0][0], params[0][1]
    m = nn.LSTM(Wx0.shape[1], Wh0.shape[1], num_layers=len(params), bias=bias,
                batch_first=batch_first, dtype=dtype)
    with torch.no_grad():
        for l, (Wx, Wh, bx, bh) in enumerate(params):
            getattr(m, f"weight_ih_l{l}").copy_(torch.as_tensor(Wx).to(dtype))
            getattr(m, f"weight_hh_l{l}").copy_(torch.as_tensor(Wh).to(dtype))
            if bias:
                getattr(m, f"bias_ih_l{l}").copy_(torch.as_tensor(bx).to(dtype))
                getattr(m, f"bias_hh_l{l}").copy_(torch.as_tensor(bh).to(dtype))
    return m


def nn_lstm_fwd_bwd(m, x, h0=None, c0=None, dout=None, dh_n=None, dc_n=None):
    """Run nn.LSTM forward (+ backward) and return tensors in a dict."""
    x = x.detach().clone().requires_grad_(dout is not None)
    state = None
    if h0 is not None:
        h0 = h0.detach().clone().requires_grad_(dout is not None)
        c0 = c0.detach().clone().requires_grad_(dout is not None)
        state = (h0, c0)
    for p in m.parameters():
        p.grad = None
    out, (hn, cn) = m(x, state)
    res = {"out": out.detach(), "h_n": hn.detach(), "c_n": cn.detach()}
    if dout is None:
        return res
    outs, grads = [out], [dout]
    if dh_n is not None:
        outs += [hn, cn]
        grads += [dh_n, dc_n]
    torch.autograd.backward(outs, grads)
    res["dx"] = x.grad
    if state is not None:
        res["dh0"], res["dc0"] = h0.grad, c0.grad
    for n, p in m.named_parameters():
        res["d_" + n] = p.grad.detach().clone()
    return res


def time_nn_lstm(input_size, hidden_size, num_layers, T, B, backward, reps=1, seed=0,
                 threads=None):
    """Wall-clock seconds of one nn.LSTM fp32 pass on the CPU (best of reps)."""
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    m = nn.LSTM(input_size, hidden_size, num_layers=num_layers)
    x = torch.randn(T, B, input_size, generator=g, requires_grad=backward)
    dout = torch.randn(T, B, hidden_size, generator=g)
    best = float("inf")
    for r in range(reps + 1):          # first repetition is the warm-up
        t0 = time.perf_counter()
        if backward:
            for p in m.parameters():
                p.grad = None
            x.grad = None
            out, _ = m(x)
            out.backward(dout)
        else:
            with torch.no_grad():
                m(x)
        dt = time.perf_counter() - t0
        if r > 0 or reps == 0:
            best = min(best, dt)
    return best, threads
