"""Generate the golden fixtures in this directory.

Runs ONLY where a checkout of the reference is available: its directory is
argument 1, or the environment variable FASTLSTM_REFERENCE.  It imports the reference's pure-PyTorch LSTM path
(fastlstm/lstm.py:1087-1245, `naive_lstm_fwd`, `naive_lstm_bwd`,
`FastLSTM(version="naive-pt")`) on CPU through two stubs that leave the
reference untouched: a dummy `flashrnn` module (third-party competitor wrapper
imported at fastlstm/lstm.py:13, not installed) and a fake
`torch.cuda.get_device_properties` (queried at import by fastlstm/configs.py:5-6).
It also records torch.nn.LSTM results for the options the reference path lacks
(batch_first, bias=False, gradients through h_n/c_n).

Usage:  python tests/golden/make_golden.py [/path/to/reference]
Writes: naive_single.npz, naive_stacked.npz, nn_batch_first.npz, nn_nobias.npz
"""
import os
import sys
import types

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(path):
    fr = types.ModuleType("flashrnn")
    fr.flashrnn = lambda *a, **k: None
    sys.modules["flashrnn"] = fr

    class _Props:
        multi_processor_count = 148
        shared_memory_per_block = 49152

    torch.cuda.get_device_properties = lambda *a, **k: _Props()
    sys.path.insert(0, path)
    import fastlstm.lstm as L
    # the reference switches fp32 matmuls to TF32 on import; irrelevant on CPU,
    # but put the global default back
    torch.backends.cuda.matmul.fp32_precision = "ieee"
    return L


def u(gen, *shape, k):
    return (torch.rand(*shape, generator=gen) * 2 - 1) * k


def main():
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FASTLSTM_REFERENCE")
    if not where:
        sys.exit("usage: make_golden.py <directory of the reference checkout>")
    ref = import_reference(where)
    torch.set_num_threads(1)

    # ---- A: one layer through naive_lstm_fwd / naive_lstm_bwd, non-zero h0,c0,dc_n
    g = torch.Generator().manual_seed(2001)
    T, B, I, H = 6, 3, 5, 4
    k = 1 / H ** 0.5
    x = torch.randn(T, B, I, generator=g)
    h0 = torch.randn(B, H, generator=g) * 0.1
    c0 = torch.randn(B, H, generator=g) * 0.1
    Wx, Wh = u(g, 4 * H, I, k=k), u(g, 4 * H, H, k=k)
    bx, bh = u(g, 4 * H, k=k), u(g, 4 * H, k=k)
    dout = torch.randn(T, B, H, generator=g)
    dc_n = torch.randn(B, H, generator=g)
    out, cell, ifgo = ref.naive_lstm_fwd(x, h0, c0, Wx, bx, Wh, bh)
    dx, dh0, dc0, dWx, dbx, dWh, dbh = ref.naive_lstm_bwd(
        dout, dc_n.clone(), x, out, cell, ifgo, Wx, Wh)
    # reference naive layout is [T,B,H,4]; fixtures keep the kernels' [T,B,4H]
    ifgo_k = ifgo.permute(0, 1, 3, 2).reshape(T, B, 4 * H)
    np.savez(os.path.join(HERE, "naive_single.npz"),
             x=x, h0=h0, c0=c0, Wx=Wx, Wh=Wh, bx=bx, bh=bh, dout=dout, dc_n=dc_n,
             out=out, cell=cell, ifgo=ifgo_k, dx=dx, dh0=dh0, dc0=dc0,
             dWx=dWx, dWh=dWh, dbx=dbx, dbh=dbh)

    # ---- B: two layers through FastLSTM(version="naive-pt") and autograd
    torch.manual_seed(123)
    T, B, I, H = 9, 4, 7, 5
    m = ref.FastLSTM(I, H, num_layers=2, version="naive-pt")
    g = torch.Generator().manual_seed(2002)
    x = torch.randn(T, B, I, generator=g, requires_grad=True)
    dout = torch.randn(T, B, H, generator=g)
    y, (hn, cn) = m(x)
    y.backward(dout)
    d = {"x": x.detach(), "dout": dout, "out": y.detach(), "h_n": hn.detach(),
         "c_n": cn.detach(), "dx": x.grad}
    for n, p in m.named_parameters():
        d[n] = p.detach()
        d["d_" + n] = p.grad
    np.savez(os.path.join(HERE, "naive_stacked.npz"), **{k_: v.numpy() for k_, v in d.items()})

    # ---- C: nn.LSTM, batch_first, non-zero states, gradients through h_n/c_n
    torch.manual_seed(321)
    T, B, I, H = 8, 4, 16, 16
    m = nn.LSTM(I, H, num_layers=1, batch_first=True)
    g = torch.Generator().manual_seed(2003)
    x = torch.randn(B, T, I, generator=g, requires_grad=True)
    h0 = (torch.randn(1, B, H, generator=g) * 0.1).requires_grad_()
    c0 = (torch.randn(1, B, H, generator=g) * 0.1).requires_grad_()
    dout = torch.randn(B, T, H, generator=g)
    dh_n = torch.randn(1, B, H, generator=g)
    dc_n = torch.randn(1, B, H, generator=g)
    y, (hn, cn) = m(x, (h0, c0))
    torch.autograd.backward([y, hn, cn], [dout, dh_n, dc_n])
    d = {"x": x.detach(), "h0": h0.detach(), "c0": c0.detach(), "dout": dout,
         "dh_n": dh_n, "dc_n": dc_n, "out": y.detach(), "h_n": hn.detach(),
         "c_n": cn.detach(), "dx": x.grad, "dh0": h0.grad, "dc0": c0.grad}
    for n, p in m.named_parameters():
        d[n] = p.detach()
        d["d_" + n] = p.grad
    np.savez(os.path.join(HERE, "nn_batch_first.npz"), **{k_: v.numpy() for k_, v in d.items()})

    # ---- D: nn.LSTM, bias=False, two layers, ragged sizes
    torch.manual_seed(77)
    T, B, I, H = 7, 5, 11, 9
    m = nn.LSTM(I, H, num_layers=2, bias=False)
    g = torch.Generator().manual_seed(2004)
    x = torch.randn(T, B, I, generator=g, requires_grad=True)
    dout = torch.randn(T, B, H, generator=g)
    y, (hn, cn) = m(x)
    y.backward(dout)
    d = {"x": x.detach(), "dout": dout, "out": y.detach(), "h_n": hn.detach(),
         "c_n": cn.detach(), "dx": x.grad}
    for n, p in m.named_parameters():
        d[n] = p.detach()
        d["d_" + n] = p.grad
    np.savez(os.path.join(HERE, "nn_nobias.npz"), **{k_: v.numpy() for k_, v in d.items()})
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
