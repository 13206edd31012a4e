"""Pin the numpy oracle against fixtures produced by the reference's own
pure-PyTorch path and torch.nn.LSTM (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from oracle import lstm_oracle as O

TOL = dict(rtol=1e-5, atol=2e-6)


def _load(golden_dir, name):
    return dict(np.load(os.path.join(golden_dir, name)))


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_single_layer_matches_reference_naive_path(golden_dir, dt):
    g = _load(golden_dir, "naive_single.npz")
    a = {k: v.astype(dt) for k, v in g.items()}
    out, cell, ifgo = O.lstm_fwd(a["x"], a["h0"], a["c0"], a["Wx"], a["bx"], a["Wh"], a["bh"])
    np.testing.assert_allclose(out, g["out"], **TOL)
    np.testing.assert_allclose(cell, g["cell"], **TOL)
    np.testing.assert_allclose(ifgo, g["ifgo"], **TOL)
    dx, dh0, dc0, dWx, dWh, db = O.lstm_bwd(a["dout"], None, a["dc_n"], a["x"], out, cell,
                                            ifgo, a["Wx"], a["Wh"])
    for got, key in [(dx, "dx"), (dh0, "dh0"), (dc0, "dc0"), (dWx, "dWx"), (dWh, "dWh"),
                     (db, "dbx"), (db, "dbh")]:
        np.testing.assert_allclose(got, g[key], err_msg=key, **TOL)


def _params(g, L, bias=True):
    ps = []
    for l in range(L):
        ps.append((g[f"weight_ih_l{l}"], g[f"weight_hh_l{l}"],
                   g[f"bias_ih_l{l}"] if bias else None, g[f"bias_hh_l{l}"] if bias else None))
    return ps


def test_stacked_matches_reference_module(golden_dir):
    g = {k: v.astype(np.float64) for k, v in _load(golden_dir, "naive_stacked.npz").items()}
    r = O.stacked_fwd_bwd(g["x"], None, None, _params(g, 2), dout=g["dout"])
    for k in ("out", "h_n", "c_n", "dx"):
        np.testing.assert_allclose(r[k], g[k], err_msg=k, **TOL)
    for l in range(2):
        dWx, dWh, db = r["grads"][l]
        np.testing.assert_allclose(dWx, g[f"d_weight_ih_l{l}"], **TOL)
        np.testing.assert_allclose(dWh, g[f"d_weight_hh_l{l}"], **TOL)
        np.testing.assert_allclose(db, g[f"d_bias_ih_l{l}"], **TOL)
        np.testing.assert_allclose(db, g[f"d_bias_hh_l{l}"], **TOL)


def test_batch_first_states_and_terminal_grads(golden_dir):
    g = {k: v.astype(np.float64) for k, v in _load(golden_dir, "nn_batch_first.npz").items()}
    x = g["x"].transpose(1, 0, 2).copy()
    dout = g["dout"].transpose(1, 0, 2).copy()
    r = O.stacked_fwd_bwd(x, g["h0"], g["c0"], _params(g, 1), dout=dout,
                          dh_n=g["dh_n"], dc_n=g["dc_n"])
    np.testing.assert_allclose(r["out"].transpose(1, 0, 2), g["out"], **TOL)
    np.testing.assert_allclose(r["dx"].transpose(1, 0, 2), g["dx"], **TOL)
    for k in ("h_n", "c_n", "dh0", "dc0"):
        np.testing.assert_allclose(r[k], g[k], err_msg=k, **TOL)
    dWx, dWh, db = r["grads"][0]
    np.testing.assert_allclose(dWx, g["d_weight_ih_l0"], **TOL)
    np.testing.assert_allclose(dWh, g["d_weight_hh_l0"], **TOL)
    np.testing.assert_allclose(db, g["d_bias_hh_l0"], **TOL)


def test_no_bias_two_layers(golden_dir):
    g = {k: v.astype(np.float64) for k, v in _load(golden_dir, "nn_nobias.npz").items()}
    r = O.stacked_fwd_bwd(g["x"], None, None, _params(g, 2, bias=False), dout=g["dout"])
    for k in ("out", "h_n", "c_n", "dx"):
        np.testing.assert_allclose(r[k], g[k], err_msg=k, **TOL)
    for l in range(2):
        dWx, dWh, _ = r["grads"][l]
        np.testing.assert_allclose(dWx, g[f"d_weight_ih_l{l}"], **TOL)
        np.testing.assert_allclose(dWh, g[f"d_weight_hh_l{l}"], **TOL)


def test_oracle_agrees_with_torch_cpu_lstm():
    """Second oracle (nn.LSTM fp32 on CPU) vs. the numpy restatement, ragged sizes."""
    import torch
    from oracle.torch_cpu import make_nn_lstm, nn_lstm_fwd_bwd
    rng = np.random.default_rng(5)
    T, B, I, H = 11, 6, 13, 10
    ps = [(rng.uniform(-.3, .3, (4 * H, I if l == 0 else H)), rng.uniform(-.3, .3, (4 * H, H)),
           rng.uniform(-.3, .3, 4 * H), rng.uniform(-.3, .3, 4 * H)) for l in range(2)]
    x = rng.standard_normal((T, B, I))
    dout = rng.standard_normal((T, B, H))
    r = O.stacked_fwd_bwd(x, None, None, ps, dout=dout)
    m = make_nn_lstm(ps, dtype=torch.float64)
    t = nn_lstm_fwd_bwd(m, torch.tensor(x), dout=torch.tensor(dout))
    np.testing.assert_allclose(r["out"], t["out"].numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(r["dx"], t["dx"].numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(r["grads"][0][0], t["d_weight_ih_l0"].numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(r["grads"][1][1], t["d_weight_hh_l1"].numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(r["grads"][1][2], t["d_bias_ih_l1"].numpy(), rtol=1e-9, atol=1e-11)
