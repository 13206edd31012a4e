"""The five benchmark shapes at their FULL sizes: CUDA path vs. torch.nn.LSTM fp32 on the host cores
(the reference's own oracle) on identical 16-bit-rounded inputs, plus size-independent properties
where the CPU oracle would take too long (config 5)."""
import numpy as np
import pytest
import torch

from _util import assert_half_parity, make_case, norm_rel, run_module
from oracle.torch_cpu import make_nn_lstm, nn_lstm_fwd_bwd

pytestmark = pytest.mark.gpu


def _cpu_oracle(case, backward):
    torch.set_num_threads(max(1, torch.get_num_threads()))
    m = make_nn_lstm(case["params"])
    st = (case["h0"], case["c0"]) if case["h0"] is not None else (None, None)
    r = nn_lstm_fwd_bwd(m, case["x"], st[0], st[1], dout=case["dout"] if backward else None)
    f = lambda t: t.double().numpy()
    ref = {"out": f(r["out"]), "h_n": f(r["h_n"]), "c_n": f(r["c_n"])}
    if backward:
        ref["dx"] = f(r["dx"])
        if st[0] is not None:
            ref["dh0"], ref["dc0"] = f(r["dh0"]), f(r["dc0"])
        ref["grads"] = [(f(r[f"d_weight_ih_l{l}"]), f(r[f"d_weight_hh_l{l}"]), f(r[f"d_bias_ih_l{l}"]))
                        for l in range(case["L"])]
    return ref


def test_config2_full_forward_fp16():
    """fp16 forward, B=64 T=1024 I=H=256, zero initial state, W,b ~ U(+-1/16)."""
    case = make_case(1002, T=1024, B=64, I=256, H=256, dtype="fp16", wscale=1 / 16)
    ref = _cpu_oracle(case, backward=False)
    res = run_module(case, backward=False)
    for k in ("out", "h_n", "c_n"):
        assert float(np.max(np.abs(res[k] - ref[k]))) <= 2e-2, k


def test_config3_full_forward_backward_fp16():
    """fp16 fwd+bwd, B=256 T=512 I=H=1024, h0=c0~N(0,0.01), W ~ U(+-1/32)."""
    case = make_case(1003, T=512, B=256, I=1024, H=1024, dtype="fp16", h0_std=0.01, wscale=1 / 32)
    ref = _cpu_oracle(case, backward=True)
    res = run_module(case)
    assert_half_parity(res, ref, has_state=True)


def test_config4_full_forward_backward_bf16():
    """bf16 fwd+bwd, B=32 T=1024 I=H=2048 (Wh streamed: it does not fit in shared memory)."""
    case = make_case(1004, T=1024, B=32, I=2048, H=2048, dtype="bf16")
    ref = _cpu_oracle(case, backward=True)
    res = run_module(case)
    assert_half_parity(res, ref)


def test_config5_full_size_properties_bf16():
    """2-layer bf16, T=256, I=H=512 at the per-GPU batch of the 8-GPU run (512) and at 2048 rows:
    repeat runs are bit-identical, a batch shard alone reproduces its rows (to rounding: the two batch
    sizes use different tilings, hence different fp32 summation orders), and the weight gradients of
    the shards add up to those of the whole batch (the multi-GPU contract)."""
    case = make_case(1005, T=256, B=2048, I=512, H=512, L=2, dtype="bf16")
    full = run_module(case)
    again = run_module(case)
    assert np.array_equal(full["out"], again["out"]) and np.array_equal(full["dx"], again["dx"])
    acc = None
    for s in range(4):
        sh = dict(case)
        sl = slice(512 * s, 512 * (s + 1))
        sh["B"], sh["x"], sh["dout"] = 512, case["x"][:, sl].contiguous(), case["dout"][:, sl].contiguous()
        r = run_module(sh)
        assert float(np.max(np.abs(r["out"] - full["out"][:, sl]))) <= 2e-2
        assert norm_rel(r["dx"], full["dx"][:, sl]) <= 2e-2
        g = [np.stack([x for x in layer if x is not None and x.ndim == 2][:1]) for layer in r["grads"]]
        acc = g if acc is None else [a + b for a, b in zip(acc, g)]
    for l in range(2):
        assert norm_rel(acc[l][0], full["grads"][l][0]) < 2e-2
