"""Shared helpers for the GPU parity tests: seeded inputs, oracle runs, comparisons."""
import numpy as np
import torch

from oracle import lstm_oracle as O

TORCH_DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def make_case(seed, T, B, I, H, L=1, dtype="fp32", h0_std=0.0, bias=True, wscale=None,
              terminal_grads=False):
    """Seeded CPU tensors (fp32 master copies already rounded to `dtype`)."""
    g = torch.Generator().manual_seed(seed)
    dt = TORCH_DT[dtype]
    rnd = lambda t: t.to(dt).to(torch.float32)
    k = wscale if wscale is not None else 1.0 / H ** 0.5
    u = lambda *s: rnd((torch.rand(*s, generator=g) * 2 - 1) * k)
    params = []
    for l in range(L):
        params.append((u(4 * H, I if l == 0 else H), u(4 * H, H),
                       u(4 * H) if bias else None, u(4 * H) if bias else None))
    case = {"T": T, "B": B, "I": I, "H": H, "L": L, "dtype": dtype, "params": params,
            "x": rnd(torch.randn(T, B, I, generator=g)),
            "dout": rnd(torch.randn(T, B, H, generator=g)), "h0": None, "c0": None,
            "dh_n": None, "dc_n": None}
    if h0_std > 0:
        case["h0"] = rnd(torch.randn(L, B, H, generator=g) * h0_std)
        case["c0"] = rnd(torch.randn(L, B, H, generator=g) * h0_std)
    if terminal_grads:
        case["dh_n"] = rnd(torch.randn(L, B, H, generator=g))
        case["dc_n"] = rnd(torch.randn(L, B, H, generator=g))
    return case


def run_oracle(case, np_dtype=np.float64):
    n = lambda t: None if t is None else t.numpy().astype(np_dtype)
    params = [tuple(n(p) for p in ps) for ps in case["params"]]
    return O.stacked_fwd_bwd(n(case["x"]), n(case["h0"]), n(case["c0"]), params,
                             dout=n(case["dout"]), dh_n=n(case["dh_n"]), dc_n=n(case["dc_n"]))


def build_module(case, device="cuda", batch_first=False):
    from fastlstm_b200 import FastLSTM
    dt = TORCH_DT[case["dtype"]]
    bias = case["params"][0][2] is not None
    m = FastLSTM(case["I"], case["H"], num_layers=case["L"], bias=bias, batch_first=batch_first,
                 device=device, dtype=dt)
    with torch.no_grad():
        for l, (Wx, Wh, bx, bh) in enumerate(case["params"]):
            getattr(m, f"weight_ih_l{l}").copy_(Wx)
            getattr(m, f"weight_hh_l{l}").copy_(Wh)
            if bias:
                getattr(m, f"bias_ih_l{l}").copy_(bx)
                getattr(m, f"bias_hh_l{l}").copy_(bh)
    return m


def run_module(case, device="cuda", batch_first=False, backward=True):
    """Run FastLSTM on the GPU; returns numpy fp64 arrays in the oracle's dict layout."""
    import fastlstm_b200
    dt = TORCH_DT[case["dtype"]]
    m = build_module(case, device, batch_first)
    dev = lambda t: None if t is None else t.to(device=device, dtype=dt)
    x = dev(case["x"])
    dout = dev(case["dout"])
    if batch_first:
        x, dout = x.transpose(0, 1).contiguous(), dout.transpose(0, 1).contiguous()
    x.requires_grad_(backward)
    state = None
    if case["h0"] is not None:
        state = (dev(case["h0"]).requires_grad_(backward), dev(case["c0"]).requires_grad_(backward))
    out, (hn, cn) = m(x, state)
    f = lambda t: t.detach().double().cpu().numpy()
    res = {"out": f(out.transpose(0, 1) if batch_first else out), "h_n": f(hn), "c_n": f(cn)}
    if backward:
        outs, grads = [out], [dout]
        if case["dh_n"] is not None:
            outs += [hn, cn]
            grads += [dev(case["dh_n"]), dev(case["dc_n"])]
        torch.autograd.backward(outs, grads)
        res["dx"] = f(x.grad.transpose(0, 1) if batch_first else x.grad)
        if state is not None:
            res["dh0"], res["dc0"] = f(state[0].grad), f(state[1].grad)
        res["grads"] = []
        for l in range(case["L"]):
            gW = f(getattr(m, f"weight_ih_l{l}").grad)
            gH = f(getattr(m, f"weight_hh_l{l}").grad)
            gb = f(getattr(m, f"bias_ih_l{l}").grad) if m.bias else None
            if m.bias:
                assert torch.equal(getattr(m, f"bias_ih_l{l}").grad, getattr(m, f"bias_hh_l{l}").grad)
            res["grads"].append((gW, gH, gb))
    torch.cuda.synchronize()
    fastlstm_b200.check_status()
    return res


def max_rel(got, ref):
    """max |got-ref| / max |ref|  (per-tensor relative error)."""
    scale = max(float(np.max(np.abs(ref))), 1e-30)
    return float(np.max(np.abs(got - ref))) / scale


def norm_rel(got, ref):
    return float(np.linalg.norm((got - ref).ravel()) / max(np.linalg.norm(ref.ravel()), 1e-30))


def assert_fp32_parity(res, ref, tol=1e-5, has_state=False):
    """fp32 bar: 1e-5 relative (max-abs error / max-abs reference, per tensor) on outputs and gradients."""
    keys = ["out", "h_n", "c_n", "dx"] + (["dh0", "dc0"] if has_state else [])
    for k in keys:
        e = max_rel(res[k], ref[k])
        assert e <= tol, f"{k}: rel err {e:.3e} > {tol}"
    for l, (g, r) in enumerate(zip(res["grads"], ref["grads"])):
        for name, a, b in zip(("dWx", "dWh", "db"), g, r):
            if a is None:
                continue
            e = max_rel(a, b)
            assert e <= tol, f"layer {l} {name}: rel err {e:.3e} > {tol}"


def assert_half_parity(res, ref, has_state=False, abs_hc=2e-2, rel_w=5e-2):
    """16-bit bar: 2e-2 absolute on h/c, 5e-2 relative on weight gradients
    (norm-wise), against the fp32/fp64 oracle run on the same rounded inputs."""
    for k in ("out", "h_n", "c_n"):
        e = float(np.max(np.abs(res[k] - ref[k])))
        assert e <= abs_hc, f"{k}: abs err {e:.3e} > {abs_hc}"
    keys = ["dx"] + (["dh0", "dc0"] if has_state else [])
    for k in keys:
        e = norm_rel(res[k], ref[k])
        assert e <= rel_w, f"{k}: norm-rel err {e:.3e} > {rel_w}"
    for l, (g, r) in enumerate(zip(res["grads"], ref["grads"])):
        for name, a, b in zip(("dWx", "dWh", "db"), g, r):
            if a is None:
                continue
            e = norm_rel(a, b)
            assert e <= rel_w, f"layer {l} {name}: norm-rel err {e:.3e} > {rel_w}"
