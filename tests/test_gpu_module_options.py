"""nn.LSTM options the reference lists as missing (README.md:92-93) and this module adds:
`bidirectional` and inter-layer `dropout`.  Oracle: torch.nn.LSTM in float64 on the CPU with
the same state dict (the comparison every reference test makes, tests/test_lstm.py:53,120,196)."""
import numpy as np
import pytest
import torch

from _util import TORCH_DT, max_rel

pytestmark = pytest.mark.gpu


def _pair(I, H, L, dtype, seed, bidirectional=True, dropout=0.0, bias=True):
    import fastlstm_b200 as F
    torch.manual_seed(seed)
    ref = torch.nn.LSTM(I, H, num_layers=L, bias=bias, bidirectional=bidirectional).double()
    dt = TORCH_DT[dtype]
    with torch.no_grad():                       # both sides see weights already rounded to `dtype`
        for p in ref.parameters():
            p.copy_(p.to(dt).double())
    m = F.FastLSTM(I, H, num_layers=L, bias=bias, bidirectional=bidirectional, dropout=dropout,
                   device="cuda", dtype=dt)
    m.load_state_dict({k: v.to(dt) for k, v in ref.state_dict().items()})
    return m, ref


def _run_both(m, ref, T, B, I, H, L, dtype, seed, states=True):
    dt = TORCH_DT[dtype]
    nd = 2 if m.bidirectional else 1
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dt).double()
    x, dout = rnd(T, B, I), rnd(T, B, nd * H)
    h0, c0 = rnd(L * nd, B, H) * 0.1, rnd(L * nd, B, H) * 0.1
    h0, c0 = h0.to(dt).double(), c0.to(dt).double()
    dhn, dcn = rnd(L * nd, B, H), rnd(L * nd, B, H)

    def go(mod, cast):
        xi = cast(x).requires_grad_(True)
        st = (cast(h0).requires_grad_(True), cast(c0).requires_grad_(True)) if states else None
        out, (hn, cn) = mod(xi, st)
        torch.autograd.backward([out, hn, cn], [cast(dout), cast(dhn), cast(dcn)])
        f = lambda t: t.detach().double().cpu().numpy()
        res = {"out": f(out), "h_n": f(hn), "c_n": f(cn), "dx": f(xi.grad)}
        if states:
            res["dh0"], res["dc0"] = f(st[0].grad), f(st[1].grad)
        for n, p in mod.named_parameters():
            res["grad:" + n] = f(p.grad)
        return res

    got = go(m, lambda t: t.to("cuda", dt))
    want = go(ref, lambda t: t.clone())
    torch.cuda.synchronize()
    return got, want


def test_bidirectional_fp32_matches_nn_lstm():
    import fastlstm_b200 as F
    T, B, I, H, L = 9, 5, 11, 24, 2
    m, ref = _pair(I, H, L, "fp32", seed=3)
    got, want = _run_both(m, ref, T, B, I, H, L, "fp32", seed=4)
    F.check_status()
    assert got["out"].shape == (T, B, 2 * H) and got["h_n"].shape == (2 * L, B, H)
    for k in want:
        assert max_rel(got[k], want[k]) <= 1e-5, k


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_bidirectional_half_on_tensor_core_kernels(dtype):
    import fastlstm_b200 as F
    T, B, I, H, L = 12, 130, 64, 64, 2            # H % 64 == 0: the tcgen05 kernels run
    m, ref = _pair(I, H, L, dtype, seed=5)
    got, want = _run_both(m, ref, T, B, I, H, L, dtype, seed=6)
    F.check_status()
    for k in ("out", "h_n", "c_n"):
        assert float(np.max(np.abs(got[k] - want[k]))) <= 2e-2, k
    for k in want:
        if k.startswith("grad:weight"):
            e = float(np.linalg.norm(got[k] - want[k]) / np.linalg.norm(want[k]))
            assert e <= 5e-2, (k, e)


def test_dropout_only_acts_between_layers_while_training():
    import fastlstm_b200 as F
    T, B, I, H, L = 7, 6, 10, 16, 3
    m, _ = _pair(I, H, L, "fp32", seed=7, bidirectional=False, dropout=0.5)
    plain, _ = _pair(I, H, L, "fp32", seed=7, bidirectional=False, dropout=0.0)
    x = torch.randn(T, B, I, device="cuda")
    m.eval()
    assert torch.equal(m(x)[0], plain(x)[0])                    # inactive in eval mode
    m.train()
    torch.manual_seed(11)
    a = m(x)[0]
    torch.manual_seed(11)
    b = m(x)[0]
    assert torch.equal(a, b) and not torch.equal(a, plain(x)[0])   # seeded, and it does drop
    xg = x.clone().requires_grad_(True)
    m(xg)[0].sum().backward()
    assert torch.isfinite(xg.grad).all() and all(torch.isfinite(p.grad).all() for p in m.parameters())
    one, _ = _pair(I, H, 1, "fp32", seed=7, bidirectional=False, dropout=0.5)
    one.train()
    assert torch.equal(one(x)[0], one(x)[0])                     # a single layer has nothing to drop
    F.check_status()


@pytest.mark.parametrize("dtype,bidirectional,H", [("fp32", False, 24), ("fp32", True, 40), ("bf16", True, 128)])
def test_packed_sequence_matches_nn_lstm(dtype, bidirectional, H):
    """PackedSequence input (sequences of different lengths, unsorted): packed output, states at every
    sequence's own last step, the reverse direction from every sequence's own end, and the gradients
    through the output and h_n, against torch.nn.LSTM float64 on the CPU."""
    import fastlstm_b200 as F
    from torch.nn.utils.rnn import pack_padded_sequence
    I, L, B, T = 12, 2, 6, 9
    m, ref = _pair(I, H, L, dtype, seed=21, bidirectional=bidirectional)
    dt = TORCH_DT[dtype]
    nd = 2 if bidirectional else 1
    g = torch.Generator().manual_seed(22)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dt).double()
    x = rnd(T, B, I)
    lengths = torch.tensor([4, 9, 1, 6, 9, 2])
    h0, c0 = rnd(L * nd, B, H) * 0.1, rnd(L * nd, B, H) * 0.1
    h0, c0 = h0.to(dt).double(), c0.to(dt).double()

    def go(mod, cast):
        xi = cast(x).requires_grad_(True)
        out, (hn, cn) = mod(pack_padded_sequence(xi, lengths, enforce_sorted=False), (cast(h0), cast(c0)))
        (out.data.float().square().sum() + hn.float().sum()).backward()
        f = lambda t: t.detach().double().cpu().numpy()
        res = {"out": f(out.data), "h_n": f(hn), "c_n": f(cn), "dx": f(xi.grad), "bs": out.batch_sizes.clone()}
        for n, p in mod.named_parameters():
            res["grad:" + n] = f(p.grad)
        return res

    got = go(m, lambda t: t.to("cuda", dt))
    want = go(ref, lambda t: t.clone())
    torch.cuda.synchronize()
    F.check_status()
    assert torch.equal(got["bs"], want["bs"])
    for k in want:
        if k == "bs":
            continue
        if dtype == "fp32":
            assert max_rel(got[k], want[k]) <= 2e-5, k
        elif k in ("out", "h_n", "c_n"):
            assert float(np.max(np.abs(got[k] - want[k]))) <= 2e-2, k
        else:
            e = float(np.linalg.norm(got[k] - want[k]) / max(np.linalg.norm(want[k]), 1e-30))
            assert e <= 5e-2, (k, e)


@pytest.mark.parametrize("dtype,bidirectional,H,P", [("fp32", False, 24, 10), ("fp32", True, 40, 16), ("bf16", False, 128, 64)])
def test_proj_size_matches_nn_lstm(dtype, bidirectional, H, P):
    """Output projection (nn.LSTM's proj_size; the reference lists it as missing, README.md:92-93):
    outputs, projected h_n, c_n and every gradient (weight_hr included) against torch.nn.LSTM in float64."""
    import fastlstm_b200 as F
    T, B, I, L = 7, 6, 16, 2
    dt = TORCH_DT[dtype]
    nd = 2 if bidirectional else 1
    torch.manual_seed(31)
    ref = torch.nn.LSTM(I, H, num_layers=L, bidirectional=bidirectional, proj_size=P).double()
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.to(dt).double())
    m = F.FastLSTM(I, H, num_layers=L, bidirectional=bidirectional, proj_size=P, device="cuda", dtype=dt)
    assert [n for n, _ in m.named_parameters()] == [n for n, _ in ref.named_parameters()]
    m.load_state_dict({k: v.to(dt) for k, v in ref.state_dict().items()})
    g = torch.Generator().manual_seed(32)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dt).double()
    x, dout = rnd(T, B, I), rnd(T, B, nd * P)
    h0, c0 = rnd(L * nd, B, P) * 0.1, rnd(L * nd, B, H) * 0.1
    h0, c0 = h0.to(dt).double(), c0.to(dt).double()

    def go(mod, cast):
        xi = cast(x).requires_grad_(True)
        out, (hn, cn) = mod(xi, (cast(h0), cast(c0)))
        torch.autograd.backward([out, hn], [cast(dout), torch.ones_like(hn)])
        f = lambda t: t.detach().double().cpu().numpy()
        res = {"out": f(out), "h_n": f(hn), "c_n": f(cn), "dx": f(xi.grad)}
        for n, p in mod.named_parameters():
            res["grad:" + n] = f(p.grad)
        return res

    got = go(m, lambda t: t.to("cuda", dt))
    want = go(ref, lambda t: t.clone())
    F.check_status()
    assert got["out"].shape == (T, B, nd * P) and got["h_n"].shape == (L * nd, B, P) and got["c_n"].shape == (L * nd, B, H)
    for k in want:
        if dtype == "fp32":
            assert max_rel(got[k], want[k]) <= 2e-5, k
        elif k in ("out", "h_n", "c_n"):
            assert np.abs(got[k] - want[k]).max() <= 2e-2, k
        else:
            assert max_rel(got[k], want[k]) <= 5e-2, k


@pytest.mark.parametrize("B,states", [(512, False), (300, True), (64, True)])
def test_layer_wavefront_matches_the_sequential_stack(monkeypatch, B, states):
    """Two layers, few batch tiles: the stack runs as a wavefront over time chunks on two streams
    (layer 1 on chunk k beside layer 0 on chunk k+1).  Same results as the layers run one after the
    other, up to the cell state crossing chunk boundaries in bf16; gradients of inputs, initial states
    and parameters included."""
    import fastlstm_b200 as F
    T, I, H, L = 96, 512, 512, 2
    dt = torch.bfloat16
    torch.manual_seed(5)
    m = F.FastLSTM(I, H, num_layers=L, device="cuda", dtype=dt)
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(T, B, I, generator=g, device="cuda").to(dt)
    dout = torch.randn(T, B, H, generator=g, device="cuda").to(dt)
    dhn = torch.randn(L, B, H, generator=g, device="cuda").to(dt)
    h0 = (torch.randn(L, B, H, generator=g, device="cuda") * 0.1).to(dt)
    c0 = (torch.randn(L, B, H, generator=g, device="cuda") * 0.1).to(dt)
    assert m._wavefront_chunks(x.requires_grad_(True), None, None) == 4

    def run(on):
        monkeypatch.setenv("FASTLSTM_B200_WAVEFRONT", "1" if on else "0")
        xi = x.detach().clone().requires_grad_(True)
        st = (h0.clone().requires_grad_(True), c0.clone().requires_grad_(True)) if states else None
        m.zero_grad()
        out, (hn, cn) = m(xi, st)
        torch.autograd.backward([out, hn], [dout, dhn])
        torch.cuda.synchronize()
        F.check_status()
        res = {"out": out, "h_n": hn, "c_n": cn, "dx": xi.grad}
        if states:
            res["dh0"], res["dc0"] = st[0].grad, st[1].grad
        for n, p in m.named_parameters():
            res["grad:" + n] = p.grad.clone()
        return {k: v.detach().float().cpu().numpy() for k, v in res.items()}

    want, got = run(False), run(True)
    for k in want:
        if k in ("out", "h_n", "c_n"):
            assert np.abs(got[k] - want[k]).max() <= 2e-2, k
        else:
            assert max_rel(got[k], want[k]) <= 3e-2, k
    again = run(True)
    for k in got:
        assert np.array_equal(got[k], again[k]), k      # deterministic
    # the same wavefront without anything saved for backward (inference): identical outputs
    monkeypatch.setenv("FASTLSTM_B200_WAVEFRONT", "1")
    with torch.no_grad():
        out, (hn, cn) = m(x.detach(), (h0, c0) if states else None)
    torch.cuda.synchronize()
    F.check_status()
    assert np.array_equal(out.float().cpu().numpy(), got["out"]) and np.array_equal(cn.float().cpu().numpy(), got["c_n"])
