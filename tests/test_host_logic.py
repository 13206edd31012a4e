"""Host-side behaviour of the module that needs no GPU."""
import pytest
import torch
import torch.nn as nn

from fastlstm_b200 import FastLSTM, lstm_persistent_fwd


def test_init_matches_nn_lstm_rng_order():
    # same check as the reference's tests/test_lstm.py:116-129
    torch.manual_seed(123)
    m1 = FastLSTM(8, 3, num_layers=2)
    torch.manual_seed(123)
    m2 = nn.LSTM(8, 3, num_layers=2)
    names = [n for n, _ in m1.named_parameters()]
    assert names == [n for n, _ in m2.named_parameters()]
    for n, p in m1.named_parameters():
        torch.testing.assert_close(p, getattr(m2, n))


def test_state_dict_interchange_and_no_bias():
    m1 = FastLSTM(5, 4, num_layers=2, bias=False)
    m2 = nn.LSTM(5, 4, num_layers=2, bias=False)
    m1.load_state_dict(m2.state_dict())
    m2.load_state_dict(m1.state_dict())
    assert all("bias" not in n for n, _ in m1.named_parameters())


def test_cpu_tensors_are_rejected_loudly():
    m = FastLSTM(4, 4)
    with pytest.raises(ValueError, match="CUDA"):
        m(torch.randn(3, 2, 4))
    with pytest.raises(ValueError):
        lstm_persistent_fwd(torch.randn(3, 2, 4), None, None, torch.randn(16, 4), None,
                            torch.randn(16, 4), None)


def test_unknown_version_rejected():
    with pytest.raises(ValueError):
        FastLSTM(4, 4, version="graph")


def test_bidirectional_parameters_match_nn_lstm_and_options_are_validated():
    m = FastLSTM(12, 8, num_layers=2, bidirectional=True, dropout=0.25)
    ref = nn.LSTM(12, 8, num_layers=2, bidirectional=True, dropout=0.25)
    assert [(n, tuple(p.shape)) for n, p in m.named_parameters()] == \
           [(n, tuple(p.shape)) for n, p in ref.named_parameters()]
    m.load_state_dict(ref.state_dict())
    ref.load_state_dict(m.state_dict())
    with pytest.raises(ValueError):
        FastLSTM(4, 4, proj_size=4)           # like nn.LSTM: smaller than hidden_size
    with pytest.raises(ValueError):
        FastLSTM(4, 4, dropout=1.5)


class _TorchLayer:
    """Stand-in for PersistentLSTMfn on CPU: the same call signature, plain differentiable torch ops."""

    @staticmethod
    def apply(x, h0, c0, Wx, bx, Wh, bh, inference=None, sink=None, want_cells=False):
        T, B, _ = x.shape
        H = Wh.shape[1]
        h = x.new_zeros(B, H) if h0 is None else h0
        c = x.new_zeros(B, H) if c0 is None else c0
        outs, cells = [], []
        for t in range(T):
            a = x[t] @ Wx.T + h @ Wh.T + (0 if bx is None else bx + bh)
            i, f, g, o = a.split(H, dim=1)
            c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
            h = torch.sigmoid(o) * torch.tanh(c)
            outs.append(h)
            cells.append(c)
        out = torch.stack(outs)
        res = (out, out[-1], cells[-1])
        return res + (torch.stack(cells).detach(),) if want_cells else res


@pytest.mark.parametrize("bidirectional", [False, True])
def test_packed_sequence_plumbing_matches_nn_lstm(monkeypatch, bidirectional):
    """PackedSequence in, PackedSequence out, states at every sequence's own last step, the reverse
    direction from every sequence's own end, gradients through the packed output and h_n - checked on
    CPU with a torch stand-in for the CUDA layer against torch.nn.LSTM."""
    import fastlstm_b200.lstm as mod
    from torch.nn.utils.rnn import pack_padded_sequence
    monkeypatch.setattr(mod, "PersistentLSTMfn", _TorchLayer)
    torch.manual_seed(4)
    I, H, L = 5, 6, 2
    ref = torch.nn.LSTM(I, H, num_layers=L, bidirectional=bidirectional).double()
    m = mod.FastLSTM(I, H, num_layers=L, bidirectional=bidirectional, dtype=torch.float64)
    m.load_state_dict(ref.state_dict())
    lengths = torch.tensor([3, 7, 1, 5])
    x = torch.randn(7, 4, I, dtype=torch.float64)
    nd = 2 if bidirectional else 1
    h0, c0 = torch.randn(L * nd, 4, H, dtype=torch.float64), torch.randn(L * nd, 4, H, dtype=torch.float64)
    results = []
    for net in (ref, m):
        xi = x.clone().requires_grad_()
        out, (hn, cn) = net(pack_padded_sequence(xi, lengths, enforce_sorted=False), (h0, c0))
        (out.data.square().sum() + hn.sum()).backward()
        results.append((out, hn, cn, xi.grad, [p.grad.clone() for p in net.parameters()]))
        net.zero_grad()
    (o1, h1, c1, g1, p1), (o2, h2, c2, g2, p2) = results
    assert torch.equal(o1.batch_sizes, o2.batch_sizes) and torch.equal(o1.sorted_indices, o2.sorted_indices)
    for a, b in ((o1.data, o2.data), (h1, h2), (c1, c2), (g1, g2)):
        torch.testing.assert_close(a, b, rtol=1e-9, atol=1e-10)
    for a, b in zip(p1, p2):
        torch.testing.assert_close(a, b, rtol=1e-9, atol=1e-10)


def test_persistent_plans_fit_the_device_for_a_sweep_of_shapes():
    """Every tensor-core plan must be launchable on a 148-SM part: the forward grid within the SM count,
    the backward grid within the 33 clusters of four that can be resident at once, shared memory
    within the 227 KB a CTA may have.  (Geometry only: nothing is launched.)"""
    import re
    from fastlstm_b200 import plan_detail
    seen = set()
    for H in (64, 128, 192, 256, 320, 384, 512, 640, 768, 1024, 1280, 1536, 2048):
        for B in (1, 32, 100, 128, 129, 256, 400, 512, 640, 1024, 1300, 2048, 2304, 4096, 4800, 8192):
            for phase in ("fwd", "bwd"):
                s = plan_detail(torch.bfloat16, 8, B, H, H, phase)
                assert s.startswith("sm100"), (B, H, phase, s)
                grid = int(re.search(r"grid=(\d+)", s).group(1))
                assert grid <= (132 if phase == "bwd" else 148), (B, H, phase, s)
                if phase == "bwd":
                    assert grid % 4 == 0, s
                m = re.search(r"smem=(\d+)", s)
                if m:
                    assert int(m.group(1)) <= 232448, (B, H, phase, s)
                seen.add(re.sub(r"grid=\d+|smem=\d+", "", s))
    assert len(seen) > 20      # the sweep meets many different plans


@pytest.mark.parametrize("bidirectional", [False, True])
def test_proj_size_plumbing_matches_nn_lstm(monkeypatch, bidirectional):
    """nn.LSTM's output projection (proj_size): parameter names, shapes and order, the stepwise layer with
    the projected state zero-padded to the cell's width, initial states of the projected width, packed
    input - checked on CPU with a torch stand-in for the CUDA cell against torch.nn.LSTM."""
    import fastlstm_b200.lstm as mod
    from torch.nn.utils.rnn import pack_padded_sequence
    monkeypatch.setattr(mod, "PersistentLSTMfn", _TorchLayer)
    torch.manual_seed(7)
    I, H, P, L = 5, 8, 3, 2
    ref = torch.nn.LSTM(I, H, num_layers=L, bidirectional=bidirectional, proj_size=P).double()
    m = mod.FastLSTM(I, H, num_layers=L, bidirectional=bidirectional, proj_size=P, dtype=torch.float64)
    assert [n for n, _ in m.named_parameters()] == [n for n, _ in ref.named_parameters()]
    assert [tuple(p.shape) for p in m.parameters()] == [tuple(p.shape) for p in ref.parameters()]
    m.load_state_dict(ref.state_dict())
    nd = 2 if bidirectional else 1
    x = torch.randn(6, 4, I, dtype=torch.float64)
    h0, c0 = torch.randn(L * nd, 4, P, dtype=torch.float64), torch.randn(L * nd, 4, H, dtype=torch.float64)
    for packed in (False, True):
        results = []
        for net in (ref, m):
            xi = x.clone().requires_grad_()
            inp = pack_padded_sequence(xi, torch.tensor([6, 2, 5, 1]), enforce_sorted=False) if packed else xi
            out, (hn, cn) = net(inp, (h0, c0))
            data = out.data if packed else out
            (data.square().sum() + hn.sum() + (0 if packed else cn.sum())).backward()
            results.append((data, hn, cn, xi.grad, [p.grad.clone() for p in net.parameters()]))
            net.zero_grad()
        (o1, h1, c1, g1, p1), (o2, h2, c2, g2, p2) = results
        assert o2.shape[-1] == P * nd and h2.shape == (L * nd, 4, P) and c2.shape == (L * nd, 4, H)
        for a, b in ((o1, o2), (h1, h2), (c1, c2), (g1, g2)):
            torch.testing.assert_close(a, b, rtol=1e-9, atol=1e-10)
        for a, b in zip(p1, p2):
            torch.testing.assert_close(a, b, rtol=1e-9, atol=1e-10)
    # without initial states, and the constructor's checks
    out, (hn, cn) = m(x)
    ro, (rh, rc) = ref(x)
    torch.testing.assert_close(out, ro, rtol=1e-9, atol=1e-10)
    with pytest.raises(ValueError):
        mod.FastLSTM(I, H, proj_size=H)
    with pytest.raises(ValueError):
        mod.FastLSTM(I, H, proj_size=-1)
