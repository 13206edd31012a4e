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
    with pytest.raises(NotImplementedError):
        FastLSTM(4, 4, proj_size=2)
    with pytest.raises(ValueError):
        FastLSTM(4, 4, dropout=1.5)
