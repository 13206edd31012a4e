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
