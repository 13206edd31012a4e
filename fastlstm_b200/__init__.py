"""fastlstm_b200 — B200 (sm_100a) LSTM layer behind the FastLSTM module surface.

The CUDA library (libfastlstm_b200.so, C ABI in include/fastlstm_b200.h) is
loaded on first use; there is no CPU or PyTorch fallback.
"""
from .lstm import (FastLSTM, PersistentLSTMfn, Wgrad, check_status, lstm_persistent_bwd,
                   lstm_persistent_fwd, persistent_lstm, plan_detail, plan_name)

__all__ = ["FastLSTM", "PersistentLSTMfn", "Wgrad", "check_status", "lstm_persistent_bwd",
           "lstm_persistent_fwd", "persistent_lstm", "plan_detail", "plan_name"]
