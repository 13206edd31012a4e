"""The kernel variants the default benchmark runs (2-layer bf16, I=H=512, thousands of batch rows:
wide hidden slices and interleaved batch tiles in the forward recurrence, four interleaved tiles in
the backward recurrence) compared DIRECTLY with the numpy oracle at a sequence length the oracle
finishes in seconds, and the growth of the 16-bit error with sequence length (the gate maths of the
tensor-core kernels use the hardware tanh approximation)."""
import numpy as np
import pytest
import torch

from _util import assert_half_parity, make_case, norm_rel, run_module, run_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B", [4096, 1300])
def test_benchmark_plan_against_the_oracle(B):
    """B=4096: the benchmark's own geometry.  B=1300: same kernels with a ragged last batch tile."""
    import fastlstm_b200 as F
    T, H, L = 16, 512, 2
    assert F.plan_name(torch.bfloat16, T, B, H, H, "fwd") == "sm100"
    assert F.plan_name(torch.bfloat16, T, B, H, H, "bwd") == "sm100"
    fwd, bwd = F.plan_detail(torch.bfloat16, T, B, H, H, "fwd"), F.plan_detail(torch.bfloat16, T, B, H, H, "bwd")
    if B == 4096:   # what `bench.py` launches at one GPU
        assert "TI=1" not in fwd and "TI=1" not in bwd, (fwd, bwd)     # interleaved batch tiles
    case = make_case(4242 + B, T=T, B=B, I=H, H=H, L=L, dtype="bf16")
    ref = run_oracle(case)
    res = run_module(case)
    assert_half_parity(res, ref)


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_error_growth_with_sequence_length(seed):
    """fwd+bwd at H=512 over three seeds: the error against the fp64 oracle at T=256 stays inside
    the 16-bit bars and does not blow up relative to T=32."""
    B, H = 128, 512
    errs = {}
    for T in (32, 256):
        case = make_case(seed, T=T, B=B, I=H, H=H, dtype="bf16")
        ref = run_oracle(case)
        res = run_module(case)
        assert_half_parity(res, ref)
        errs[T] = (float(np.max(np.abs(res["out"] - ref["out"]))), norm_rel(res["dx"], ref["dx"]),
                   norm_rel(res["grads"][0][1], ref["grads"][0][1]))
    # the recurrence is contractive for these weight scales: a 8x longer sequence may not cost more
    # than a few times the short one's error
    assert errs[256][0] <= max(4 * errs[32][0], 1e-2), errs
    assert errs[256][1] <= max(4 * errs[32][1], 2e-2), errs
    assert errs[256][2] <= max(4 * errs[32][2], 2e-2), errs
