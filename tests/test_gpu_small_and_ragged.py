"""Tiny sizes on the single-kernel forward (input projection inside the time loop; the reference's
fully fused kernel, fastlstm/kernels.py:672-819, dispatch fastlstm/lstm.py:40-47) and ragged 16-bit
sizes zero-padded onto the tensor-core kernels (the reference's shape grid, tests/test_lstm.py:160-185,
runs these sizes on tl.dot), both against the numpy oracle."""
import numpy as np
import pytest
import torch

from _util import assert_fp32_parity, assert_half_parity, make_case, run_module, run_oracle
from fastlstm_b200 import _lib

pytestmark = pytest.mark.gpu
TD = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


@pytest.mark.parametrize("dtype,T,B,I,H", [("fp32", 12, 10, 32, 32), ("fp32", 9, 7, 20, 24), ("fp32", 6, 33, 5, 16),
                                           ("fp32", 5, 3, 32, 7), ("bf16", 10, 40, 64, 64), ("fp16", 8, 9, 48, 40),
                                           ("fp16", 7, 130, 33, 64)])
def test_fused_forward_against_the_oracle(dtype, T, B, I, H):
    import fastlstm_b200 as F
    assert F.plan_name(TD[dtype], T, B, I, H, "fwd_op") == "fused"
    case = make_case(300 + H + I, T=T, B=B, I=I, H=H, L=2 if H <= 32 else 1, dtype=dtype, h0_std=0.3,
                     terminal_grads=True)
    ref = run_oracle(case)
    res = run_module(case)
    if dtype == "fp32":
        assert_fp32_parity(res, ref, tol=1e-5, has_state=True)
    else:
        assert_half_parity(res, ref, has_state=True)


@pytest.mark.parametrize("dtype,T,B,I,H", [("fp32", 11, 13, 24, 32), ("bf16", 6, 70, 40, 64)])
def test_fused_forward_matches_projection_plus_recurrence(dtype, T, B, I, H):
    """blstm_fwd with and without BLSTM_FLAG_NO_FUSED through the C ABI; also the inference flag."""
    lib = _lib.load()
    dt = TD[dtype]
    g = torch.Generator(device="cuda").manual_seed(T * B)
    r = lambda *s: torch.randn(*s, generator=g, device="cuda")
    x = r(T, B, I).to(dt)
    Wx, Wh = (r(4 * H, I) / I ** 0.5).to(dt), (r(4 * H, H) / H ** 0.5).to(dt)
    bx, bh = (r(4 * H) * 0.1).to(dt), (r(4 * H) * 0.1).to(dt)
    h0, c0 = (r(B, H) * 0.3).to(dt), (r(B, H) * 0.3).to(dt)

    def fwd(flags):
        d = _lib.Desc(_lib.DTYPE_CODE[dtype], T, B, I, H, flags, 0, 0)
        out = torch.zeros(T + 1, B, H, device="cuda", dtype=dt)
        cell = torch.zeros(T + 1, B, H, device="cuda", dtype=dt)
        ifgo = torch.zeros(T, B, 4 * H, device="cuda", dtype=dt)
        n = lib.blstm_workspace_bytes(d, _lib.PHASE_FWD)
        ws = torch.zeros(n, dtype=torch.uint8, device="cuda")
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.blstm_fwd(d, x.data_ptr(), h0.data_ptr(), c0.data_ptr(), Wx.data_ptr(), Wh.data_ptr(),
                                 bx.data_ptr(), bh.data_ptr(), out.data_ptr(), cell.data_ptr(), ifgo.data_ptr(),
                                 ws.data_ptr(), n, s), "blstm_fwd")
        _lib.check(lib.blstm_read_status(ws.data_ptr(), None, s), "status")
        return out, cell, ifgo

    o1, c1, g1 = fwd(0)
    o2, c2, g2 = fwd(_lib.FLAG_NO_FUSED)
    tol = 2e-5 if dtype == "fp32" else 3e-2
    assert float((o1.float() - o2.float()).abs().max()) <= tol
    assert float((c1.float() - c2.float()).abs().max()) <= 2 * tol
    assert float((g1.float() - g2.float()).abs().max()) <= 4 * tol
    o3, c3, g3 = fwd(_lib.FLAG_INFERENCE)
    assert torch.equal(o3, o1) and torch.equal(c3[T], c1[T])
    assert float(g3.abs().max()) == 0.0 and (T == 1 or float(c3[1:T].abs().max()) == 0.0)


@pytest.mark.parametrize("dtype,T,B,I,H", [("fp16", 10, 44, 123, 65), ("bf16", 6, 100, 257, 257), ("fp16", 5, 4, 100, 72)])
def test_ragged_16bit_sizes_run_padded_on_the_tensor_core_kernels(dtype, T, B, I, H):
    import fastlstm_b200 as F
    import fastlstm_b200.lstm as mod
    Ip, Hp = mod._padded_sizes(TD[dtype], I, H)
    assert Ip % 8 == 0 and Hp % 64 == 0
    assert F.plan_name(TD[dtype], T, B, Ip, Hp, "fwd") == "sm100" and F.plan_name(TD[dtype], T, B, Ip, Hp, "bwd") == "sm100"
    case = make_case(500 + H, T=T, B=B, I=I, H=H, L=2, dtype=dtype, h0_std=0.2, terminal_grads=True)
    ref = run_oracle(case)
    res = run_module(case)
    assert_half_parity(res, ref, has_state=True)
    assert res["out"].shape == (T, B, H) and res["grads"][0][0].shape == (4 * H, I)
