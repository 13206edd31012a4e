"""tcgen05 GEMM entry points (projection, input gradient, weight gradients) through the C ABI,
against an fp32 torch matmul of the same 16-bit operands and against the CUDA-core kernels."""
import pytest
import torch

from fastlstm_b200 import _lib

pytestmark = pytest.mark.gpu

TD = {"fp16": torch.float16, "bf16": torch.bfloat16}
# (T, B, I, H): aligned, ragged M, ragged N/K, split-K; CTA pairs (N % 256 == 0, M >= 256) with a ragged
# last tile row, with an odd CTA whose rows are all past M, and over many tiles
SHAPES = [(4, 64, 64, 64), (3, 50, 72, 40), (16, 128, 256, 256), (64, 256, 512, 128), (7, 33, 136, 200),
          (5, 77, 256, 64), (3, 100, 128, 128), (40, 512, 512, 512)]


def _desc(dtype, T, B, I, H, flags=0):
    return _lib.Desc(_lib.DTYPE_CODE[dtype], T, B, I, H, flags, 0, 0)


def _report(name, got, ref, tol):
    err = (got.float() - ref).abs()
    scale = ref.abs().max().clamp_min(1e-6)
    bad = err > tol * scale
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        rows = bad.any(dim=1).nonzero().flatten()
        cols = bad.any(dim=0).nonzero().flatten()
        pytest.fail(f"{name}: {int(bad.sum())}/{bad.numel()} bad, max err {float(err.max()):.4g} "
                    f"(scale {float(scale):.4g}), first bad {idx}, got {float(got[tuple(idx)]):.5g} "
                    f"want {float(ref[tuple(idx)]):.5g}; bad rows {rows[:8].tolist()}..{rows[-1].item()} "
                    f"bad cols {cols[:8].tolist()}..{cols[-1].item()}")


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("shape", SHAPES)
def test_projection_dgrad_wgrad(dtype, shape):
    lib = _lib.load()
    T, B, I, H = shape
    dt = TD[dtype]
    g = torch.Generator(device="cuda").manual_seed(T * 1000 + H)
    r = lambda *s: torch.randn(*s, generator=g, device="cuda")
    x, Wx = r(T, B, I).to(dt), (r(4 * H, I) * 0.1).to(dt)
    bx, bh = (r(4 * H) * 0.1).to(dt), (r(4 * H) * 0.1).to(dt)
    dg, out = r(T, B, 4 * H).to(dt), r(T + 1, B, H).to(dt)
    st = torch.cuda.current_stream().cuda_stream
    d = _desc(dtype, T, B, I, H)
    assert lib.blstm_plan_name(d, 0) in (b"generic", b"sm100")
    tol = 2e-3 if dtype == "fp16" else 1.2e-2

    # projection
    ifgo = torch.full((T, B, 4 * H), float("nan"), device="cuda", dtype=dt)
    _lib.check(lib.blstm_input_projection(d, x.data_ptr(), Wx.data_ptr(), bx.data_ptr(), bh.data_ptr(),
                                          ifgo.data_ptr(), st), "proj")
    ref = x.float().view(T * B, I) @ Wx.float().T + bx.float() + bh.float()
    _report("projection", ifgo.view(T * B, -1), ref, tol)
    # without biases
    _lib.check(lib.blstm_input_projection(d, x.data_ptr(), Wx.data_ptr(), None, None, ifgo.data_ptr(), st), "proj")
    _report("projection(no bias)", ifgo.view(T * B, -1), x.float().view(T * B, I) @ Wx.float().T, tol)

    n = lib.blstm_workspace_bytes(d, _lib.PHASE_BWD)
    ws = torch.zeros(n, dtype=torch.uint8, device="cuda")
    # input gradient
    dx = torch.full((T, B, I), float("nan"), device="cuda", dtype=dt)
    _lib.check(lib.blstm_dgrad_input(d, dg.data_ptr(), Wx.data_ptr(), dx.data_ptr(), ws.data_ptr(), n, st), "dgrad")
    _report("dgrad", dx.view(T * B, I), dg.float().view(T * B, -1) @ Wx.float(), tol)
    # weight gradients (fp32 outputs)
    dWx = torch.full((4 * H, I), float("nan"), device="cuda")
    dWh = torch.full((4 * H, H), float("nan"), device="cuda")
    _lib.check(lib.blstm_wgrad(d, dg.data_ptr(), x.data_ptr(), out.data_ptr(), dWx.data_ptr(), dWh.data_ptr(),
                               ws.data_ptr(), n, st), "wgrad")
    dg2 = dg.float().view(T * B, -1)
    _report("dWx", dWx, dg2.T @ x.float().view(T * B, I), 1e-4)
    _report("dWh", dWh, dg2.T @ out[:-1].float().reshape(T * B, H), 1e-4)
    torch.cuda.synchronize()


def test_gemm_entry_points_agree_with_cuda_core_kernels():
    """Same inputs through the tcgen05 GEMMs and through the CUDA-core GEMMs (force flag)."""
    lib = _lib.load()
    T, B, I, H = 8, 96, 128, 64
    dt = torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(T, B, I, generator=g, device="cuda").to(dt)
    Wx = (torch.randn(4 * H, I, generator=g, device="cuda") * 0.1).to(dt)
    st = torch.cuda.current_stream().cuda_stream
    outs = []
    for flags in (0, _lib.FLAG_FORCE_GENERIC):
        d = _desc("bf16", T, B, I, H, flags)
        o = torch.empty(T, B, 4 * H, device="cuda", dtype=dt)
        _lib.check(lib.blstm_input_projection(d, x.data_ptr(), Wx.data_ptr(), None, None, o.data_ptr(), st), "proj")
        outs.append(o.float())
    torch.cuda.synchronize()
    assert (outs[0] - outs[1]).abs().max() <= 2e-2 * outs[1].abs().max()
