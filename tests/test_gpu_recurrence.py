"""tcgen05 persistent recurrence kernels through the C ABI against the CUDA-core kernels
(same inputs, force flag) and against an fp32 step-by-step torch evaluation."""
import pytest
import torch

from fastlstm_b200 import _lib

pytestmark = pytest.mark.gpu
TD = {"fp16": torch.float16, "bf16": torch.bfloat16}

# (T, B, H): single tile; ragged batch tile; several hidden tiles; H=1024 slices; wide slices +
# interleaved tiles (UH=32, TI=2); ragged with interleave; ...; narrow slices with two tiles, with four
# tiles of which one is missing, and with two chunks of interleaved tiles (4 + 1)
FWD_SHAPES = [(3, 128, 64), (5, 200, 128), (8, 256, 256), (4, 64, 1024), (6, 1300, 512), (4, 2304, 256),
              (40, 96, 256), (3, 32, 2048), (5, 130, 1536), (4, 384, 1024), (5, 640, 1024), (3, 1280, 1024), (5, 130, 768),
              (5, 1024, 512), (3, 4800, 64)]


def _desc(dtype, T, B, H, flags=0):
    return _lib.Desc(_lib.DTYPE_CODE[dtype], T, B, H, H, flags, 0, 0)


def _fwd(lib, d, pre, Wh, h0, c0):
    T, B, H = d.seq_len, d.batch, d.hidden_size
    ifgo = pre.clone()
    st = torch.zeros(2, T + 1, B, H, device="cuda", dtype=pre.dtype)
    st[0, 0], st[1, 0] = h0, c0
    n = lib.blstm_workspace_bytes(d, _lib.PHASE_FWD)
    ws = torch.zeros(n, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.blstm_fwd_recurrence(d, ifgo.data_ptr(), Wh.data_ptr(), st[0].data_ptr(), st[1].data_ptr(),
                                        ws.data_ptr(), n, s), "fwd_recurrence")
    _lib.check(lib.blstm_read_status(ws.data_ptr(), None, s), "status")
    return ifgo, st[0], st[1]


def _torch_fwd(pre, Wh, h0, c0):
    """fp32 math with h fed back at storage precision (what both kernels do)."""
    T, B, G = pre.shape
    H = G // 4
    dt = pre.dtype
    W = Wh.float()
    h, c = h0.float(), c0.float()
    outs, cells, gates = [], [], []
    for t in range(T):
        a = pre[t].float() + h @ W.T
        gates.append(a)
        i, f, g, o = a.split(H, dim=1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        h = (torch.sigmoid(o) * torch.tanh(c)).to(dt).float()
        outs.append(h)
        cells.append(c)
    return torch.stack(gates), torch.stack(outs), torch.stack(cells)


def _cmp(name, got, ref, atol):
    err = (got.float() - ref.float()).abs()
    if float(err.max()) > atol:
        idx = (err > atol).nonzero()
        first = idx[0].tolist()
        rows = sorted(set(idx[:, -2].tolist()))
        cols = sorted(set(idx[:, -1].tolist()))
        ts = sorted(set(idx[:, 0].tolist()))
        pytest.fail(f"{name}: max err {float(err.max()):.4g} > {atol}; {idx.shape[0]}/{err.numel()} bad; first {first} "
                    f"got {float(got[tuple(first)]):.5g} want {float(ref[tuple(first)]):.5g}; t {ts[:6]} "
                    f"rows {rows[:6]}..{rows[-1]} cols {cols[:6]}..{cols[-1]}")


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("shape", FWD_SHAPES)
def test_forward_recurrence(dtype, shape):
    lib = _lib.load()
    T, B, H = shape
    dt = TD[dtype]
    g = torch.Generator(device="cuda").manual_seed(B + H)
    pre = (torch.randn(T, B, 4 * H, generator=g, device="cuda")).to(dt)
    Wh = ((torch.rand(4 * H, H, generator=g, device="cuda") * 2 - 1) / H ** 0.5).to(dt)
    h0 = (torch.randn(B, H, generator=g, device="cuda") * 0.3).to(dt)
    c0 = (torch.randn(B, H, generator=g, device="cuda") * 0.3).to(dt)
    d = _desc(dtype, T, B, H)
    assert lib.blstm_plan_name(d, 0) == b"sm100"
    ifgo, out, cell = _fwd(lib, d, pre, Wh, h0, c0)
    rg, ro, rc = _torch_fwd(pre, Wh, h0, c0)
    tol = 4e-3 if dtype == "fp16" else 3e-2
    _cmp("ifgo", ifgo, rg, tol * 4)
    _cmp("out", out[1:], ro, tol)
    _cmp("cell", cell[1:], rc, tol * 2)
    # and against the CUDA-core kernels
    ifgo2, out2, cell2 = _fwd(lib, _desc(dtype, T, B, H, _lib.FLAG_FORCE_GENERIC), pre, Wh, h0, c0)
    _cmp("out vs generic", out, out2, tol)
    _cmp("cell vs generic", cell, cell2, tol * 2)
    # bit-identical when repeated
    ifgo3, out3, _ = _fwd(lib, d, pre, Wh, h0, c0)
    assert torch.equal(out, out3) and torch.equal(ifgo, ifgo3)


BWD_SHAPES = [(3, 128, 64), (5, 200, 128), (8, 256, 256), (4, 64, 1024), (6, 1300, 512), (1, 40, 64), (30, 96, 256),
              (3, 32, 2048), (4, 130, 1536), (4, 384, 1024), (5, 640, 1024), (3, 1280, 1024), (5, 130, 768),
              (4, 2304, 256), (5, 1024, 512), (4, 640, 512), (3, 4800, 64), (3, 400, 768), (3, 2000, 320),
              (5, 2560, 512), (3, 4096, 512)]


def _bwd(lib, d, dout, dh_n, dc_n, ifgo, cell, Wh):
    T, B, H = d.seq_len, d.batch, d.hidden_size
    dg = torch.full((T, B, 4 * H), float("nan"), device="cuda", dtype=ifgo.dtype)
    dh0 = torch.full((B, H), float("nan"), device="cuda", dtype=ifgo.dtype)
    dc0 = torch.full((B, H), float("nan"), device="cuda", dtype=ifgo.dtype)
    db = torch.full((4 * H,), float("nan"), device="cuda")
    n = lib.blstm_workspace_bytes(d, _lib.PHASE_BWD)
    ws = torch.zeros(n, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.blstm_bwd_recurrence(d, dout.data_ptr(), dh_n.data_ptr(), dc_n.data_ptr(), ifgo.data_ptr(),
                                        cell.data_ptr(), Wh.data_ptr(), dg.data_ptr(), dh0.data_ptr(),
                                        dc0.data_ptr(), db.data_ptr(), ws.data_ptr(), n, s), "bwd_recurrence")
    _lib.check(lib.blstm_read_status(ws.data_ptr(), None, s), "status")
    return dg, dh0, dc0, db


def _torch_bwd(dout, dh_n, dc_n, ifgo, cell, Wh):
    """fp32 evaluation of the reverse recurrence, independent of both CUDA kernels: d_ifgo[t] is
    rounded to the storage type before it feeds dh[t-1] = d_ifgo[t] x Wh (the kernels read it back
    at storage precision); the dh and dc carries stay fp32.  Equations: fastlstm/kernels.py:1291-1316
    and :1362-1383."""
    T, B, G = ifgo.shape
    H = G // 4
    dt = ifgo.dtype
    W = Wh.float()
    dh_c, dc = dh_n.float(), dc_n.float()
    dgs = [None] * T
    for t in reversed(range(T)):
        pi, pf, pg, po = ifgo[t].float().split(H, dim=1)
        si, sf, so, tg = torch.sigmoid(pi), torch.sigmoid(pf), torch.sigmoid(po), torch.tanh(pg)
        tc = torch.tanh(cell[t + 1].float())
        dh = dout[t].float() + dh_c
        dcv = dc + dh * so * (1 - tc * tc)
        d = torch.cat([dcv * tg * si * (1 - si), dcv * cell[t].float() * sf * (1 - sf),
                       dcv * si * (1 - tg * tg), dh * tc * so * (1 - so)], dim=1).to(dt)
        dgs[t] = d
        dc = dcv * sf
        dh_c = d.float() @ W
    return torch.stack(dgs), dh_c, dc


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("shape", BWD_SHAPES)
def test_backward_recurrence(dtype, shape):
    lib = _lib.load()
    T, B, H = shape
    dt = TD[dtype]
    g = torch.Generator(device="cuda").manual_seed(B * 3 + H)
    ifgo = torch.randn(T, B, 4 * H, generator=g, device="cuda").to(dt)
    cell = (torch.randn(T + 1, B, H, generator=g, device="cuda") * 0.7).to(dt)
    dout = torch.randn(T, B, H, generator=g, device="cuda").to(dt)
    dh_n = torch.randn(B, H, generator=g, device="cuda").to(dt)
    dc_n = torch.randn(B, H, generator=g, device="cuda").to(dt)
    Wh = ((torch.rand(4 * H, H, generator=g, device="cuda") * 2 - 1) / H ** 0.5).to(dt)
    d = _desc(dtype, T, B, H)
    assert lib.blstm_plan_name(d, 1) == b"sm100"
    got = _bwd(lib, d, dout, dh_n, dc_n, ifgo, cell, Wh)
    ref = _bwd(lib, _desc(dtype, T, B, H, _lib.FLAG_FORCE_GENERIC), dout, dh_n, dc_n, ifgo, cell, Wh)
    tol = 6e-3 if dtype == "fp16" else 4e-2
    scale = float(ref[0].float().abs().max())
    _cmp("d_ifgo", got[0], ref[0], tol * max(scale, 1.0))
    _cmp("dh0", got[1][None], ref[1][None], tol * max(float(ref[1].float().abs().max()), 1.0))
    _cmp("dc0", got[2][None], ref[2][None], tol * max(float(ref[2].float().abs().max()), 1.0))
    assert torch.allclose(got[3], got[0].float().sum(dim=(0, 1)), rtol=1e-4, atol=1e-3 * T * B ** 0.5)
    # and against independent fp32 maths (not only the library's other kernel)
    rg, rh, rc = _torch_bwd(dout, dh_n, dc_n, ifgo, cell, Wh)
    _cmp("d_ifgo vs fp32 maths", got[0], rg, tol * max(float(rg.float().abs().max()), 1.0))
    _cmp("dh0 vs fp32 maths", got[1][None], rh[None], tol * max(float(rh.abs().max()), 1.0))
    _cmp("dc0 vs fp32 maths", got[2][None], rc[None], tol * max(float(rc.abs().max()), 1.0))
    again = _bwd(lib, d, dout, dh_n, dc_n, ifgo, cell, Wh)
    assert torch.equal(got[0], again[0]) and torch.equal(got[1], again[1]) and torch.equal(got[3], again[3])


# One tile in flight (arrivals by the epilogue warps) and interleaved tiles (arrivals by the
# publisher warp; for the backward kernel also the cluster exchange has to give up cleanly).
@pytest.mark.parametrize("shape", [(4, 128, 64), (4, 1300, 512)])
@pytest.mark.parametrize("phase", ["fwd", "bwd"])
def test_tensor_core_kernels_give_up_with_a_status_when_nothing_arrives(phase, shape):
    """Failure detection without a fault: with the test hook that suppresses every arrival the
    bounded waits of the tcgen05 kernels run out (20 ms), every role leaves its loop, the kernel
    returns, the control block holds BLSTM_E_WAIT_TIMEOUT, and the next ordinary launch works."""
    import ctypes
    lib = _lib.load()
    T, B, H = shape
    dt = torch.bfloat16
    d = _lib.Desc(_lib.DTYPE_CODE["bf16"], T, B, H, H, _lib.FLAG_TEST_NO_ARRIVE, 20000, 0)
    assert lib.blstm_plan_name(d, 0 if phase == "fwd" else 1) == b"sm100"
    s = torch.cuda.current_stream().cuda_stream
    z = lambda *shape_: torch.zeros(*shape_, device="cuda", dtype=dt)
    Wh = z(4 * H, H)
    detail = (ctypes.c_int32 * 2)()
    if phase == "fwd":
        n = lib.blstm_workspace_bytes(d, _lib.PHASE_FWD)
        ws = torch.zeros(n, dtype=torch.uint8, device="cuda")
        ifgo, out, cell = z(T, B, 4 * H), z(T + 1, B, H), z(T + 1, B, H)
        assert lib.blstm_fwd_recurrence(d, ifgo.data_ptr(), Wh.data_ptr(), out.data_ptr(), cell.data_ptr(),
                                        ws.data_ptr(), n, s) == 0
    else:
        n = lib.blstm_workspace_bytes(d, _lib.PHASE_BWD)
        ws = torch.zeros(n, dtype=torch.uint8, device="cuda")
        ifgo, cell, dout, dg = z(T, B, 4 * H), z(T + 1, B, H), z(T, B, H), z(T, B, 4 * H)
        dh0, dc0 = z(B, H), z(B, H)
        assert lib.blstm_bwd_recurrence(d, dout.data_ptr(), None, None, ifgo.data_ptr(), cell.data_ptr(),
                                        Wh.data_ptr(), dg.data_ptr(), dh0.data_ptr(), dc0.data_ptr(), None,
                                        ws.data_ptr(), n, s) == 0
    assert lib.blstm_read_status(ws.data_ptr(), detail, s) == _lib.E_WAIT_TIMEOUT
    # the context is intact: the same problem without the hook runs to completion
    ok = _lib.Desc(_lib.DTYPE_CODE["bf16"], T, B, H, H, 0, 0, 0)
    ws.zero_()
    if phase == "fwd":
        assert lib.blstm_fwd_recurrence(ok, ifgo.data_ptr(), Wh.data_ptr(), out.data_ptr(), cell.data_ptr(),
                                        ws.data_ptr(), n, s) == 0
    else:
        assert lib.blstm_bwd_recurrence(ok, dout.data_ptr(), None, None, ifgo.data_ptr(), cell.data_ptr(),
                                        Wh.data_ptr(), dg.data_ptr(), dh0.data_ptr(), dc0.data_ptr(), None,
                                        ws.data_ptr(), n, s) == 0
    assert lib.blstm_read_status(ws.data_ptr(), None, s) == 0


# generic fp32; tcgen05 with one tile in flight, two and four interleaved tiles (16 units per CTA) and
# 32 units per CTA with two interleaved tiles
INFERENCE_CASES = [("fp32", 5, 40, 48), ("bf16", 6, 128, 256), ("fp16", 5, 2304, 256), ("bf16", 4, 1280, 1024),
                   ("bf16", 6, 1300, 512)]


@pytest.mark.parametrize("case", INFERENCE_CASES)
def test_inference_flag_leaves_outputs_bit_identical(case):
    """BLSTM_FLAG_INFERENCE skips the stores only backward needs: out[1..T] and cell[T] must be
    bit-identical to a training-mode launch, and the saved tensors must really stay unwritten."""
    lib = _lib.load()
    dtype, T, B, H = case
    dt = {"fp32": torch.float32, **TD}[dtype]
    g = torch.Generator(device="cuda").manual_seed(T * B + H)
    pre = torch.randn(T, B, 4 * H, generator=g, device="cuda").to(dt)
    Wh = ((torch.rand(4 * H, H, generator=g, device="cuda") * 2 - 1) / H ** 0.5).to(dt)
    h0 = (torch.randn(B, H, generator=g, device="cuda") * 0.3).to(dt)
    c0 = (torch.randn(B, H, generator=g, device="cuda") * 0.3).to(dt)
    train = _desc(dtype, T, B, H)
    infer = _desc(dtype, T, B, H, _lib.FLAG_INFERENCE)
    _, out1, cell1 = _fwd(lib, train, pre, Wh, h0, c0)
    ifgo2, out2, cell2 = _fwd(lib, infer, pre, Wh, h0, c0)
    assert torch.equal(out1, out2)
    assert torch.equal(cell1[T], cell2[T])
    assert torch.equal(ifgo2, pre), "inference mode wrote the saved pre-activations"
    if T > 1:
        assert float(cell2[1:T].abs().max()) == 0.0, "inference mode wrote cell[1..T-1]"


# one cluster of 4, 8 and 16 CTAs; ragged tile; seven tiles (the most clusters of 16 that fit at once)
CLUSTER_SHAPES = [(7, 64, 64), (9, 100, 128), (12, 64, 256), (5, 896, 256), (1, 40, 256)]


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("shape", CLUSTER_SHAPES)
def test_cluster_hand_off_forward_matches_general_kernel(dtype, shape):
    """Small hidden sizes hand h over inside one cluster per batch tile (shared memory, no counters).
    Against the general tcgen05 kernel on the same inputs (BLSTM_FLAG_NO_CLUSTER) the results may only
    differ by the order of the fp32 partial sums, and both must agree with fp32 maths."""
    lib = _lib.load()
    T, B, H = shape
    dt = TD[dtype]
    g = torch.Generator(device="cuda").manual_seed(7 * B + H)
    pre = torch.randn(T, B, 4 * H, generator=g, device="cuda").to(dt)
    Wh = ((torch.rand(4 * H, H, generator=g, device="cuda") * 2 - 1) / H ** 0.5).to(dt)
    h0 = (torch.randn(B, H, generator=g, device="cuda") * 0.3).to(dt)
    c0 = (torch.randn(B, H, generator=g, device="cuda") * 0.3).to(dt)
    import ctypes
    buf = ctypes.create_string_buffer(512)
    assert lib.blstm_plan_detail(_desc(dtype, T, B, H), 0, buf, 512) == 0 and b"cluster=" in buf.value, buf.value
    ifgo, out, cell = _fwd(lib, _desc(dtype, T, B, H), pre, Wh, h0, c0)
    ifgo2, out2, cell2 = _fwd(lib, _desc(dtype, T, B, H, _lib.FLAG_NO_CLUSTER), pre, Wh, h0, c0)
    rg, ro, rc = _torch_fwd(pre, Wh, h0, c0)
    tol = 4e-3 if dtype == "fp16" else 3e-2
    _cmp("out vs fp32 maths", out[1:], ro, tol)
    _cmp("cell vs fp32 maths", cell[1:], rc, tol * 2)
    _cmp("ifgo vs fp32 maths", ifgo, rg, tol * 4)
    _cmp("out vs general kernel", out, out2, tol)
    _cmp("ifgo vs general kernel", ifgo, ifgo2, tol * 4)
    ifgo3, out3, _ = _fwd(lib, _desc(dtype, T, B, H), pre, Wh, h0, c0)
    assert torch.equal(out, out3) and torch.equal(ifgo, ifgo3)


# Geometry sweep: every hidden size class against batches of one row, a ragged second tile, more tiles
# than CTA rows, and far more (two steps are enough to cross a hand-off in each direction).
SWEEP_SHAPES = [(2, B, H) for H in (64, 192, 320, 640, 1280, 2048) for B in (1, 129, 1300, 4800)]


@pytest.mark.parametrize("shape", SWEEP_SHAPES)
def test_both_recurrences_over_a_sweep_of_geometries(shape):
    lib = _lib.load()
    T, B, H = shape
    dtype, dt = "bf16", torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(B * 7 + H)
    pre = torch.randn(T, B, 4 * H, generator=g, device="cuda").to(dt)
    Wh = ((torch.rand(4 * H, H, generator=g, device="cuda") * 2 - 1) / H ** 0.5).to(dt)
    h0 = (torch.randn(B, H, generator=g, device="cuda") * 0.3).to(dt)
    c0 = (torch.randn(B, H, generator=g, device="cuda") * 0.3).to(dt)
    d = _desc(dtype, T, B, H)
    assert lib.blstm_plan_name(d, 0) == b"sm100" and lib.blstm_plan_name(d, 1) == b"sm100"
    ifgo, out, cell = _fwd(lib, d, pre, Wh, h0, c0)
    rg, ro, rc = _torch_fwd(pre, Wh, h0, c0)
    _cmp("ifgo", ifgo, rg, 0.12)
    _cmp("out", out[1:], ro, 3e-2)
    _cmp("cell", cell[1:], rc, 6e-2)
    dout = torch.randn(T, B, H, generator=g, device="cuda").to(dt)
    dh_n = torch.randn(B, H, generator=g, device="cuda").to(dt)
    dc_n = torch.randn(B, H, generator=g, device="cuda").to(dt)
    got = _bwd(lib, d, dout, dh_n, dc_n, ifgo, cell, Wh)
    wg, wh, wc = _torch_bwd(dout, dh_n, dc_n, ifgo, cell, Wh)
    _cmp("d_ifgo", got[0], wg, 4e-2 * max(float(wg.float().abs().max()), 1.0))
    _cmp("dh0", got[1][None], wh[None], 4e-2 * max(float(wh.abs().max()), 1.0))
    _cmp("dc0", got[2][None], wc[None], 4e-2 * max(float(wc.abs().max()), 1.0))
    assert torch.allclose(got[3], got[0].float().sum(dim=(0, 1)), rtol=1e-4, atol=1e-3 * T * B ** 0.5)
