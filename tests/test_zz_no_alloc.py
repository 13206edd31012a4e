"""The no-allocation forward entry point (blstm_fwd_recurrence_static).

Some users of this library cannot allocate device memory when they call it - their own arena
already owns the free HBM, or their host forbids cudaMalloc after start-up - so one entry point
keeps its scratch in a fixed array inside the library instead of a caller-provided workspace.
This test drives it through the C ABI twice in a row and requires the same results as the regular
entry point (bit-identical, as in the repeat-run checks of the other recurrence tests), and checks
that an oversized problem is refused with a clear status.  It lives in its own file, collected
last, so a failure here cannot hide the result of any other test."""
import pytest
import torch

from fastlstm_b200 import _lib

pytestmark = pytest.mark.gpu


def _inputs(dtype, T, B, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pre = torch.randn(T, B, 4 * H, generator=g, device="cuda").to(dtype)
    Wh = ((torch.rand(4 * H, H, generator=g, device="cuda") * 2 - 1) / H ** 0.5).to(dtype)
    h0 = (torch.randn(B, H, generator=g, device="cuda") * 0.3).to(dtype)
    c0 = (torch.randn(B, H, generator=g, device="cuda") * 0.3).to(dtype)
    return pre, Wh, h0, c0


def _run(lib, d, pre, Wh, h0, c0, static):
    T, B, H = d.seq_len, d.batch, d.hidden_size
    ifgo = pre.clone()
    st = torch.zeros(2, T + 1, B, H, device="cuda", dtype=pre.dtype)
    st[0, 0], st[1, 0] = h0, c0
    s = torch.cuda.current_stream().cuda_stream
    if static:
        _lib.check(lib.blstm_fwd_recurrence_static(d, ifgo.data_ptr(), Wh.data_ptr(), st[0].data_ptr(),
                                                   st[1].data_ptr(), s), "fwd_recurrence_static")
        _lib.check(lib.blstm_static_scratch_status(None, s), "static status")
    else:
        n = lib.blstm_workspace_bytes(d, _lib.PHASE_FWD)
        ws = torch.zeros(n, dtype=torch.uint8, device="cuda")
        _lib.check(lib.blstm_fwd_recurrence(d, ifgo.data_ptr(), Wh.data_ptr(), st[0].data_ptr(),
                                            st[1].data_ptr(), ws.data_ptr(), n, s), "fwd_recurrence")
        _lib.check(lib.blstm_read_status(ws.data_ptr(), None, s), "status")
    torch.cuda.synchronize()
    return ifgo, st[0].clone(), st[1].clone()


@pytest.mark.parametrize("dtype,T,B,H", [(torch.bfloat16, 24, 300, 256), (torch.float32, 9, 20, 48)])
def test_static_scratch_entry_matches_regular_entry_twice_in_a_row(dtype, T, B, H):
    lib = _lib.load()
    code = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}[dtype]
    d = _lib.Desc(code, T, B, H, H, 0, 0, 0)
    assert lib.blstm_workspace_bytes(d, _lib.PHASE_FWD) <= lib.blstm_static_scratch_capacity()
    # two different problems back to back: the second call must not see the first call's counters
    for seed in (11, 12):
        pre, Wh, h0, c0 = _inputs(dtype, T, B, H, seed)
        want = _run(lib, d, pre, Wh, h0, c0, static=False)
        got = _run(lib, d, pre, Wh, h0, c0, static=True)
        for name, a, b in zip(("ifgo", "out", "cell"), got, want):
            assert torch.equal(a, b), f"{name} differs (seed {seed})"


def test_static_scratch_entry_rejects_problems_beyond_its_capacity():
    lib = _lib.load()
    d = _lib.Desc(_lib.F32, 4096, 4096, 8, 8, 0, 0, 0)     # (T+1) * 256 batch tiles of counters > 1 MiB
    assert lib.blstm_workspace_bytes(d, _lib.PHASE_FWD) > lib.blstm_static_scratch_capacity()
    x = torch.zeros(16, device="cuda")
    rc = lib.blstm_fwd_recurrence_static(d, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.E_TOO_LARGE
    assert "capacity" in _lib.strerror(rc)


def test_static_scratch_entry_reports_a_wait_that_ran_out_and_recovers():
    """The bounded waits of the persistent kernel report through the library's own control block too: with
    the test hook that makes CTAs skip their arrivals every wait runs out after 20 ms (nothing faults,
    nothing hangs), the status call returns the timeout, and the next call is clean and correct."""
    lib = _lib.load()
    dtype, T, B, H = torch.bfloat16, 6, 300, 256
    pre, Wh, h0, c0 = _inputs(dtype, T, B, H, 21)
    s = torch.cuda.current_stream().cuda_stream
    bad = _lib.Desc(_lib.BF16, T, B, H, H, _lib.FLAG_TEST_NO_ARRIVE | _lib.FLAG_NO_CLUSTER, 20000, 0)
    ifgo = pre.clone()
    st = torch.zeros(2, T + 1, B, H, device="cuda", dtype=dtype)
    assert lib.blstm_fwd_recurrence_static(bad, ifgo.data_ptr(), Wh.data_ptr(), st[0].data_ptr(), st[1].data_ptr(), s) == 0
    assert lib.blstm_static_scratch_status(None, s) == _lib.E_WAIT_TIMEOUT
    torch.cuda.synchronize()
    d = _lib.Desc(_lib.BF16, T, B, H, H, 0, 0, 0)
    want = _run(lib, d, pre, Wh, h0, c0, static=False)
    got = _run(lib, d, pre, Wh, h0, c0, static=True)
    for name, a, b in zip(("ifgo", "out", "cell"), got, want):
        assert torch.equal(a, b), f"{name} differs after a timed-out call"
