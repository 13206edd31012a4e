"""Host side of the B200 LSTM layer: the reference's module surface over the C ABI.

Mirrors oleicht/FastLSTM `fastlstm/lstm.py`:

  lstm_persistent_fwd   <- fastlstm/lstm.py:31-146
  lstm_persistent_bwd   <- fastlstm/lstm.py:236-334
  Wgrad                 <- fastlstm/lstm.py:494-501
  PersistentLSTMfn      <- fastlstm/lstm.py:504-538
  FastLSTM              <- fastlstm/lstm.py:586-698

Differences (all additions): `bias` and `batch_first` constructor arguments,
gradients through the returned (h_n, c_n), fp32 weight/bias gradients, fp32
matmuls stay fp32 (the reference flips the global TF32 switch on import,
fastlstm/lstm.py:15-19; this module does not).  PyTorch is used for device
memory, streams and autograd only; every device computation goes through
libfastlstm_b200.so and there is no fallback path.
"""
from __future__ import annotations

import os
import threading

import torch
import torch.nn as nn

from . import _lib

_DTYPE_CODE = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}

# Set FASTLSTM_B200_SYNC_CHECK=1 to read the device status word (and wait for
# the stream) after every recurrence launch; otherwise it is read lazily.
_SYNC_CHECK = os.environ.get("FASTLSTM_B200_SYNC_CHECK", "0") == "1"
_FORCE_GENERIC = os.environ.get("FASTLSTM_B200_FORCE_GENERIC", "0") == "1"
_WAIT_LIMIT_US = int(os.environ.get("FASTLSTM_B200_WAIT_LIMIT_US", "0"))


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _desc(dtype, T, B, I, H, flags=0):
    if dtype not in _DTYPE_CODE:
        raise ValueError(f"unsupported dtype {dtype}; expected float32, float16 or bfloat16")
    if _FORCE_GENERIC:
        flags |= _lib.FLAG_FORCE_GENERIC
    return _lib.Desc(_DTYPE_CODE[dtype], T, B, I, H, flags, _WAIT_LIMIT_US, 0)


def _require(t, name, dtype=None, shape=None, device=None):
    if t is None:
        return
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if device is not None and t.device != device:
        raise ValueError(f"{name} is on {t.device}, expected {device}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")


# ---------------------------------------------------------------------------
# Deferred device-status checks: each recurrence launch leaves a status word in
# its workspace; it is copied to pinned memory on the same stream and examined
# once the copy has completed (at a later call, or in check_status()).
# ---------------------------------------------------------------------------
class _StatusRing:
    def __init__(self):
        self.lock = threading.Lock()
        self.pending = []   # (event, pinned tensor, label)
        self.free = []

    def push(self, ws, label):
        with self.lock:
            host = self.free.pop() if self.free else torch.empty(4, dtype=torch.int32, pin_memory=True)
        host.copy_(ws[:16].view(torch.int32), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(ws.device))
        with self.lock:
            self.pending.append((ev, host, label))

    def poll(self, wait=False):
        with self.lock:
            items, self.pending = self.pending, []
        keep, err = [], None
        for ev, host, label in items:
            if wait:
                ev.synchronize()
            if ev.query():
                code = int(host[1])
                if code != 0 and err is None:
                    err = (code, label, int(host[2]), int(host[3]))
                with self.lock:
                    self.free.append(host)
            else:
                keep.append((ev, host, label))
        with self.lock:
            self.pending = keep + self.pending
        if err is not None:
            code, label, d0, d1 = err
            raise _lib.BlstmError(code, f"{label} (step {d0}, batch tile {d1})")


_status = _StatusRing()


def check_status(wait: bool = True):
    """Raise if any finished launch recorded a device-side error (a bounded wait
    that ran out).  With wait=True, first waits for all outstanding launches."""
    _status.poll(wait=wait)


def _after_launch(desc, ws, label):
    if _SYNC_CHECK:
        rc = _lib.load().blstm_read_status(ws.data_ptr(), None, _stream(ws))
        _lib.check(rc, label)
    else:
        _status.push(ws, label)
        _status.poll(wait=False)


_PHASES = {"fwd": _lib.PHASE_FWD, "bwd": _lib.PHASE_BWD, "fwd_op": _lib.PHASE_FWD_OP}


def plan_name(dtype, T, B, I, H, phase="fwd"):
    """Kernel family ("generic" / "sm100", for phase "fwd_op" also "fused") the library picks for this
    problem.  Phases: "fwd" / "bwd" = the recurrences, "fwd_op" = the whole forward operator."""
    d = _desc(dtype, T, B, I, H)
    return _lib.load().blstm_plan_name(d, _PHASES[phase]).decode()


def plan_detail(dtype, T, B, I, H, phase="fwd"):
    """One-line description of the launch geometry the library picks for this problem."""
    import ctypes
    d = _desc(dtype, T, B, I, H)
    buf = ctypes.create_string_buffer(512)
    _lib.check(_lib.load().blstm_plan_detail(d, _PHASES[phase], buf, 512), "blstm_plan_detail")
    return buf.value.decode()


# ---------------------------------------------------------------------------
# Operator functions (same names and argument meaning as the reference)
# ---------------------------------------------------------------------------
def lstm_persistent_fwd(x, h0, c0, Wx, bx, Wh, bh, inference=False, half_device=False):
    """Forward of one layer.  x [T,B,I]; h0,c0 [B,H] or None; Wx [4H,I]; Wh [4H,H];
    bx,bh [4H] or None.  Returns (out[T+1,B,H], cell[T+1,B,H], ifgo[T,B,4H]);
    slot 0 of out/cell is the initial state.  (fastlstm/lstm.py:31-146)
    inference=True: nothing is saved for backward - ifgo and cell[1..T-1] are left unwritten
    (cell[T] is still c_n), which halves the bytes each step moves.
    half_device=True: the recurrence is planned for half of the SMs (two layers side by side)."""
    lib = _lib.load()
    if x.dim() == 2:
        x = x[None]
    T, B, I = x.shape
    H = Wh.shape[1]
    dt, dev = x.dtype, x.device
    _require(x, "x")
    _require(Wx, "Wx", dt, (4 * H, I), dev)
    _require(Wh, "Wh", dt, (4 * H, H), dev)
    _require(bx, "bx", dt, (4 * H,), dev)
    _require(bh, "bh", dt, (4 * H,), dev)
    if (h0 is None) != (c0 is None):
        raise ValueError("h0 and c0 must both be given or both be None")
    _require(h0, "h0", dt, (B, H), dev)
    _require(c0, "c0", dt, (B, H), dev)
    d = _desc(dt, T, B, I, H, (_lib.FLAG_INFERENCE if inference else 0) | (_lib.FLAG_HALF_DEVICE if half_device else 0))
    with torch.cuda.device(dev):
        states = torch.empty((2, T + 1, B, H), device=dev, dtype=dt)
        out, cell = states.unbind(0)
        ifgo = torch.empty((T, B, 4 * H), device=dev, dtype=dt)
        ws_bytes = lib.blstm_workspace_bytes(d, _lib.PHASE_FWD)
        ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
        rc = lib.blstm_fwd(d, _ptr(x), _ptr(h0), _ptr(c0), _ptr(Wx), _ptr(Wh), _ptr(bx), _ptr(bh),
                           _ptr(out), _ptr(cell), _ptr(ifgo), _ptr(ws), ws_bytes, _stream(x))
        _lib.check(rc, "blstm_fwd")
        _after_launch(d, ws, "forward recurrence")
    return out, cell, ifgo


def lstm_persistent_bwd(dh, dc_n, dh_n, x, h, cell, ifgo, Wx, Wh, need_dx=True, wgrads=None, half_device=False):
    """Backward of one layer.  dh [T,B,H] gradient of out[1:]; dc_n, dh_n [B,H]
    (or None) gradients of the final states; h = out[T+1,B,H] from forward.
    Returns (d_x, dh_0, dc_0, dWx, dbx, dWh, dbh); weight and bias gradients are
    fp32, dbx is dbh.  (fastlstm/lstm.py:236-334)
    wgrads: optional flat fp32 tensor of 4H*(I+H+1) elements laid out dWx | dWh | db that the
    kernels write into (a data-parallel gradient bucket); allocated here when None."""
    lib = _lib.load()
    T, B, H = dh.shape
    I = x.shape[-1]
    dt, dev = x.dtype, x.device
    dh = dh.contiguous()
    _require(dh, "dh", dt, (T, B, H), dev)
    _require(dh_n, "dh_n", dt, (B, H), dev)
    _require(dc_n, "dc_n", dt, (B, H), dev)
    _require(h, "h", dt, (T + 1, B, H), dev)
    _require(cell, "cell", dt, (T + 1, B, H), dev)
    _require(ifgo, "ifgo", dt, (T, B, 4 * H), dev)
    d = _desc(dt, T, B, I, H, _lib.FLAG_HALF_DEVICE if half_device else 0)
    with torch.cuda.device(dev):
        d_ifgo = torch.empty_like(ifgo)
        d_x = torch.empty((T, B, I), device=dev, dtype=dt) if need_dx else None
        carries = torch.empty((2, B, H), device=dev, dtype=dt)
        dh_0, dc_0 = carries.unbind(0)
        if wgrads is None:
            wgrads = torch.empty(4 * H * (I + H + 1), device=dev, dtype=torch.float32)
        _require(wgrads, "wgrads", torch.float32, (4 * H * (I + H + 1),), dev)
        dWx = wgrads[:4 * H * I].view(4 * H, I)
        dWh = wgrads[4 * H * I:4 * H * (I + H)].view(4 * H, H)
        db = wgrads[4 * H * (I + H):]
        ws_bytes = lib.blstm_workspace_bytes(d, _lib.PHASE_BWD)
        ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
        rc = lib.blstm_bwd(d, _ptr(dh), _ptr(dh_n), _ptr(dc_n), _ptr(x), _ptr(h), _ptr(cell),
                           _ptr(ifgo), _ptr(Wx), _ptr(Wh), _ptr(d_ifgo), _ptr(d_x), _ptr(dh_0),
                           _ptr(dc_0), _ptr(dWx), _ptr(dWh), _ptr(db), _ptr(ws), ws_bytes, _stream(x))
        _lib.check(rc, "blstm_bwd")
        _after_launch(d, ws, "backward recurrence")
    return d_x, dh_0, dc_0, dWx, db, dWh, db


def Wgrad(d_ifgo, x, h):
    """(dbx, dbh, dWx, dWh) from d_ifgo [T,B,4H], x [T,B,I], h = out[T+1,B,H].
    (fastlstm/lstm.py:494-501; fp32 results, no transpose copy)"""
    lib = _lib.load()
    T, B, G = d_ifgo.shape
    H, I = G // 4, x.shape[-1]
    d = _desc(x.dtype, T, B, I, H)
    dev = x.device
    with torch.cuda.device(dev):
        dWx = torch.empty((G, I), device=dev, dtype=torch.float32)
        dWh = torch.empty((G, H), device=dev, dtype=torch.float32)
        ws_bytes = lib.blstm_workspace_bytes(d, _lib.PHASE_BWD)
        ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
        rc = lib.blstm_wgrad(d, _ptr(d_ifgo), _ptr(x), _ptr(h), _ptr(dWx), _ptr(dWh), _ptr(ws),
                             ws_bytes, _stream(x))
        _lib.check(rc, "blstm_wgrad")
        db = torch.empty(G, device=dev, dtype=torch.float32)
        rc = lib.blstm_bias_grad(d, _ptr(d_ifgo), _ptr(db), _ptr(ws), ws_bytes, _stream(x))
        _lib.check(rc, "blstm_bias_grad")
    return db, db, dWx, dWh


# ---------------------------------------------------------------------------
# Ragged 16-bit shapes on the tensor-core kernels: TMA wants 16-byte row pitches (I % 8 == 0) and the
# tcgen05 recurrences hidden sizes in multiples of 64.  Other shapes are zero-padded on the host: a padded
# hidden unit has zero weights, bias and state, so its pre-activations are 0, its cell and output stay
# exactly 0 and it feeds nothing into the real units; padded input columns meet zero weights.  The
# padded copies cost a few small kernels per call - far less than the CUDA-core kernels they replace.
# ---------------------------------------------------------------------------
def _padded_sizes(dtype, I, H):
    """(Ip, Hp) when the layer should run zero-padded on the tensor-core kernels, else None."""
    if dtype not in (torch.float16, torch.bfloat16) or _FORCE_GENERIC:
        return None
    if max(I, H) <= 64:                       # tiny sizes have the fused kernel
        return None
    Ip, Hp = -(-I // 8) * 8, -(-H // 64) * 64
    if (Ip, Hp) == (I, H) or Hp > 2048:
        return None
    return Ip, Hp


def _pad_last(t, n):
    return t if t is None or t.shape[-1] == n else torch.nn.functional.pad(t, (0, n - t.shape[-1]))


def _pad_gates(W, H, Hp, cols=None):
    """[4H, K] (or [4H]) -> [4Hp, cols or K]: every gate's block padded with zero rows (and columns)."""
    if W is None:
        return None
    if W.dim() == 1:
        return torch.nn.functional.pad(W.view(4, H), (0, Hp - H)).reshape(4 * Hp)
    K = W.shape[1]
    cols = K if cols is None else cols
    return torch.nn.functional.pad(W.view(4, H, K), (0, cols - K, 0, Hp - H)).reshape(4 * Hp, cols)


def _unpad_gates(G, H, Hp, cols=None):
    """inverse of _pad_gates for gradients: [4Hp, Kp] -> [4H, cols]."""
    if G.dim() == 1:
        return G.view(4, Hp)[:, :H].reshape(4 * H)
    cols = G.shape[1] if cols is None else cols
    return G.view(4, Hp, G.shape[1])[:, :H, :cols].reshape(4 * H, cols)


class PersistentLSTMfn(torch.autograd.Function):
    """autograd Function of one layer (fastlstm/lstm.py:504-538).

    forward(x, h_0, c_0, Wx, bx, Wh, bh) -> (out[T,B,H], h_n[B,H], c_n[B,H]);
    unlike the reference, h_n and c_n are flat outputs and differentiable."""

    @staticmethod
    def forward(ctx, x, h_0, c_0, Wx, bx, Wh, bh, inference=None, sink=None, want_cells=False):
        if torch.is_autocast_enabled("cuda"):
            target = torch.get_autocast_dtype("cuda")
            x, Wx, Wh = x.to(target), Wx.to(target), Wh.to(target)
            bx = None if bx is None else bx.to(target)
            bh = None if bh is None else bh.to(target)
            h_0 = None if h_0 is None else h_0.to(target)
            c_0 = None if c_0 is None else c_0.to(target)
        x = x.contiguous()
        I, H = x.shape[-1], Wh.shape[1]
        ctx.pad = _padded_sizes(x.dtype, I, H)
        ctx.sizes = (I, H)
        if ctx.pad is not None:
            Ip, Hp = ctx.pad
            x = _pad_last(x, Ip)
            Wx, Wh = _pad_gates(Wx, H, Hp, Ip), _pad_gates(Wh, H, Hp, Hp)
            bx, bh = _pad_gates(bx, H, Hp), _pad_gates(bh, H, Hp)
            h_0, c_0 = _pad_last(h_0, Hp), _pad_last(c_0, Hp)
        # Grad mode is always off inside Function.forward and needs_input_grad mirrors requires_grad
        # whatever the grad mode, so the caller (persistent_lstm / FastLSTM.forward) decides whether
        # anything has to be saved; a bare apply() with the reference's seven arguments saves unless
        # no input requires a gradient.
        if inference is None:
            inference = not any(ctx.needs_input_grad)
        ctx.inference = bool(inference)
        ctx.sink = sink
        with torch.autograd.profiler.record_function("fastlstm_b200::fwd"):
            out, cell, ifgo = lstm_persistent_fwd(
                x, None if h_0 is None else h_0.contiguous(), None if c_0 is None else c_0.contiguous(),
                Wx.contiguous(), bx, Wh.contiguous(), bh, inference=inference)
        ctx.h0_is_none = h_0 is None
        ctx.has_bias = (bx is not None, bh is not None)
        ctx.save_for_backward(x, out, cell, ifgo, Wx, Wh)
        ctx.want_cells = bool(want_cells)
        res = (out[1:, :, :H], out[-1, :, :H], cell[-1, :, :H]) if ctx.pad is not None else (out[1:], out[-1], cell[-1])
        if want_cells:
            # cell states of every step, for callers that need c at a step other than the last (packed
            # sequences of different lengths); no gradient flows back through this output
            cells = cell[1:, :, :H] if ctx.pad is not None else cell[1:]
            ctx.mark_non_differentiable(cells)
            return res + (cells,)
        return res

    @staticmethod
    def backward(ctx, d_out, d_hn, d_cn, *_):
        if ctx.inference:
            raise RuntimeError("this forward ran in inference mode (nothing was saved); backward is not possible")
        x, out, cell, ifgo, Wx, Wh = ctx.saved_tensors
        T, B, H = out.shape[0] - 1, out.shape[1], out.shape[2]
        if d_out is None:
            d_out = torch.zeros((T, B, H), device=x.device, dtype=x.dtype)
        d_out = d_out.to(x.dtype)
        d_hn = None if d_hn is None else d_hn.to(x.dtype)
        d_cn = None if d_cn is None else d_cn.to(x.dtype)
        if ctx.pad is not None:
            d_out, d_hn, d_cn = _pad_last(d_out, H), _pad_last(d_hn, H), _pad_last(d_cn, H)   # H is the padded size here
        d_out = d_out.contiguous()
        d_hn = None if d_hn is None else d_hn.contiguous()
        d_cn = None if d_cn is None else d_cn.contiguous()
        with torch.autograd.profiler.record_function("fastlstm_b200::bwd"):
            d_x, dh_0, dc_0, dWx, dbx, dWh, dbh = lstm_persistent_bwd(
                d_out, d_cn, d_hn, x, out, cell, ifgo, Wx.contiguous(), Wh.contiguous(),
                need_dx=ctx.needs_input_grad[0],
                wgrads=None if (ctx.sink is None or ctx.pad is not None) else ctx.sink.buffer)
        if ctx.pad is not None:
            I0, H0 = ctx.sizes
            d_x = None if d_x is None else d_x[..., :I0]
            dh_0, dc_0 = dh_0[:, :H0], dc_0[:, :H0]
            dWx, dWh = _unpad_gates(dWx, H0, H, I0), _unpad_gates(dWh, H0, H, H0)
            dbx = dbh = _unpad_gates(dbx, H0, H)
        if ctx.h0_is_none:
            dh_0 = dc_0 = None
        if ctx.sink is not None and ctx.pad is not None:
            # padded layer: the kernels wrote padded gradients, the bucket takes the unpadded ones
            n1, n2 = dWx.numel(), dWx.numel() + dWh.numel()
            ctx.sink.buffer[:n1].copy_(dWx.reshape(-1))
            ctx.sink.buffer[n1:n2].copy_(dWh.reshape(-1))
            ctx.sink.buffer[n2:].copy_(dbx)
        if ctx.sink is not None:
            # the fp32 gradients went straight into the caller's bucket segment: autograd sees none
            # (it would round them to the parameter dtype), the bucket hands them to p.grad later
            ctx.sink.filled()
            return (d_x, dh_0, dc_0, None, None, None, None, None, None, None)
        return (d_x, dh_0, dc_0, dWx, dbx if ctx.has_bias[0] else None, dWh,
                dbh if ctx.has_bias[1] else None, None, None, None)


_side_streams = {}


def _side_stream(device):
    """One extra stream per device for the layer wavefront (created once, reused)."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=key)
    return _side_streams[key]


class WavefrontLSTMfn(torch.autograd.Function):
    """A unidirectional stack of layers as ONE autograd node that runs the layers as a wavefront over
    time chunks: layer l works on chunk k while layer l-1 works on chunk k+1, on two streams, each
    recurrence planned for half of the SMs (the reference runs the layers one after the other,
    fastlstm/lstm.py:685-696, and lists the wavefront as missing, README.md:94).  It pays when a
    layer alone cannot fill the GPU: few batch tiles, every CTA with one tile, every step one
    hand-off chain.  A chunk is an ordinary call of the layer operators with the previous chunk's
    final state as its initial state (the cell state crosses a chunk boundary in the storage dtype).

    forward(x[T,B,I], n_chunks, sinks, inference, h0, c0, *params) with params = (Wx, bx, Wh, bh) per
    layer, h0/c0 [L,B,H] or None  ->  (out[T,B,H], h_n[L,B,H], c_n[L,B,H]).  inference=True: nothing is
    saved for backward and the recurrences skip the stores only backward needs."""

    @staticmethod
    def forward(ctx, x, n_chunks, sinks, inference, h0, c0, *params):
        L = len(params) // 4
        T = x.shape[0]
        x = x.contiguous()
        bounds = [(T * k) // n_chunks for k in range(n_chunks + 1)]
        chunks = [(bounds[k], bounds[k + 1]) for k in range(n_chunks) if bounds[k + 1] > bounds[k]]
        NC = len(chunks)
        main = torch.cuda.current_stream(x.device)
        streams = [main, _side_stream(x.device)]
        streams[1].wait_stream(main)
        saved = [[None] * NC for _ in range(L)]
        done = [[None] * NC for _ in range(L)]
        with torch.autograd.profiler.record_function("fastlstm_b200::wavefront_fwd"):
            for diag in range(NC + L - 1):
                for l in range(L):
                    k = diag - l
                    if k < 0 or k >= NC:
                        continue
                    Wx, bx, Wh, bh = params[4 * l:4 * l + 4]
                    st = streams[l % 2]
                    if l > 0:
                        st.wait_event(done[l - 1][k])
                    with torch.cuda.stream(st):
                        t0, t1 = chunks[k]
                        xc = x[t0:t1] if l == 0 else saved[l - 1][k][1][1:]
                        if k == 0:
                            hp = None if h0 is None else h0[l].contiguous()
                            cp = None if c0 is None else c0[l].contiguous()
                        else:
                            hp, cp = saved[l][k - 1][1][-1], saved[l][k - 1][2][-1]
                        out, cell, ifgo = lstm_persistent_fwd(xc, hp, cp, Wx.contiguous(), bx, Wh.contiguous(), bh,
                                                              inference=bool(inference), half_device=True)
                        saved[l][k] = (xc, out, cell, None if inference else ifgo)
                        done[l][k] = torch.cuda.Event()
                        done[l][k].record(st)
            # every later use (the concatenation below, backward, the allocator) comes after both streams
            main.wait_stream(streams[1])
            streams[1].wait_stream(main)
            top = saved[L - 1]
            y = torch.cat([top[k][1][1:] for k in range(NC)], dim=0) if NC > 1 else top[0][1][1:].clone()
            h_n = torch.stack([saved[l][NC - 1][1][-1] for l in range(L)])
            c_n = torch.stack([saved[l][NC - 1][2][-1] for l in range(L)])
        ctx.inference = bool(inference)
        if not inference:
            ctx.saved = saved
            ctx.params = params
            ctx.sinks = sinks
            ctx.chunks = chunks
            ctx.had_state = h0 is not None
        return y, h_n, c_n

    @staticmethod
    def backward(ctx, d_out, d_hn, d_cn):
        if ctx.inference:
            raise RuntimeError("this forward ran in inference mode (nothing was saved); backward is not possible")
        saved, params, chunks, sinks = ctx.saved, ctx.params, ctx.chunks, ctx.sinks
        L, NC = len(saved), len(chunks)
        x0 = saved[0][0][0]
        dt, dev = x0.dtype, x0.device
        B, H = saved[0][0][1].shape[1], saved[0][0][1].shape[2]
        main = torch.cuda.current_stream(dev)
        streams = [main, _side_stream(dev)]
        streams[1].wait_stream(main)
        d_out = None if d_out is None else d_out.to(dt).contiguous()
        d_hn = None if d_hn is None else d_hn.to(dt).contiguous()
        d_cn = None if d_cn is None else d_cn.to(dt).contiguous()
        need_dx0 = ctx.needs_input_grad[0]
        dx = [[None] * NC for _ in range(L)]
        carry = [[None] * NC for _ in range(L)]
        done = [[None] * NC for _ in range(L)]
        acc = [None] * L
        with torch.autograd.profiler.record_function("fastlstm_b200::wavefront_bwd"):
            for diag in range(NC + L - 1):
                for li in range(L):
                    l = L - 1 - li
                    k = NC - 1 - (diag - li)
                    if k < 0 or k >= NC:
                        continue
                    Wx, bx, Wh, bh = params[4 * l:4 * l + 4]
                    st = streams[l % 2]
                    if l < L - 1:
                        st.wait_event(done[l + 1][k])
                    with torch.cuda.stream(st):
                        xc, out, cell, ifgo = saved[l][k]
                        t0, t1 = chunks[k]
                        if l == L - 1:
                            dh = d_out[t0:t1] if d_out is not None else torch.zeros((t1 - t0, B, H), device=dev, dtype=dt)
                        else:
                            dh = dx[l + 1][k]
                        if k == NC - 1:
                            dh_n = None if d_hn is None else d_hn[l]
                            dc_n = None if d_cn is None else d_cn[l]
                        else:
                            dh_n, dc_n = carry[l][k + 1]
                        I = xc.shape[-1]
                        first = acc[l] is None
                        buf = torch.empty(4 * H * (I + H + 1), device=dev, dtype=torch.float32)
                        d_x, dh_0, dc_0, _, _, _, _ = lstm_persistent_bwd(
                            dh, dc_n, dh_n, xc, out, cell, ifgo, Wx.contiguous(), Wh.contiguous(),
                            need_dx=(l > 0 or need_dx0), wgrads=buf, half_device=True)
                        if first:
                            acc[l] = buf
                        else:
                            acc[l].add_(buf)
                        dx[l][k], carry[l][k] = d_x, (dh_0, dc_0)
                        if k == 0 and sinks is not None:
                            # the layer's fp32 gradients go straight into its bucket segment, whose
                            # all-reduce starts here, beside the backward of the layers below
                            sinks[l].buffer.copy_(acc[l])
                            sinks[l].filled()
                        done[l][k] = torch.cuda.Event()
                        done[l][k].record(st)
            main.wait_stream(streams[1])
            streams[1].wait_stream(main)
            d_x = None
            if need_dx0:
                d_x = torch.cat(dx[0], dim=0) if NC > 1 else dx[0][0]
            dh0 = dc0 = None
            if ctx.had_state:
                dh0 = torch.stack([carry[l][0][0] for l in range(L)])
                dc0 = torch.stack([carry[l][0][1] for l in range(L)])
        grads = []
        for l in range(L):
            Wx, bx, Wh, bh = params[4 * l:4 * l + 4]
            if sinks is not None:
                grads += [None, None, None, None]
                continue
            I = Wx.shape[1]
            dWx = acc[l][:4 * H * I].view(4 * H, I)
            dWh = acc[l][4 * H * I:4 * H * (I + H)].view(4 * H, H)
            db = acc[l][4 * H * (I + H):]
            grads += [dWx, db if bx is not None else None, dWh, db if bh is not None else None]
        return (d_x, None, None, None, dh0, dc0, *grads)


def _nothing_to_save(*tensors):
    """True when no backward can follow this forward: grad mode is off, or no input requires one."""
    return not (torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors))


def persistent_lstm(x, h_0, c_0, Wx, bx, Wh, bh):
    """Reference-shaped call: returns (out, (h_n, c_n)) like PersistentLSTMfn.apply
    does in fastlstm/lstm.py:522."""
    inference = _nothing_to_save(x, h_0, c_0, Wx, bx, Wh, bh)
    out, h_n, c_n = PersistentLSTMfn.apply(x, h_0, c_0, Wx, bx, Wh, bh, inference, None)
    return out, (h_n, c_n)


class FastLSTM(nn.Module):
    """nn.LSTM-style stacked LSTM on the B200 kernels (fastlstm/lstm.py:586-698).

    Parameters have nn.LSTM's names, shapes, registration order, init distribution and RNG order
    (weight_ih_l{k}[_reverse], weight_hh_l{k}[_reverse], bias_ih_l{k}[_reverse],
    bias_hh_l{k}[_reverse]), so state dicts are interchangeable with torch.nn.LSTM.  `version` is
    accepted for source compatibility; only "persistent" exists here.

    Beyond the reference (which lists them as missing, README.md:92-93): `bidirectional` runs the
    same kernels on the time-reversed input and concatenates the two directions' outputs
    (states are ordered layer-major, direction-minor, like nn.LSTM); `dropout` is applied to
    the outputs of every layer but the last while training; a `PackedSequence` input gives a
    `PackedSequence` output and the states at every sequence's own last step.  `proj_size` > 0 adds
    nn.LSTM's output projection (`weight_hr_l{k}`: h_t = W_hr (o * tanh(c_t)), recurrent weights
    [4H, proj_size]); a projected layer runs step by step - one launch of the cell per timestep
    with the projection between the steps - which is complete but not fast."""

    def __init__(self, input_size, hidden_size, num_layers=1, *, bias=True, batch_first=False,
                 version="persistent", device=None, dtype=None, dropout=0.0, bidirectional=False,
                 proj_size=0):
        # Everything after num_layers is keyword-only: the reference's positional order continues with
        # (version, device, dtype), nn.LSTM's with (bias, batch_first, dropout, ...); a positional call
        # written for either would silently bind the wrong option here, so it raises TypeError instead.
        super().__init__()
        if not isinstance(bias, bool) or not isinstance(batch_first, bool):
            raise TypeError("bias and batch_first must be bool")
        if version != "persistent":
            raise ValueError(f"Not implemented: {version} (only 'persistent' exists)")
        if not isinstance(proj_size, int) or proj_size < 0:
            raise ValueError("proj_size should be a positive integer or zero to disable projections")
        if proj_size >= hidden_size:
            raise ValueError("proj_size has to be a positive integer, smaller than hidden_size")
        if not 0.0 <= float(dropout) <= 1.0:
            raise ValueError("dropout should be a number in range [0, 1]")
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.bias, self.batch_first, self.version = bias, batch_first, version
        self.dropout, self.bidirectional = float(dropout), bool(bidirectional)
        self.num_directions = 2 if bidirectional else 1
        self.proj_size = proj_size
        self._sinks = None            # per (layer, direction) gradient sinks of a GradBucket, or None
        k = 1.0 / hidden_size ** 0.5
        fk = dict(device=device, dtype=dtype)

        def u(*shape):
            return nn.Parameter(torch.rand(*shape, **fk) * 2 * k - k)

        out_size = proj_size if proj_size > 0 else hidden_size       # width of h (and of a layer's output)
        for layer in range(num_layers):
            in_l = input_size if layer == 0 else out_size * self.num_directions
            for sfx in self._suffixes():
                setattr(self, f"weight_ih_l{layer}{sfx}", u(4 * hidden_size, in_l))
                setattr(self, f"weight_hh_l{layer}{sfx}", u(4 * hidden_size, out_size))
                if bias:
                    setattr(self, f"bias_ih_l{layer}{sfx}", u(4 * hidden_size))
                    setattr(self, f"bias_hh_l{layer}{sfx}", u(4 * hidden_size))
                if proj_size > 0:
                    setattr(self, f"weight_hr_l{layer}{sfx}", u(proj_size, hidden_size))

    def _suffixes(self):
        return ("", "_reverse") if self.bidirectional else ("",)

    def layer_params(self, layer, reverse=False):
        sfx = "_reverse" if reverse else ""
        g = lambda n: getattr(self, f"{n}_l{layer}{sfx}", None)
        return g("weight_ih"), g("bias_ih"), g("weight_hh"), g("bias_hh")

    def _projected_layer(self, x_d, h0, c0, Wx, bx, Wh, bh, Whr, inference):
        """One direction of one layer with an output projection (nn.LSTM's proj_size): the recurrent
        input is the projected state, so the layer is run as T single-step calls of the cell (the same
        operator with T = 1; the projected state is zero-padded to the cell's width and `Wh` [4H,P] to
        [4H,H], which is exact) with the projection h_t = (o * tanh(c_t)) W_hr^T in between.  Autograd
        chains the steps.  Returns (out [T,B,P], cells [T,B,H], h_n [B,P], c_n [B,H])."""
        T, B = x_d.shape[0], x_d.shape[1]
        H, P = self.hidden_size, self.proj_size
        pad = torch.nn.functional.pad
        Wh_wide = pad(Wh, (0, H - P))
        h = x_d.new_zeros(B, P) if h0 is None else h0
        c = c0
        outs, cells = [], []
        for t in range(T):
            o, _, c = PersistentLSTMfn.apply(x_d[t:t + 1], pad(h, (0, H - P)), c, Wx, bx, Wh_wide, bh, inference, None)
            h = o[0] @ Whr.t()
            outs.append(h)
            cells.append(c)
        return torch.stack(outs), torch.stack(cells), h, c

    def forward(self, x, h_c_0=None):
        if isinstance(x, torch.nn.utils.rnn.PackedSequence):
            return self._forward_packed(x, h_c_0)
        if x.dim() != 3:
            raise ValueError("expected a 3-D input [T,B,I] (or [B,T,I] with batch_first)")
        if self.batch_first:
            x = x.transpose(0, 1)
        return self._forward_padded(x, h_c_0, None)

    def _forward_packed(self, seq, h_c_0):
        """PackedSequence input (torch.nn.LSTM's convention; the reference lists it as missing,
        README.md:92-93).  The sequences are padded to the longest, every layer runs over all T steps
        (steps past a sequence's end compute values nobody reads - the recurrence is causal), the
        final states are read at each sequence's own last step, and the output is packed again with
        the input's ordering.  The reverse direction of a bidirectional layer walks every sequence
        from its own end.  Gradients flow through the packed output and h_n; c_n of sequences shorter
        than the longest carries no gradient."""
        from torch.nn.utils.rnn import PackedSequence, pack_padded_sequence, pad_packed_sequence
        x, lengths = pad_packed_sequence(seq, batch_first=False)          # [T,B,I], original batch order
        out, states = self._forward_padded(x, h_c_0, lengths.to(x.device))
        if seq.sorted_indices is not None:
            out, lengths = out.index_select(1, seq.sorted_indices), lengths[seq.sorted_indices.cpu()]
        data = pack_padded_sequence(out, lengths, enforce_sorted=True).data
        return PackedSequence(data, seq.batch_sizes, seq.sorted_indices, seq.unsorted_indices), states

    def _wavefront_chunks(self, x, h_c_0, lengths):
        """Number of time chunks for the layer wavefront, or 0 when the stack runs layer after layer.
        The wavefront needs two or more layers of one direction on the tensor-core kernels and pays
        when a layer alone leaves the GPU latency bound: every CTA has a single batch tile on the
        whole device and at most two on half of it."""
        if os.environ.get("FASTLSTM_B200_WAVEFRONT", "1") == "0":
            return 0
        if (self.num_layers < 2 or self.num_directions != 1 or self.proj_size > 0 or lengths is not None
                or (self.dropout > 0.0 and self.training) or not x.is_cuda
                or x.dtype not in (torch.float16, torch.bfloat16) or torch.is_autocast_enabled("cuda")):
            return 0
        T, B, I = x.shape
        H = self.hidden_size
        if H % 64 != 0 or H > 1024 or I % 8 != 0 or T < 64:
            return 0
        if any(p.dtype != x.dtype for p in self.parameters()):
            return 0
        sms = 148
        tiles, ctas_per_tile = -(-B // 128), H // 16
        if ctas_per_tile > sms // 2:          # (a single tile's CTAs must fit on half of the SMs)
            return 0
        if tiles > sms // ctas_per_tile or tiles > 2 * ((sms // 2) // ctas_per_tile):
            return 0
        return max(1, min(int(os.environ.get("FASTLSTM_B200_WAVEFRONT_CHUNKS", "4")), T // 16))

    def _forward_wavefront(self, x, h_c_0, n_chunks):
        h0 = c0 = None
        if h_c_0 is not None:
            h0, c0 = h_c_0
            if h0 is None or c0 is None:
                raise ValueError("h_c_0 must be a pair (h_0, c_0) of [num_layers, B, H] tensors or None")
            h0 = torch.stack(list(h0)) if not torch.is_tensor(h0) else h0
            c0 = torch.stack(list(c0)) if not torch.is_tensor(c0) else c0
            if h0.shape[0] != self.num_layers or c0.shape[0] != self.num_layers:
                raise ValueError(f"expected {self.num_layers} initial states, got {h0.shape[0]} / {c0.shape[0]}")
            h0, c0 = h0.to(x.dtype), c0.to(x.dtype)
        params = []
        for layer in range(self.num_layers):
            params += list(self.layer_params(layer))
        inference = _nothing_to_save(x, h0, c0, *params)
        out, h_n, c_n = WavefrontLSTMfn.apply(x, n_chunks, self._sinks, inference, h0, c0, *params)
        if self.batch_first:
            out = out.transpose(0, 1)
        return out, (h_n, c_n)

    def _forward_padded(self, x, h_c_0, lengths):
        """x [T,B,I]; lengths: None, or the [B] valid lengths (device tensor) of padded sequences."""
        n_chunks = self._wavefront_chunks(x, h_c_0, lengths)
        if n_chunks:
            return self._forward_wavefront(x, h_c_0, n_chunks)
        nd = self.num_directions
        T, B = x.shape[0], x.shape[1]
        if lengths is not None:
            steps = torch.arange(T, device=x.device)[:, None]                       # [T,1]
            valid = steps < lengths[None, :]                                         # [T,B]
            # per-sequence time reversal (identity past the end) and the index of the last valid step
            rev = torch.where(valid, lengths[None, :] - 1 - steps, steps)            # [T,B]
            last = (lengths - 1).clamp(min=0)                                        # [B]

            def reverse_time(t):
                return t.gather(0, rev[:, :, None].expand(-1, -1, t.shape[2]))

            def at_last(t):                                                          # [T,B,H] -> [B,H]
                return t.gather(0, last[None, :, None].expand(1, -1, t.shape[2]))[0]
        if h_c_0 is None:
            h_0 = c_0 = [None] * (self.num_layers * nd)
        else:
            h_0, c_0 = h_c_0
            if h_0 is None or c_0 is None:
                raise ValueError("h_c_0 must be a pair (h_0, c_0) of [num_layers * num_directions, B, H] "
                                 "tensors or None")
            if len(h_0) != self.num_layers * nd or len(c_0) != self.num_layers * nd:
                raise ValueError(f"expected {self.num_layers * nd} initial states, got {len(h_0)} / {len(c_0)}")
        h_n, c_n = [], []
        for layer in range(self.num_layers):
            outs = []
            for d in range(nd):
                Wx, bx, Wh, bh = self.layer_params(layer, reverse=(d == 1))
                # the reverse direction walks t = T-1 .. 0 (every sequence from its own end when packed)
                x_d = x if d == 0 else (x.flip(0) if lengths is None else reverse_time(x))
                hl, cl = h_0[layer * nd + d], c_0[layer * nd + d]
                inference = _nothing_to_save(x_d, hl, cl, Wx, bx, Wh, bh)
                sink = None if self._sinks is None else self._sinks[layer * nd + d]
                if self.proj_size > 0:
                    Whr = getattr(self, f"weight_hr_l{layer}{'_reverse' if d == 1 else ''}")
                    if hl is not None and cl is None or hl is None and cl is not None:
                        raise ValueError("h_0 and c_0 must both be given or both be None")
                    cl_ = x_d.new_zeros(B, self.hidden_size) if cl is None else cl
                    o, cells, h_i, c_i = self._projected_layer(x_d, hl, cl_, Wx, bx, Wh, bh, Whr, inference)
                    if lengths is not None:
                        h_i, c_i = at_last(o), at_last(cells)
                        o = o * valid[:, :, None].to(o.dtype)
                elif lengths is None:
                    o, h_i, c_i = PersistentLSTMfn.apply(x_d, hl, cl, Wx, bx, Wh, bh, inference, sink)
                else:
                    o, _, _, cells = PersistentLSTMfn.apply(x_d, hl, cl, Wx, bx, Wh, bh, inference, sink, True)
                    h_i, c_i = at_last(o), at_last(cells)      # states at each sequence's own last step
                    o = o * valid[:, :, None].to(o.dtype)      # steps past the end read as zeros
                outs.append(o if d == 0 else (o.flip(0) if lengths is None else reverse_time(o)))
                h_n.append(h_i)
                c_n.append(c_i)
            x = outs[0] if nd == 1 else torch.cat(outs, dim=-1)
            if self.dropout > 0.0 and self.training and layer < self.num_layers - 1:
                x = torch.nn.functional.dropout(x, self.dropout, True)
        if self.batch_first and lengths is None:
            x = x.transpose(0, 1)
        return x, (torch.stack(h_n), torch.stack(c_n))
