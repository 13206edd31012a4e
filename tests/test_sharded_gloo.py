"""world_size-2 gloo test of the batch-sharding host logic (CPU, no GPU): per-shard weight
gradients (computed by the oracle, since the kernels need a GPU) summed through GradBucket's
single allreduce must equal the full-batch gradients, and shard outputs concatenate exactly."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fastlstm_b200.sharded import GradBucket, shard_batch, shard_bounds


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import lstm_oracle as O
    rng = np.random.default_rng(11)
    T, B, I, H = 6, 10, 5, 4
    Wx, Wh = rng.uniform(-.5, .5, (4 * H, I)), rng.uniform(-.5, .5, (4 * H, H))
    bx, bh = rng.uniform(-.5, .5, 4 * H), rng.uniform(-.5, .5, 4 * H)
    x, dout = rng.standard_normal((T, B, I)), rng.standard_normal((T, B, H))
    xs = shard_batch(torch.tensor(x), rank, world).numpy()
    ds = shard_batch(torch.tensor(dout), rank, world).numpy()
    r = O.stacked_fwd_bwd(xs, None, None, [(Wx, Wh, bx, bh)], dout=ds)
    m = torch.nn.LSTM(I, H)           # only a parameter container with nn.LSTM's names
    bucket = GradBucket(m)
    bucket.attach()
    dWx, dWh, db = r["grads"][0]
    m.weight_ih_l0.grad.copy_(torch.tensor(dWx))
    m.weight_hh_l0.grad.copy_(torch.tensor(dWh))
    m.bias_ih_l0.grad.copy_(torch.tensor(db))
    m.bias_hh_l0.grad.copy_(torch.tensor(db))
    bucket.allreduce()
    outs = [None] * world
    dist.all_gather_object(outs, r["out"])
    if rank == 0:
        full = O.stacked_fwd_bwd(x, None, None, [(Wx, Wh, bx, bh)], dout=dout)
        ok = np.array_equal(np.concatenate(outs, axis=1), full["out"])
        fW, fH, fb = full["grads"][0]
        ok &= np.allclose(m.weight_ih_l0.grad.numpy(), fW, rtol=1e-5, atol=1e-6)
        ok &= np.allclose(m.weight_hh_l0.grad.numpy(), fH, rtol=1e-5, atol=1e-6)
        ok &= np.allclose(m.bias_hh_l0.grad.numpy(), fb, rtol=1e-5, atol=1e-6)
        q.put(bool(ok))
    dist.barrier()
    dist.destroy_process_group()


def _sink_worker(rank, world, port, q, dtype_name):
    """FastLSTM + GradBucket: each layer's fp32 gradients are written into the bucket's segment
    (here by the oracle standing in for the kernels, which need a GPU), the segment's allreduce is
    started from `filled()`, and allreduce() hands the sums to p.grad in the parameter dtype."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fastlstm_b200 import FastLSTM
    from oracle import lstm_oracle as O
    dt = {"fp32": torch.float32, "bf16": torch.bfloat16}[dtype_name]
    T, B, I, H, L = 5, 10, 6, 4, 2
    torch.manual_seed(3)
    m = FastLSTM(I, H, num_layers=L, dtype=dt)       # parameters only: forward needs a GPU
    rng = np.random.default_rng(5)
    x, dout = rng.standard_normal((T, B, I)), rng.standard_normal((T, B, H))
    f = lambda p: p.detach().double().numpy()
    params = [tuple(f(p) for p in m.layer_params(l)) for l in range(L)]
    params = [(Wx, Wh, bx, bh) for (Wx, bx, Wh, bh) in params]
    xs = shard_batch(torch.tensor(x), rank, world).numpy()
    ds = shard_batch(torch.tensor(dout), rank, world).numpy()
    r = O.stacked_fwd_bwd(xs, None, None, params, dout=ds)
    bucket = GradBucket(m)
    for p in m.parameters():
        p.grad = None                                  # what optimizer.zero_grad() leaves behind
    bucket.attach()
    assert m._sinks is not None and len(m._sinks) == L
    for l in reversed(range(L)):                       # backward order: last layer first
        dWx, dWh, db = r["grads"][l]
        flat = np.concatenate([dWx.ravel(), dWh.ravel(), db.ravel()])
        m._sinks[l].buffer.copy_(torch.tensor(flat, dtype=torch.float32))
        m._sinks[l].filled()
    bucket.allreduce()
    if rank == 0:
        full = O.stacked_fwd_bwd(x, None, None, params, dout=dout)
        tol = dict(rtol=1e-5, atol=1e-6) if dt == torch.float32 else dict(rtol=2e-2, atol=2e-2)
        ok = True
        for l in range(L):
            fW, fH, fb = full["grads"][l]
            Wx, bx, Wh, bh = m.layer_params(l)
            for p, want in ((Wx, fW), (Wh, fH), (bx, fb), (bh, fb)):
                ok &= p.grad is not None and p.grad.dtype == dt
                ok &= np.allclose(p.grad.double().numpy(), want, **tol)
            ok &= bx.grad is not bh.grad and bx.grad.data_ptr() != bh.grad.data_ptr()
        q.put(bool(ok))
    dist.barrier()
    dist.destroy_process_group()


def _run_two_ranks(target, *extra):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, 2, port, q) + extra) for r in range(2)]
    for p in procs:
        p.start()
    codes = []
    for p in procs:
        p.join(120)
        if p.is_alive():                     # a hung worker must not outlive the test session
            p.kill()
            p.join(10)
        codes.append(p.exitcode)
    assert codes == [0, 0], codes
    assert q.get(timeout=5) is True


def test_two_rank_gloo_grad_allreduce_matches_full_batch():
    _run_two_ranks(_worker)


def test_two_rank_gloo_fastlstm_sinks_fp32_and_bf16():
    _run_two_ranks(_sink_worker, "fp32")
    _run_two_ranks(_sink_worker, "bf16")


def test_plain_module_scatter_after_grads_were_reset():
    """fp32 parameters whose .grad was set to None after attach(): allreduce() must still leave the
    summed gradients in p.grad (single process: the sum is the identity)."""
    m = torch.nn.LSTM(3, 2)
    bucket = GradBucket(m)
    bucket.attach()
    for p in m.parameters():
        p.grad = None
    for i, p in enumerate(m.parameters()):
        p.grad = torch.full_like(p, float(i + 1))
    bucket.allreduce()
    for i, (p, v) in enumerate(zip(bucket.params, bucket.views)):
        assert p.grad is v and float(v.flatten()[0]) == float(i + 1)


def test_shard_bounds_cover_batch_without_overlap():
    for B in (1, 7, 4096):
        for w in (1, 2, 3, 8):
            spans = [shard_bounds(B, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
