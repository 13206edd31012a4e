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


def test_two_rank_gloo_grad_allreduce_matches_full_batch():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


def test_shard_bounds_cover_batch_without_overlap():
    for B in (1, 7, 4096):
        for w in (1, 2, 3, 8):
            spans = [shard_bounds(B, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
