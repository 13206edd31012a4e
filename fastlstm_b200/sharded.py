"""Batch-sharded data parallelism for the LSTM layer.

The batch dimension is the only natural shard of the path: batch rows never
interact in the forward or in the backward recurrence, only the weight-gradient
sums run over the batch.  Each rank therefore runs the full single-GPU path on
its slice of the batch and the ranks sum one flat fp32 bucket holding every
layer's dWx, dWh and db (NCCL over NVLink on GPUs, gloo in the CPU tests).
The reference (oleicht/FastLSTM) has no distributed code; this file has no
counterpart there.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(global_batch: int, rank: int, world: int):
    """[lo, hi) rows of the global batch owned by `rank`; the first
    global_batch % world ranks get one extra row."""
    base, rem = divmod(global_batch, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch(t: torch.Tensor, rank: int, world: int, batch_dim: int = 1):
    lo, hi = shard_bounds(t.shape[batch_dim], rank, world)
    return t.narrow(batch_dim, lo, hi - lo).contiguous()


class GradSink:
    """One (layer, direction)'s fp32 segment of a GradBucket, laid out dWx | dWh | db - the layout
    the weight-gradient kernels write.  PersistentLSTMfn.backward writes into `buffer` and then
    calls `filled()`, which lets the bucket start that segment's allreduce at once."""

    def __init__(self, bucket, index, buffer):
        self.bucket, self.index, self.buffer = bucket, index, buffer

    def filled(self):
        self.bucket._segment_filled(self.index)


class GradBucket:
    """One flat fp32 buffer holding every parameter gradient of a module.

    For a FastLSTM the bucket is cut into one segment per (layer, direction) in the kernels' own
    layout (dWx | dWh | db; the two biases of a layer share the db slot since their gradients are
    identical).  After `attach()` the backward of each layer writes its fp32 gradients straight
    into its segment - autograd never sees them, so nothing is rounded to a 16-bit parameter dtype
    before the cross-rank sum - and the segment's allreduce is started right there, asynchronously,
    so that it runs beside the backward of the layers below.  `allreduce()` then waits for the
    segments and hands the sums to p.grad, converting to the parameter dtype once.  One forward
    and one backward per `allreduce()`: a second backward would overwrite, not accumulate.

    For any other module the bucket is the concatenation of the parameters in order: `attach()`
    points fp32 p.grad at it, `allreduce()` copies gradients that are not views of it
    in (and back out), and sums in a single collective."""

    def __init__(self, module: torch.nn.Module, overlap: bool = True):
        self.module = module
        self.overlap = overlap
        self.params = [p for p in module.parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("module has no trainable parameters")
        dev = self.params[0].device
        self.sinks = None
        self._pending = []          # (segment index, work handle or None)
        self._filled = set()
        from .lstm import FastLSTM
        if isinstance(module, FastLSTM) and module.proj_size == 0:    # (projected layers: plain-module path)
            self._init_segments(module, dev)
        else:
            n = sum(p.numel() for p in self.params)
            self.flat = torch.zeros(n, device=dev, dtype=torch.float32)
            self.views = []
            off = 0
            for p in self.params:
                self.views.append(self.flat[off:off + p.numel()].view_as(p))
                off += p.numel()
        self._direct = all(p.dtype == torch.float32 for p in self.params)

    # ------------------------------------------------------------------ FastLSTM: per-layer segments
    def _init_segments(self, m, dev):
        H, nd = m.hidden_size, m.num_directions
        sizes = []
        for layer in range(m.num_layers):
            in_l = m.input_size if layer == 0 else H * nd
            sizes += [4 * H * (in_l + H + 1)] * nd
        self.flat = torch.zeros(sum(sizes), device=dev, dtype=torch.float32)
        self.sinks, self.segments = [], []      # segments: (buffer, [(param, view, shared?)...])
        off = 0
        for idx, n in enumerate(sizes):
            layer, d = divmod(idx, nd)
            in_l = m.input_size if layer == 0 else H * nd
            buf = self.flat[off:off + n]
            off += n
            Wx, bx, Wh, bh = m.layer_params(layer, reverse=(d == 1))
            a, b = 4 * H * in_l, 4 * H * (in_l + H)
            entries = [(Wx, buf[:a].view(4 * H, in_l), False), (Wh, buf[a:b].view(4 * H, H), False)]
            if bx is not None:
                entries += [(bx, buf[b:], False), (bh, buf[b:], True)]
            self.segments.append((buf, entries))
            self.sinks.append(GradSink(self, idx, buf))

    def _segment_filled(self, idx):
        self._filled.add(idx)
        work = None
        if self.overlap and dist.is_initialized() and dist.get_world_size() > 1:
            work = dist.all_reduce(self.segments[idx][0], op=dist.ReduceOp.SUM, async_op=True)
        self._pending.append((idx, work))

    # ------------------------------------------------------------------ common surface
    def attach(self):
        """FastLSTM: route the layers' weight gradients into the bucket.  Other modules: point fp32
        p.grad at the bucket and zero it."""
        self._pending, self._filled = [], set()
        if self.sinks is not None:
            self.module._sinks = self.sinks
            return
        self.flat.zero_()
        if self._direct:
            for p, v in zip(self.params, self.views):
                p.grad = v

    def detach(self):
        if self.sinks is not None:
            self.module._sinks = None

    def gather(self):
        """Copy p.grad into the bucket when the gradients are not views of it (plain modules)."""
        if self.sinks is not None:
            return
        for p, v in zip(self.params, self.views):
            if p.grad is v:
                continue
            v.copy_(p.grad if p.grad is not None else torch.zeros_like(v))

    def scatter(self):
        """Hand the bucket's contents to p.grad (converted to the parameter dtype once)."""
        if self.sinks is not None:
            for _, entries in self.segments:
                for p, v, shared in entries:
                    g = v if p.dtype == torch.float32 else v.to(p.dtype)
                    # the second bias gets a tensor of its own: in-place gradient clipping must not
                    # scale one shared tensor twice
                    p.grad = g.clone() if (shared and p.dtype == torch.float32) else g
            return
        for p, v in zip(self.params, self.views):
            if p.dtype == torch.float32:
                if p.grad is not v:
                    p.grad = v
            else:
                p.grad = v.to(p.dtype)

    def allreduce(self, group=None, average: bool = False):
        """Sum (or average) the bucket over the ranks, then fill p.grad.  Segments whose allreduce
        was started during backward are only waited for."""
        multi = dist.is_initialized() and dist.get_world_size(group) > 1
        if self.sinks is not None:
            for idx, work in self._pending:
                if work is not None:
                    work.wait()
                elif multi:
                    dist.all_reduce(self.segments[idx][0], op=dist.ReduceOp.SUM, group=group)
            self._pending, self._filled = [], set()
        else:
            self.gather()
            if multi:
                dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
        if multi and average:
            self.flat.div_(dist.get_world_size(group))
        self.scatter()
        return self.flat
