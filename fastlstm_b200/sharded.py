"""Batch-sharded data parallelism for the LSTM layer.

The batch dimension is the only natural shard of the path: batch rows never
interact in the forward or in the backward recurrence, only the weight-gradient
sums run over the batch.  Each rank therefore runs the full single-GPU path on
its slice of the batch and the ranks exchange one flat fp32 bucket holding every
layer's dWx, dWh and db in a single sum-allreduce (NCCL over NVLink on GPUs,
gloo in the CPU tests).  The reference (oleicht/FastLSTM) has no distributed
code; this file has no counterpart there.
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


class GradBucket:
    """One flat fp32 buffer aliasing every parameter gradient of a module.

    After `attach`, p.grad of every parameter is a view into the bucket, so
    backward accumulates straight into it and `allreduce` needs no copy."""

    def __init__(self, module: torch.nn.Module):
        self.params = [p for p in module.parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("module has no trainable parameters")
        dev = self.params[0].device
        n = sum(p.numel() for p in self.params)
        self.flat = torch.zeros(n, device=dev, dtype=torch.float32)
        self.views = []
        off = 0
        for p in self.params:
            self.views.append(self.flat[off:off + p.numel()].view_as(p))
            off += p.numel()
        self._direct = all(p.dtype == torch.float32 for p in self.params)

    def attach(self):
        """Point p.grad at the bucket (fp32 parameters only) and zero it."""
        self.flat.zero_()
        if self._direct:
            for p, v in zip(self.params, self.views):
                p.grad = v

    def gather(self):
        """Copy p.grad into the bucket when the gradients are not views of it."""
        if self._direct and all(p.grad is v for p, v in zip(self.params, self.views)):
            return
        for p, v in zip(self.params, self.views):
            v.copy_(p.grad if p.grad is not None else torch.zeros_like(v))

    def scatter(self):
        if self._direct:
            return
        for p, v in zip(self.params, self.views):
            p.grad = v.to(p.dtype)

    def allreduce(self, group=None, average: bool = False):
        """Sum (or average) the bucket over the ranks of `group` in one collective."""
        self.gather()
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
            if average:
                self.flat.div_(dist.get_world_size(group))
        self.scatter()
        return self.flat
