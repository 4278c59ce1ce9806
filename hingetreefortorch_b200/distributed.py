"""Batch-sharded data parallelism for hinge forests: one process per GPU over torch.distributed.

The evaluation path shards by rows: every (sample, position) is evaluated independently against
replicated tree parameters, so the forward needs no communication, and outputs and input
gradients are row-local.  Training needs exactly one exchange per step: the sum over ranks of
the parameter gradients (thresholds, leaf weights and, where present, the linear layer).  They
are small (tens of MB at most), so the cost is latency: all of them are packed into one flat
buffer and reduced with a single all-reduce (NCCL over NVLink on GPUs, gloo in CPU tests).
"""
import torch
import torch.distributed as dist


def shard_bounds(rows, rank, world_size):
    """Contiguous, balanced row range [lo, hi) of `rank`: the first rows % world_size ranks get one extra row."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank %d outside world of size %d" % (rank, world_size))
    base, extra = divmod(rows, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_rows(x, rank=None, world_size=None):
    """This rank's contiguous slice of a batch that every rank holds in full."""
    rank = dist.get_rank() if rank is None else rank
    world_size = dist.get_world_size() if world_size is None else world_size
    lo, hi = shard_bounds(x.shape[0], rank, world_size)
    return x[lo:hi]


class GradientBucket:
    """One flat buffer for the gradients of a fixed list of parameters, reduced with one collective."""

    def __init__(self, parameters):
        self.parameters = [p for p in parameters if p.requires_grad]
        if not self.parameters:
            raise ValueError("no trainable parameters")
        first = self.parameters[0]
        for p in self.parameters:
            if p.dtype != first.dtype or p.device != first.device:
                raise ValueError("parameters of one bucket must share dtype and device")
        self.sizes = [p.numel() for p in self.parameters]
        self.flat = torch.zeros(sum(self.sizes), dtype=first.dtype, device=first.device)
        self.views = []
        offset = 0
        for p, n in zip(self.parameters, self.sizes):
            self.views.append(self.flat[offset:offset + n].view(p.shape))
            offset += n

    @property
    def nbytes(self):
        return self.flat.numel() * self.flat.element_size()

    def all_reduce(self, group=None, average=False):
        """Sum (or average) the gradients over the ranks of `group`, in place.  A missing gradient counts as zero."""
        for p, view in zip(self.parameters, self.views):
            if p.grad is None:
                view.zero_()
            else:
                grad = p.grad.to_dense() if p.grad.is_sparse else p.grad
                view.copy_(grad)
        dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            self.flat.div_(dist.get_world_size(group))
        for p, view in zip(self.parameters, self.views):
            if p.grad is None or p.grad.is_sparse:
                p.grad = view.clone()
            else:
                p.grad.copy_(view)


def all_reduce_gradients(module, group=None, average=False):
    """Convenience wrapper: reduce the gradients of all trainable parameters of `module` once."""
    bucket = getattr(module, "_hinge_gradient_bucket", None)
    if bucket is None:
        bucket = GradientBucket(list(module.parameters()))
        module._hinge_gradient_bucket = bucket
    bucket.all_reduce(group, average)
    return bucket


def gather_rows(local, rows, group=None):
    """Concatenate the per-rank row shards of an output back into the full batch (rank order)."""
    world_size = dist.get_world_size(group)
    counts = [shard_bounds(rows, r, world_size) for r in range(world_size)]
    parts = [torch.empty((hi - lo,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
             for lo, hi in counts]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts)
