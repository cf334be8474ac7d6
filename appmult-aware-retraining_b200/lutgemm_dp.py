"""Data-parallel plumbing for the LUT-GEMM path: one process per GPU, the batch (M) dimension sharded
across ranks, and the weight gradient - the only quantity that sums over M - all-reduced.

The reference is single-GPU (it has no distributed code); this module is the one exchange step the
sharded path needs.  Forward rows and grad_a rows of a shard depend on that shard only; grad_w is
`sum_m`, so ranks hold partial sums that one all-reduce(sum) completes.  In training the same
exchange is the all-reduce of the parameter gradients: `OverlappedGradReducer` launches it bucket by bucket
from gradient hooks while backward is still running.  Everything here is backend-agnostic host logic (NCCL
on GPUs, gloo in the CPU tests)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(num_rows: int, rank: int, world_size: int) -> tuple[int, int]:
    """[begin, end) of the rows rank `rank` owns: contiguous, sizes differ by at most one, the first
    `num_rows % world_size` ranks take the extra row.  Empty ranges are legal (more ranks than rows)."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} / world size {world_size}")
    base, extra = divmod(num_rows, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def allreduce_weight_grad(gw: torch.Tensor, group=None, async_op: bool = False):
    """Sum the per-shard weight gradient over all ranks in place.  With async_op=True the returned work
    handle lets the caller overlap the collective with the grad_a kernel and wait afterwards."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None
    return dist.all_reduce(gw, op=dist.ReduceOp.SUM, group=group, async_op=async_op)


def allreduce_grads_bucketed(params, group=None, bucket_bytes: int = 64 << 20) -> int:
    """Average `.grad` of the given parameters over ranks with few large all-reduces: gradients are
    packed into flat fp32 buckets of about `bucket_bytes` (NVSwitch makes collective cost latency-,
    not link-bound, so buckets are sized for launch count).  Returns the number of collectives."""
    if not dist.is_available() or not dist.is_initialized():
        return 0
    world = dist.get_world_size(group)
    if world == 1:
        return 0
    grads = [p.grad for p in params if p.grad is not None]
    n_coll, i = 0, 0
    while i < len(grads):
        bucket, size = [], 0
        while i < len(grads) and (not bucket or size + grads[i].numel() * 4 <= bucket_bytes):
            bucket.append(grads[i]); size += grads[i].numel() * 4; i += 1
        flat = torch.cat([g.reshape(-1).to(torch.float32) for g in bucket])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        flat.div_(world)
        off = 0
        for g in bucket:
            g.copy_(flat[off:off + g.numel()].view_as(g)); off += g.numel()
        n_coll += 1
    return n_coll


class OverlappedGradReducer:
    """Averages parameter gradients over ranks WHILE the backward pass is still running.

    All gradients live in one persistent flat fp32 buffer, cut into buckets of about `bucket_bytes` in the
    order in which backward produces them (last layer first); every parameter's `.grad` is a view into that
    buffer, so nothing is packed or copied back.  A post-accumulate-grad hook on each parameter counts the
    bucket's gradients as they arrive and launches the bucket's all-reduce, asynchronously, as soon as the
    last one is there: the collective of the later layers runs under the backward kernels of the earlier
    ones.  `finish()` - called between `loss.backward()` and `optimizer.step()` - waits for the collectives
    and turns the sums into means.

    Use `reducer.zero_grad()` (one fill of the flat buffer) instead of `optimizer.zero_grad(set_to_none=True)`:
    setting `.grad` to None would detach the parameters from the buffer.  With one rank, or without an
    initialised process group, the hooks only count and `finish()` returns at once.
    The reference trains on one GPU and has no counterpart."""

    def __init__(self, params, group=None, bucket_bytes: int = 32 << 20):
        self.group = group
        self.params = [p for p in params if p.requires_grad]
        self.active = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if self.active else 1
        if not self.params:
            self.flat, self.buckets = None, []
            return
        dev = self.params[0].device
        order = list(reversed(self.params))  # backward reaches the last layers first
        total = sum(p.numel() for p in order)
        self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
        self.buckets = []  # (begin, end, number of parameters)
        self._bucket_of, self._offsets = {}, {}
        begin = off = count = 0
        for p in order:
            if count and (off - begin + p.numel()) * 4 > bucket_bytes:
                self.buckets.append((begin, off, count))
                begin, count = off, 0
            self._offsets[p] = off
            p.grad = self._view_of(p)
            self._bucket_of[p] = len(self.buckets)
            off += p.numel()
            count += 1
        self.buckets.append((begin, off, count))
        self._arrived = [0] * len(self.buckets)
        self._works = []
        self.collectives = 0
        self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in order]

    def _on_grad(self, p):
        b = self._bucket_of[p]
        if p.grad.data_ptr() != self.flat.data_ptr() + 4 * self._offsets[p]:
            # someone replaced .grad (e.g. zero_grad(set_to_none=True)): fold it back into the buffer
            view = self._view_of(p)
            view.copy_(p.grad)
            p.grad = view
        self._arrived[b] += 1
        if self._arrived[b] == self.buckets[b][2]:
            self._launch(b)

    def _view_of(self, p):
        # a view with the parameter's own (dense) strides, e.g. channels-last convolution weights, so that autograd
        # accumulates into it without a layout mismatch
        off = self._offsets[p]
        if p.dim() == 4 and not p.is_contiguous() and p.is_contiguous(memory_format=torch.channels_last):
            return self.flat.as_strided(p.shape, p.stride(), off)
        return self.flat[off:off + p.numel()].view(p.shape)

    def _launch(self, b):
        if not self.active:
            return
        begin, end, _ = self.buckets[b]
        self._works.append(dist.all_reduce(self.flat[begin:end], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        self.collectives += 1

    def zero_grad(self):
        if self.flat is not None:
            self.flat.zero_()

    def finish(self) -> int:
        """Waits for the step's collectives, averages, and re-arms the hooks' counters.  Buckets whose
        gradients did not all arrive (parameters unused in this step) are reduced here.  Returns the number
        of collectives of the step."""
        for b, (_, _, count) in enumerate(self.buckets):
            if 0 < self._arrived[b] < count or (self._arrived[b] == 0 and self.active):
                self._launch(b)
        for w in self._works:
            w.wait()
        if self.active and self.flat is not None:
            self.flat.div_(self.world)
        n, self.collectives = self.collectives, 0
        self._works = []
        self._arrived = [0] * len(self.buckets)
        return n

    def close(self):
        for h in getattr(self, "_hooks", []):
            h.remove()
        self._hooks = []
