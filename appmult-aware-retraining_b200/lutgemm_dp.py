"""Data-parallel plumbing for the LUT-GEMM path: one process per GPU, the batch (M) dimension sharded
across ranks, and the weight gradient - the only quantity that sums over M - all-reduced.

The reference is single-GPU (it has no distributed code); this module is the one exchange step the
sharded path needs.  Forward rows and grad_a rows of a shard depend on that shard only; grad_w is
`sum_m`, so ranks hold partial sums that one all-reduce(sum) completes.  Everything here is
backend-agnostic host logic (NCCL on GPUs, gloo in the CPU tests)."""
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
