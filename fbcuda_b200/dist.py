"""Batch data-parallel plumbing for the convolution passes (one process per GPU).

Inputs, outputs and output gradients are sharded along the batch; weights are
replicated; updateOutput and updateGradInput need no communication;
accGradParameters needs one all-reduce (sum) of the weight gradient, taken either
in the frequency domain (between the contraction and its inverse transform) or in
the spatial domain (after it) -- equal up to rounding because the inverse transform
is linear.  The reference has no multi-GPU code; this follows what its
accGradParameters computes (fbfft/FFTIteratedConvolution.cuh:409-524) summed over
batch shards.  Only torch.distributed is used; nothing here computes.
"""
from __future__ import annotations


def shard_bounds(batch: int, world: int, rank: int):
    """Contiguous shard [lo, hi) of `batch` images for `rank`; the first
    batch % world ranks get one image more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def all_reduce_sum(tensor, group=None):
    """In-place sum over the ranks; a no-op without an initialised process group."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=group)
    return tensor
