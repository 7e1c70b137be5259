"""Sharding of a recurrent op over the GPUs of one node.

Every (batch, head) pair is an independent recurrence, so a global batch is
cut along B into one contiguous shard per rank and each rank runs the
single-GPU op on its shard; nothing is exchanged on the data path.  The only
quantity that needs a sum over ranks is the gradient of an input that is
broadcast over the batch (shape 1 in dim 0, e.g. Mamba-2's per-head ``A``):
each rank holds the contribution of its shard, and ``reduce_broadcast_grads``
all-reduces those few values.  The reference has no multi-GPU code; this is
new.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_bounds(B: int, rank: int, world: int) -> Tuple[int, int]:
    """Half-open range of batch rows owned by ``rank`` (sizes differ by at most one)."""
    assert 0 <= rank < world
    base, extra = divmod(B, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_args(inputs: Sequence[torch.Tensor], states: Sequence[torch.Tensor], rank: int, world: int):
    """Views of this rank's batch rows (inputs broadcast over B are passed whole)."""
    B = max([x.shape[0] for x in inputs] + [s.shape[0] for s in states])
    lo, hi = shard_bounds(B, rank, world)
    ins = [x if x.shape[0] == 1 and B > 1 else x[lo:hi] for x in inputs]
    sts = [s[lo:hi] for s in states]
    return ins, sts, (lo, hi)


def reduce_broadcast_grads(grads: Sequence[torch.Tensor], inputs: Sequence[torch.Tensor], global_B: int,
                           group=None) -> List[torch.Tensor]:
    """Sum over ranks the gradients of inputs that are broadcast over the batch."""
    out = []
    for g, x in zip(grads, inputs):
        if g is not None and x.shape[0] == 1 and global_B > 1 and dist.is_initialized() and dist.get_world_size(group) > 1:
            g32 = g.float()
            dist.all_reduce(g32, op=dist.ReduceOp.SUM, group=group)
            g = g32.to(g.dtype)
        out.append(g)
    return out
