"""Multi-GPU use of the operators: the batch*head dimension P is cut into contiguous
slices, one per rank; each rank calls the operator on its slice only. The sums of
different p never interact, so there is no collective on the data path; an all_gather of
the per-rank results is available for callers that want every rank to hold everything.
(The reference is single-GPU; its kernels index p by blockIdx only, e.g.
Weighted_Laplace_Sum/csrc/laplace_kernels.cu:78.)
"""

import torch
import torch.distributed as dist


def shard_range(P, rank, world):
    """[lo, hi) of the p-slice owned by `rank`: sizes differ by at most one, order preserved."""
    base, extra = divmod(P, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def sharded_call(fn, tensors, group=None, gather=False):
    """Run fn on this rank's p-slice of every tensor (dim 0 = P on all of them).

    Returns fn's outputs for the slice (None on a rank whose slice is empty), or, with
    gather=True, the outputs of all ranks concatenated along dim 0: one all_gather per
    output, with the slices padded to the longest one because the collective wants equal
    sizes. fn must return a tensor or a tuple of tensors whose dim 0 is the slice's P.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    P = tensors[0].shape[0]
    lo, hi = shard_range(P, rank, world)
    outs = fn(*[t[lo:hi].contiguous() for t in tensors]) if hi > lo else None
    if not gather or world == 1:
        return outs
    single = outs is not None and not isinstance(outs, (tuple, list))
    mine = None if outs is None else ([outs] if single else list(outs))
    # ranks with an empty slice learn the number, trailing shapes and dtypes of the outputs from the others
    meta = [None] * world
    dist.all_gather_object(meta, None if mine is None else (single, [(tuple(t.shape[1:]), t.dtype) for t in mine]), group=group)
    single, specs = next(m for m in meta if m is not None)
    longest = max(shard_range(P, r, world)[1] - shard_range(P, r, world)[0] for r in range(world))
    gathered = []
    for i, (shape, dtype) in enumerate(specs):
        padded = tensors[0].new_zeros((longest, *shape), dtype=dtype)
        if mine is not None:
            padded[:hi - lo] = mine[i]
        parts = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(parts, padded, group=group)
        gathered.append(torch.cat([parts[r][:shard_range(P, r, world)[1] - shard_range(P, r, world)[0]] for r in range(world)], 0))
    return gathered[0] if single else tuple(gathered)
