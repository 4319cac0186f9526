"""Batch-dimension sharding over the GPUs of one box (one process per GPU).

The reference picks a device per node by a heuristic and cannot move data
between GPUs (dali/array/jit/jit.cpp:367-385, memory_ops.cu.cpp:120-125).
Here the leading (batch / row) dimension is split explicitly; every rank runs
the same fused kernels on its shard and a collective is used only where the
expression reduces over the sharded dimension:

  rows independent (softmax, axis -1 reductions, LSTM cell, GEMM rows)  -> no collective
  all-axis or axis-0 sum / max / min                                     -> all_reduce of the partials
  all-axis or axis-0 argmax / argmin                                     -> all_gather of (value, global index)
                                                                            pairs, lowest index wins ties

Works with any torch.distributed backend (NCCL on the GPUs, gloo in the CPU tests).
"""
import torch
import torch.distributed as dist


def shard_range(n, rank, world):
    """[start, stop) of the rank's contiguous share of n items; the first n % world ranks get one more."""
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def combine_partials(partial, kind):
    """partial: tensor of per-rank partial results (same shape on every rank); kind: sum | max | min | prod."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        op = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "prod": dist.ReduceOp.PRODUCT}[kind]
        dist.all_reduce(partial, op=op)
    return partial


def combine_arg_partials(values, local_index, row_offset, kind):
    """values / local_index: per-rank extreme value and its index within the rank's shard (same shape on every
    rank); row_offset: what to add to make the index global.  Returns the global first-occurrence index (int64)."""
    gidx = local_index.to(torch.int64) + int(row_offset)
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return gidx
    world = dist.get_world_size()
    vals = [torch.empty_like(values) for _ in range(world)]
    idxs = [torch.empty_like(gidx) for _ in range(world)]
    dist.all_gather(vals, values.contiguous())
    dist.all_gather(idxs, gidx.contiguous())
    best_v, best_i = vals[0].clone(), idxs[0].clone()
    for v, i in zip(vals[1:], idxs[1:]):
        better = (v > best_v) if kind == "max" else (v < best_v)
        tie = (v == best_v) & (i < best_i)
        take = better | tie
        best_v = torch.where(take, v, best_v)
        best_i = torch.where(take, i, best_i)
    return best_i
