"""The two collectives of the chunk runtime, over ``torch.distributed`` (NCCL on NVLink / NVSwitch).

* gradient averaging: ``out = sum_r(inp_r / W)[my shard]`` — the reference divides the whole replicated
  block by W in the chunk dtype and then SUM-reduce-scatters it (``elixir/chunk/core/chunk.py:298-303``).
  On NCCL the division rides inside the collective as a pre-multiplied sum (each operand is scaled by
  1/W before it is added), which is the same arithmetic without the extra pass over the block.
* parameter gather: ``all_gather_into_tensor`` of the updated low-precision shards
  (``chunk.py:475-482``).
"""
import torch
import torch.distributed as dist


def _is_nccl(t: torch.Tensor) -> bool:
    return t.is_cuda


def reduce_scatter_avg(out: torch.Tensor, inp: torch.Tensor, group, async_op: bool = False):
    """``out`` (shard_size) receives this rank's slice of the rank-average of ``inp`` (chunk_size).
    ``out`` may alias the matching slice of ``inp``.  ``inp`` is clobbered on non-NCCL backends."""
    world = dist.get_world_size(group)
    if world == 1:
        if out.data_ptr() != inp.data_ptr():
            out.copy_(inp)
        return None
    if _is_nccl(inp):
        op = dist._make_nccl_premul_sum(1.0 / world)
        return dist.reduce_scatter_tensor(out, inp, op=op, group=group, async_op=async_op)
    inp.div_(world)
    return dist.reduce_scatter_tensor(out, inp, group=group, async_op=async_op)


def all_gather(out: torch.Tensor, inp: torch.Tensor, group, async_op: bool = False):
    """``out`` (chunk_size) receives every rank's ``inp`` (shard_size) in rank order."""
    if dist.get_world_size(group) == 1:
        if out.data_ptr() != inp.data_ptr():
            out.copy_(inp)
        return None
    return dist.all_gather_into_tensor(out, inp, group=group, async_op=async_op)


def agree_on_overflow(found_inf: torch.Tensor, group):
    """MAX all-reduce of the 4-byte overflow word, so that every rank takes the same skip decision.
    The reference decides per rank (``elixir/wrapper/optimizer.py:137-142``) and can diverge when only
    some ranks' shards overflowed."""
    if dist.get_world_size(group) > 1:
        dist.all_reduce(found_inf, op=dist.ReduceOp.MAX, group=group)
