"""Chunk plans: which parameters go into which chunk.

``ChunkPlan`` / ``SearchResult`` have the fields of ``elixir/search/result.py:8-32``; ``simple_plan``
produces what ``simple_search`` (``elixir/search/simple.py:77-110``) produces — parameters used by more
than one module get a private chunk each, the others are split in order into ``split_number`` public
chunks of one common size, every size rounded up to a multiple of the group size
(``search/utils.py:5-6``).  The replica cache gets ``ceil(public chunks * allocate_factor)`` blocks as in
the reference (``simple.py:72``), but ``allocate_factor`` defaults to 1 here (0.6 there): with a block per
public chunk ``ElixirModule`` keeps everything gathered from forward to the end of backward, with fewer it
schedules residency sub-module by sub-module.  ``public_block_number`` sets the count directly.  The
memory- and bandwidth-model searches of the reference are planning-time tools outside the optimizer step
and are not rebuilt.
"""
import math
from typing import Dict, List, NamedTuple, Optional

import torch
import torch.nn as nn

from ..chunk import BlockRequire, ChunkGroup, MemoryPool


class ChunkPlan(NamedTuple):
    name_list: List[str]
    chunk_size: int
    chunk_dtype: torch.dtype
    kwargs: Dict


class SearchResult:

    def __init__(self, chunk_group: ChunkGroup, chunk_plans: List[ChunkPlan],
                 param_called_per_step: Optional[List[List[str]]] = None) -> None:
        self.chunk_group = chunk_group
        self.param_chunk_plans = chunk_plans
        self.param_called_per_step = param_called_per_step


def to_divide(a: int, b: int) -> int:
    return a + (-a % b)


def get_multi_used_params(m: nn.Module) -> set:
    seen, multi = set(), set()
    for module in m.modules():
        for param in module.parameters(recurse=False):
            (multi if param in seen else seen).add(param)
    return multi


def simple_plan(m: nn.Module,
                group_size: int,
                split_number: int = 10,
                allocate_factor: float = 1.0,
                unified_dtype: torch.dtype = torch.float,
                shard_device: Optional[torch.device] = None,
                prefetch: bool = False,
                verbose: bool = False,
                chunk_size: Optional[int] = None,
                rcache_device=None,
                peer_group=None,
                public_block_number: Optional[int] = None) -> SearchResult:
    """Plan chunks for the parameters of ``m`` that require gradients.  ``chunk_size`` (elements) overrides
    the size derived from ``split_number``; parameters are then packed greedily in order.  ``peer_group`` (a
    single-node process group) places the replica cache in memory every rank of the group can address, which
    lets ``ElixirOptimizer`` run reduce-scatter and all-gather inside its kernels over NVLink."""
    names = {p: n for n, p in m.named_parameters()}
    params = [p for p in m.parameters() if p.requires_grad]
    private = get_multi_used_params(m)
    public = [p for p in params if p not in private]

    plans: List[ChunkPlan] = []
    for p in params:
        if p in private:
            plans.append(ChunkPlan([names[p]], to_divide(p.numel(), group_size), unified_dtype,
                                   dict(rcache_fused=True)))

    groups: List[List[nn.Parameter]] = []
    if chunk_size is not None:
        chunk_size = to_divide(chunk_size, group_size)
        room = 0
        for p in public:
            if p.numel() > chunk_size:
                raise ValueError(f'parameter {names[p]} ({p.numel()} elements) does not fit a chunk of {chunk_size}')
            if p.numel() > room:
                groups.append([])
                room = chunk_size
            groups[-1].append(p)
            room -= p.numel()
        public_size = chunk_size
    else:
        n_split = min(len(public), split_number)
        if n_split > 0:
            base, extra = divmod(len(public), n_split)
            it = iter(public)
            for i in range(n_split):
                groups.append([next(it) for _ in range(base + (1 if i < extra else 0))])
        public_size = to_divide(max((sum(p.numel() for p in g) for g in groups), default=0), group_size)
    for g in groups:
        plans.append(ChunkPlan([names[p] for p in g], public_size, unified_dtype, dict()))

    for plan in plans:
        if shard_device is not None:
            plan.kwargs['shard_device'] = shard_device
        if rcache_device is not None and not plan.kwargs.get('rcache_fused'):
            plan.kwargs['temp_device'] = rcache_device

    device_type = rcache_device if rcache_device is not None else 'cuda'
    slab_factory = None
    if peer_group is not None:
        # replica cache in peer-mapped memory: the optimizer step then runs its collectives inside the kernels
        from ..peer import PeerBuffer
        device = torch.device('cuda', torch.cuda.current_device())
        slab_factory = lambda numel, dtype: PeerBuffer(numel, dtype, device, peer_group)    # noqa: E731
    pool = MemoryPool(device_type, slab_factory=slab_factory)
    if public_block_number is None:
        public_block_number = math.ceil(len(groups) * allocate_factor)
    if groups:
        public_block_number = max(public_block_number, 1)
    if peer_group is not None and public_block_number < len(groups):
        raise ValueError('a replica cache in peer-mapped memory needs a block for every public chunk')
    pool.allocate(public_dtype=unified_dtype,
                  public_block_size=max(public_size, 1),
                  public_block_number=public_block_number,
                  private_block_list=[BlockRequire(pl.chunk_size, pl.chunk_dtype) for pl in plans
                                      if pl.kwargs.get('rcache_fused')])
    if verbose:
        for i, plan in enumerate(plans):
            print(f'plan {i}: {len(plan.name_list)} tensors, size {plan.chunk_size}, {plan.kwargs}')
    return SearchResult(ChunkGroup(pool), plans, None)


simple_search = simple_plan
