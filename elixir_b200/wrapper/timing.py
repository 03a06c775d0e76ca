"""Time one training iteration (forward, backward, optimizer step) of a stack of MLP blocks behind
``ElixirModule`` / ``ElixirOptimizer`` under the three ways of keeping chunks resident:

* ``all``       a replica-cache block per chunk, everything gathered before forward;
* ``fifo``      ``--blocks`` blocks, chunks fetched sub-module by sub-module on the main stream;
* ``prefetch``  the same blocks, Belady's rule on the learnt access trace, gathers ahead and reduces on
                side streams.

    python -m elixir_b200.wrapper.timing --layers 12 --hidden 4096 --tokens 8192 --blocks 3
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m elixir_b200.wrapper.timing ...

One chunk holds one block of the stack (two weight matrices and their biases).  Prints one JSON line per
mode: milliseconds per iteration (CUDA events, max over ranks), peak device memory, fetch counters.
Synthetic data, random weights.
"""
import argparse
import gc
import json
import os

import torch
import torch.distributed as dist
import torch.nn as nn

from ..optim import HybridAdam
from .module import ElixirModule
from .optimizer import ElixirOptimizer
from .plan import simple_plan


class Block(nn.Module):

    def __init__(self, hidden: int):
        super().__init__()
        self.up = nn.Linear(hidden, 4 * hidden)
        self.down = nn.Linear(4 * hidden, hidden)

    def forward(self, x):
        return x + self.down(torch.nn.functional.gelu(self.up(x)))


class Stack(nn.Module):

    def __init__(self, layers: int, hidden: int):
        super().__init__()
        self.blocks = nn.ModuleList(Block(hidden) for _ in range(layers))

    def forward(self, x):
        for block in self.blocks:
            x = block(x)
        return x.float().pow(2).mean()


def run_mode(mode: str, args, group, device) -> dict:
    torch.manual_seed(0)
    with torch.device(device):
        model = Stack(args.layers, args.hidden).to(torch.float16)
    world = dist.get_world_size(group)
    per_block = sum(p.numel() for p in model.blocks[0].parameters())
    blocks = None if mode == 'all' else args.blocks
    sr = simple_plan(model, world, unified_dtype=torch.float16, shard_device=device, chunk_size=per_block,
                     public_block_number=blocks)
    emodel = ElixirModule(model, sr, group, prefetch=(mode != 'fifo'), dtype=torch.float16)
    eoptim = ElixirOptimizer(emodel, HybridAdam(model.parameters(), lr=1e-4), initial_scale=1024.0)
    x = torch.randn(args.tokens, args.hidden, device=device, dtype=torch.float16)
    torch.cuda.reset_peak_memory_stats(device)
    rcache_gb = sr.chunk_group.rcache.public_space / 1e9

    def iteration():
        eoptim.zero_grad()
        eoptim.backward(emodel(x))
        eoptim.step()

    for _ in range(args.warmup):
        iteration()
    torch.cuda.synchronize(device)
    dist.barrier(group)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        iteration()
    stop.record()
    torch.cuda.synchronize(device)
    ms = torch.tensor([start.elapsed_time(stop) / args.steps], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=group)
    status = eoptim.engine.read_control().status
    out = dict(mode=mode, ms_per_iteration=round(float(ms), 3), world=world, layers=args.layers, hidden=args.hidden,
               tokens=args.tokens, chunk_elems=per_block, chunks=len(emodel.param_chunks),
               blocks=len(emodel.param_chunks) if blocks is None else blocks,
               replica_cache_gb=round(rcache_gb, 2),
               peak_mem_gb=round(torch.cuda.max_memory_allocated(device) / 1e9, 2),
               fetch=dict(emodel.fetcher.stats) if emodel.scheduled else None, status=status)
    del emodel, eoptim, model, sr, iteration, x
    gc.collect()    # module <-> hook cycles keep the chunks alive otherwise
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--layers', type=int, default=12)
    ap.add_argument('--hidden', type=int, default=4096)
    ap.add_argument('--tokens', type=int, default=8192)
    ap.add_argument('--blocks', type=int, default=3)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--modes', default='all,fifo,prefetch')
    args = ap.parse_args()
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local = int(os.environ.get('LOCAL_RANK', 0))
    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29577')
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
    for mode in args.modes.split(','):
        result = run_mode(mode, args, dist.group.WORLD, device)
        if rank == 0:
            print(json.dumps(result), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
