"""Generate the golden fixtures of this directory by running hpcaitech/Elixir's OWN Python code on CPU.

    python tests/golden/make_golden.py /path/to/Elixir [output directory]       (or set ELIXIR_REFERENCE)

Needs the reference checkout; the fixtures it writes (`chunk_w*.pt`, `optim_w*.pt`) are committed, so
the test-suite does not.  What runs is the reference's `elixir.chunk.Chunk` / `ChunkGroup` /
`MemoryPool` and `elixir.wrapper.ElixirModule` / `ElixirOptimizer`, unmodified, with:
  * gloo process groups of 1, 2 and 4 CPU ranks;
  * `gpu_device()` pointed at the CPU and `torch.cuda.Stream` replaced by a dummy (there is no GPU);
  * the `colossalai` stub beside this file (ColossalAI is not installable offline): its Adam delegates
    to torch.optim.Adam/AdamW, its scaler restates DynamicGradScaler.
Gradients are injected straight into the chunks (the reference's forward hooks do not run under
current PyTorch), through the same calls its autograd hook makes (`_gradient_handler`).

Fixture contents
  scheduler.json which chunk the reference's FIFOScheduler / PrefetchScheduler (elixir/chunk/scheduler/) gives
                 up at every eviction of seeded random access traces (stand-in chunk objects; no process group)
  states.json    the legal tensor-state transitions (elixir/chunk/core/states.py)
  plans.json     the chunk plans of the reference's simple search (elixir/search/simple.py: SearchSimple.search +
                 generate_chunk_plans) for two small models over group sizes, split numbers and allocate factors
  chunk_w{W}.pt  per rank: shard after close, valid_end, gathered payload, reduced shard and overflow
                 flag for a clean and for an inf-carrying gradient set (elixir/chunk/core/chunk.py)
  optim_w{W}.pt  per rank and step: overflow decision, loss scale after the step, fp32 master shards
                 (elixir/wrapper/optimizer.py:192-220)
"""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get('ELIXIR_REFERENCE', '')    # checkout of hpcaitech/Elixir; the command-line argument wins

CHUNK_SHAPES = [(2, 64), (2, 2, 128), (128,), (4, 32)]    # 896 of 1024 elements used, as test/chunk/test_chunk.py
CHUNK_SIZE = 1024


def _patch_reference_for_cpu():
    sys.path.insert(0, os.path.join(HERE, 'colossalai_stub'))
    sys.path.insert(0, REF)
    cpu = torch.device('cpu')
    import elixir.cuda
    elixir.cuda.gpu_device = lambda: cpu

    class _DummyStream:

        def wait_stream(self, other):
            pass

    torch.cuda.Stream = _DummyStream
    torch.cuda.current_stream = lambda *a, **k: _DummyStream()
    import elixir.chunk.core.chunk as ref_chunk
    ref_chunk.gpu_device = lambda: cpu
    import elixir.hook.storage as ref_storage
    ref_storage.gpu_device = lambda: cpu
    orig_init = ref_storage.BufferStore.__init__

    def cpu_init(self, buffer_size, buffer_dtype, device_str='cpu'):
        orig_init(self, buffer_size, buffer_dtype, 'cpu')

    ref_storage.BufferStore.__init__ = cpu_init
    import elixir.wrapper.module as ref_module
    import elixir.wrapper.optimizer as ref_optimizer
    ref_module.gpu_device = lambda: cpu
    ref_optimizer.gpu_device = lambda: cpu
    orig_pool_init = ref_module.MemoryPool.__init__

    def cpu_pool_init(self, device_type):
        orig_pool_init(self, 'cpu')

    ref_module.MemoryPool.__init__ = cpu_pool_init


def chunk_inputs(world):
    gen = torch.Generator().manual_seed(2261)
    tensors = [torch.randn(shape, generator=gen).half() for shape in CHUNK_SHAPES]
    grads = [[(torch.randn(shape, generator=gen) * 8).half() for shape in CHUNK_SHAPES] for _ in range(world)]
    return tensors, grads


def run_chunk(rank, world):
    from elixir.chunk import Chunk, MemoryPool, TensorState
    cpu = torch.device('cpu')
    tensors, grads = chunk_inputs(world)
    out = {}
    for case in ('clean', 'inf'):
        pool = MemoryPool('cpu')
        pool.allocate(public_dtype=torch.float16, public_block_size=CHUNK_SIZE, public_block_number=1)
        chunk = Chunk(pool, CHUNK_SIZE, torch.float16, dist.GroupMember.WORLD, temp_device=cpu, shard_device=cpu)
        held = [t.clone() for t in tensors]
        for t in held:
            chunk.append_tensor(t)
        chunk.close_chunk()
        rec = dict(shard_after_close=chunk.shard.clone(), valid_end=chunk.valid_end, shard_begin=chunk.shard_begin,
                   shard_size=chunk.shard_size)
        block = pool.get_public_block()
        chunk.access_chunk(block)
        rec['payload_after_access'] = block.payload.clone()
        for t, g in zip(held, grads[rank]):
            g = g.clone()
            if case == 'inf' and rank == world - 1 and t is held[0]:
                g.view(-1)[3] = float('inf')
            for state in (TensorState.COMPUTE, TensorState.HOLD_AFTER_BWD, TensorState.READY_FOR_REDUCE):
                chunk.tensor_trans_state(t, state)
            chunk.copy_tensor_to_chunk_slice(t, g)
        assert chunk.reduce_check
        chunk.reduce_chunk()
        rec['shard_after_reduce'] = chunk.shard.clone()
        rec['overflow'] = bool(chunk.overflow)
        out[case] = rec
    return out


class TinyNet(nn.Module):
    """Two linear layers and a LayerNorm: enough tensors to straddle shard boundaries."""

    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(24, 40)
        self.norm = nn.LayerNorm(40)
        self.fc2 = nn.Linear(40, 10)


def optim_inputs(world, steps):
    torch.manual_seed(7)
    model = TinyNet()
    gen = torch.Generator().manual_seed(99)
    grads = []
    for s in range(steps):
        per_rank = []
        for r in range(world):
            per_rank.append({n: torch.randn(p.shape, generator=gen) * 1e-3 for n, p in model.named_parameters()})
        grads.append(per_rank)
    return model, grads


OPTIM_STEPS = 6
OPTIM_CFG = dict(initial_scale=64.0, min_scale=1, growth_factor=2, backoff_factor=0.5, growth_interval=2, hysteresis=1,
                 max_scale=2**24)
OPTIM_HYPER = dict(lr=0.0009765625, betas=(0.875, 0.99609375), eps=1e-8, weight_decay=0.0078125)
OPTIM_CHUNK = 1024    # two public chunks for the 1490 parameters (the second one 48% used); divisible by 1, 2, 4
INF_STEP = 2


def run_optim(rank, world):
    from colossalai.nn.optimizer import HybridAdam
    from elixir.chunk import ChunkGroup, MemoryPool, TensorState
    from elixir.search.result import ChunkPlan, SearchResult
    from elixir.wrapper import ElixirModule, ElixirOptimizer
    from elixir.wrapper.optimizer import OptimState
    cpu = torch.device('cpu')
    model, grads = optim_inputs(world, OPTIM_STEPS)
    names = [n for n, _ in model.named_parameters()]
    plans, cur, room = [], [], 0
    sizes = {n: p.numel() for n, p in model.named_parameters()}
    for n in names:
        if sizes[n] > room:
            cur = []
            plans.append(ChunkPlan(name_list=cur, chunk_size=OPTIM_CHUNK, chunk_dtype=torch.float16,
                                   kwargs=dict(shard_device=cpu, temp_device=cpu)))
            room = OPTIM_CHUNK
        cur.append(n)
        room -= sizes[n]
    pool = MemoryPool('cpu')
    pool.allocate(public_dtype=torch.float16, public_block_size=OPTIM_CHUNK, public_block_number=len(plans))
    sr = SearchResult(ChunkGroup(pool), plans)
    inner = HybridAdam(model.parameters(), adamw_mode=True, **OPTIM_HYPER)
    emodel = ElixirModule(model, sr, dist.GroupMember.WORLD, dtype=torch.float16)
    eoptim = ElixirOptimizer(emodel, inner, **OPTIM_CFG)
    group = emodel.param_chunk_group
    chunks = sorted(group.float_chunks | group.fused_chunks, key=lambda c: c.chunk_id)
    out = dict(plans=[list(p.name_list) for p in plans], steps=[],
               init_master=[c.paired_chunk.shard.clone() for c in chunks],
               valid_end=[c.valid_end for c in chunks])
    params = dict(emodel.module.named_parameters())
    for s in range(OPTIM_STEPS):
        scale = eoptim.loss_scale
        for c in chunks:
            group.access_chunk(c)
        for n in names:
            p = params[n]
            g = (grads[s][rank][n] * scale).half()
            if s == INF_STEP and rank == world - 1 and n == 'fc2.weight':
                g.view(-1)[5] = float('inf')
            group.tensor_trans_state(p, TensorState.COMPUTE)
            group.tensor_trans_state(p, TensorState.HOLD_AFTER_BWD)
            emodel._gradient_handler(g, p)
        flags = [bool(c.overflow) for c in chunks]
        grad_shards = [c.shard.clone() for c in chunks]
        eoptim.optim_state = OptimState.SCALED
        eoptim.step()
        out['steps'].append(dict(scale_before=scale, scale_after=eoptim.loss_scale, chunk_overflow=flags,
                                 grad_shards=grad_shards,
                                 master=[c.paired_chunk.shard.clone() for c in chunks]))
    return out


class StandIn:
    """All a scheduler needs of a chunk: identity and an order."""

    def __init__(self, chunk_id):
        self.chunk_id = chunk_id

    def __hash__(self):
        return self.chunk_id

    def __eq__(self, other):
        return self.chunk_id == other.chunk_id

    def __lt__(self, other):
        return self.chunk_id < other.chunk_id


def scheduler_cases(n_cases=40, seed=4242):
    """Seeded (trace, blocks) pairs: up to 7 chunks, up to 60 fetches, 1 to 4 blocks."""
    import random
    rng = random.Random(seed)
    cases = []
    for _ in range(n_cases):
        n_chunks = rng.randint(2, 7)
        trace = [rng.randrange(n_chunks) for _ in range(rng.randint(5, 60))]
        cases.append((trace, rng.randint(1, 4)))
    return cases


def drive_scheduler(scheduler, trace, blocks, step_with_chunks=False):
    """One chunk per fetch, released right after use; returns the ids of the chunks given up, in order."""
    chunks = {i: StandIn(i) for i in set(trace)}
    resident, victims = set(), []
    scheduler.reset()
    for i in trace:
        chunk = chunks[i]
        scheduler.remove(chunk)
        if step_with_chunks:
            scheduler.step([chunk])
        else:
            scheduler.step()
        if chunk not in resident:
            if len(resident) == blocks:
                victim = scheduler.top()
                scheduler.remove(victim)
                resident.remove(victim)
                victims.append(victim.chunk_id)
            resident.add(chunk)
        scheduler.add(chunk)
    for chunk in list(resident):
        scheduler.remove(chunk)
    scheduler.clear()
    return victims


def run_scheduler():
    sys.path.insert(0, REF)
    from elixir.chunk.scheduler import FIFOScheduler, PrefetchScheduler
    out = []
    for trace, blocks in scheduler_cases():
        stand_ins = {i: StandIn(i) for i in set(trace)}
        belady = drive_scheduler(PrefetchScheduler([[stand_ins[i]] for i in trace]), trace, blocks)
        fifo = drive_scheduler(FIFOScheduler(), trace, blocks)
        out.append(dict(trace=trace, blocks=blocks, prefetch_victims=belady, fifo_victims=fifo))
    return out


class TiedNet(nn.Module):
    """An embedding shared with the output projection (a parameter used by two modules) around a few layers."""

    def __init__(self):
        super().__init__()
        self.embed = nn.Embedding(50, 32)
        self.body = nn.Sequential(nn.LayerNorm(32), nn.Linear(32, 64), nn.Tanh(), nn.Linear(64, 32), nn.LayerNorm(32))
        self.head = nn.Linear(32, 50, bias=False)
        self.head.weight = self.embed.weight


PLAN_MODELS = dict(tiny=TinyNet, tied=TiedNet)
PLAN_GRID = [(g, s, a) for g in (1, 2, 4) for s in (1, 3, 10, 50) for a in (0.6, 1.0)]


def run_plans():
    sys.path.insert(0, os.path.join(HERE, 'colossalai_stub'))
    sys.path.insert(0, REF)
    from elixir.search.simple import SearchSimple
    out = []
    for name, cls in PLAN_MODELS.items():
        torch.manual_seed(3)
        model = cls()
        for group_size, split_number, allocate_factor in PLAN_GRID:
            search = SearchSimple(model, group_size, dtype=torch.float16)
            private, public = search.search(split_number, allocate_factor)
            plans = search.generate_chunk_plans(private, public)
            out.append(dict(model=name, group_size=group_size, split_number=split_number,
                            allocate_factor=allocate_factor, public_block_size=search.public_block_size,
                            public_block_number=search.public_block_number,
                            plans=[dict(names=list(p.name_list), chunk_size=p.chunk_size,
                                        fused=bool(p.kwargs.get('rcache_fused', False))) for p in plans]))
    return out


def worker(rank, world, port, result_dir):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR='127.0.0.1',
                      MASTER_PORT=str(port))
    _patch_reference_for_cpu()
    dist.init_process_group('gloo', rank=rank, world_size=world)
    torch.save(run_chunk(rank, world), os.path.join(result_dir, f'chunk_{rank}.pt'))
    torch.save(run_optim(rank, world), os.path.join(result_dir, f'optim_{rank}.pt'))
    dist.barrier()
    dist.destroy_process_group()


def main():
    import tempfile
    global REF
    if len(sys.argv) > 1:
        REF = sys.argv[1]
    out_dir = sys.argv[2] if len(sys.argv) > 2 else HERE
    if not os.path.isdir(os.path.join(REF, 'elixir')):
        raise SystemExit('give the path of a checkout of hpcaitech/Elixir (argument or ELIXIR_REFERENCE)')
    os.environ['ELIXIR_REFERENCE'] = REF    # spawned workers re-import this module
    import json
    with open(os.path.join(out_dir, 'scheduler.json'), 'w') as f:
        json.dump(run_scheduler(), f)
    with open(os.path.join(out_dir, 'plans.json'), 'w') as f:
        json.dump(run_plans(), f)
    from elixir.chunk.core.states import legal_ts_update_list
    with open(os.path.join(out_dir, 'states.json'), 'w') as f:
        json.dump(sorted([old.name, new.name] for old, new in legal_ts_update_list), f)
    print('scheduler traces and chunk plans written')
    for i, world in enumerate((1, 2, 4)):
        with tempfile.TemporaryDirectory() as tmp:
            mp.spawn(worker, args=(world, 29600 + i, tmp), nprocs=world)
            for kind in ('chunk', 'optim'):
                per_rank = [torch.load(os.path.join(tmp, f'{kind}_{r}.pt')) for r in range(world)]
                torch.save(dict(world=world, ranks=per_rank), os.path.join(out_dir, f'{kind}_w{world}.pt'))
        print(f'world {world}: fixtures written')


if __name__ == '__main__':
    main()
