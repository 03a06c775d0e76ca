"""Host-side logic that needs no GPU: descriptor tables, segment merging, argument validation, planner and
the ElixirOptimizer bookkeeping — with the elx_* ABI served by the oracle's host-memory shim (tests only)."""
import pytest
import torch
import torch.distributed as dist

import _dist_workers as W
from _util import free_port


@pytest.fixture(scope='module')
def host_backend():
    from elixir_b200 import _lib
    saved = (_lib._LIB, _lib._HOST_MEMORY)
    W.use_host_shim()
    if not dist.is_initialized():
        dist.init_process_group('gloo', init_method=f'tcp://127.0.0.1:{free_port()}', rank=0, world_size=1)
    yield
    _lib._LIB, _lib._HOST_MEMORY = saved


def _shard(n, dtype=torch.float16):
    return torch.randn(n) * 0.02, torch.zeros(n), torch.zeros(n), torch.zeros(n, dtype=dtype)


def test_chunk_table_merges_neighbouring_segments_and_counts_tiles(host_backend):
    from elixir_b200 import kernels as K
    table = K.ChunkTable('cpu', torch.float16)
    a = _shard(10000)
    i = table.add_chunk(*a, n_valid=9000, segments=[(0, 100, 0), (100, 300, 0), (300, 400, 1), (500, 9000, 1)])
    assert table._segs_of(i) == [(0, 300, 0), (300, 400, 1), (500, 9000, 1)]
    b = _shard(4096)
    j = table.add_chunk(*b, n_valid=0)
    c = _shard(1)
    k = table.add_chunk(*c, n_valid=1, segments=[(0, 1, 2)])
    assert (i, j, k) == (0, 1, 2)
    assert table.tile_begin == [0, 3, 4, 5]
    assert table.tiles() == 5 and table.tiles(1, 2) == 2
    table.finalize()
    with pytest.raises(RuntimeError):
        table.add_chunk(*c, n_valid=1)


@pytest.mark.parametrize('segments', [
    [(10, 5, 0)],                 # empty / reversed
    [(0, 10, 0), (5, 20, 0)],     # overlapping
    [(20, 30, 0), (0, 10, 0)],    # unsorted
    [(0, 200, 0)],                # beyond n_valid
])
def test_chunk_table_rejects_bad_segments(host_backend, segments):
    from elixir_b200 import kernels as K
    table = K.ChunkTable('cpu', torch.float16)
    with pytest.raises(ValueError):
        table.add_chunk(*_shard(256), n_valid=100, segments=segments)


def test_chunk_table_rejects_mismatched_tensors(host_backend):
    from elixir_b200 import kernels as K
    table = K.ChunkTable('cpu', torch.float16)
    p, m, v, g = _shard(256)
    with pytest.raises(ValueError):
        table.add_chunk(p, m[:100].clone(), v, g, n_valid=10)
    with pytest.raises(TypeError):
        table.add_chunk(p, m, v, g.float(), n_valid=10)
    with pytest.raises(ValueError):
        table.add_chunk(p, m, v, g, n_valid=300)
    with pytest.raises(TypeError):
        K.dtype_code(torch.int8)
    with pytest.raises(ValueError):
        table.set_hyper([K.hyper()] * 65)


def test_simple_plan_packs_in_order_and_gives_tied_parameters_private_chunks(host_backend):
    import torch.nn as nn
    from elixir_b200.wrapper import simple_plan

    class Tied(nn.Module):

        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(20, 16)
            self.fc1 = nn.Linear(16, 16)
            self.fc2 = nn.Linear(16, 16)
            self.head = nn.Linear(16, 20, bias=False)
            self.head.weight = self.embed.weight

    sr = simple_plan(Tied(), 4, split_number=10, unified_dtype=torch.float16, rcache_device='cpu')
    plans = sr.param_chunk_plans
    assert plans[0].name_list == ['embed.weight'] and plans[0].kwargs.get('rcache_fused') is True
    assert plans[0].chunk_size == 320    # 20 x 16, already a multiple of 4 (elixir's test_simple.py expects 320 too)
    public = [p for p in plans if not p.kwargs.get('rcache_fused')]
    assert [p.name_list for p in public] == [['fc1.weight'], ['fc1.bias'], ['fc2.weight'], ['fc2.bias']]
    assert {p.chunk_size for p in public} == {256} and all(p.chunk_size % 4 == 0 for p in plans)
    sr2 = simple_plan(Tied(), 3, chunk_size=300, unified_dtype=torch.float16, rcache_device='cpu')
    pub2 = [p for p in sr2.param_chunk_plans if not p.kwargs.get('rcache_fused')]
    assert [p.name_list for p in pub2] == [['fc1.weight', 'fc1.bias'], ['fc2.weight', 'fc2.bias']]
    assert pub2[0].chunk_size == 300
    with pytest.raises(ValueError):
        simple_plan(Tied(), 1, chunk_size=100, unified_dtype=torch.float16, rcache_device='cpu')


def test_optimizer_bookkeeping_frozen_parameters_and_state_views(host_backend):
    import torch.nn as nn
    from elixir_b200.optim import CPUAdam, HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 12), nn.Linear(12, 4))
    model[0].bias.requires_grad_(False)    # frozen: stays out of the chunks and out of the optimizer
    sr = simple_plan(model, 1, chunk_size=128, unified_dtype=torch.float16, shard_device='cpu', rcache_device='cpu')
    inner = HybridAdam([p for p in model.parameters() if p.requires_grad], lr=1e-2)
    emodel = ElixirModule(model, sr, dist.GroupMember.WORLD, dtype=torch.float16)
    eopt = ElixirOptimizer(emodel, inner, initial_scale=8.0)
    assert '0.bias' in emodel.no_grad_state_dict and model[0].bias.dtype == torch.float16
    n_trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    covered = sum(e - b for b, e in eopt.param_to_range.values())
    assert covered == n_trainable
    for fake, (b, e) in eopt.param_to_range.items():
        st = eopt.state[fake]
        assert st['exp_avg'].numel() == e - b == st['exp_avg_sq'].numel()
    # a step moves exactly the covered ranges; the state views alias the engine's flat moments
    grads = {n: torch.full(p.shape, 0.5) for n, p in emodel.grad_state_dict.items()}
    before = [s[0].clone() for s in eopt.engine.shards]
    emodel.inject_gradients(grads)
    eopt.step()
    assert eopt.engine.read_control().step == 1 and eopt.loss_scale == 8.0
    for (m, ea, es, lp, nv), old in zip(eopt.engine.shards, before):
        assert not torch.equal(m[:nv], old[:nv]) and torch.equal(m[nv:], old[nv:])
        assert torch.equal(lp, m.half())
    first = next(iter(eopt.param_to_range))
    assert float(eopt.state[first]['exp_avg'].abs().sum()) > 0
    with pytest.raises(TypeError):
        ElixirOptimizer(emodel, object())    # not a torch optimizer at all
    with pytest.raises(ValueError):          # any torch optimizer is accepted, but only over the module's parameters
        ElixirOptimizer(emodel, torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=0.1))
    with pytest.raises(RuntimeError):
        CPUAdam([torch.nn.Parameter(torch.zeros(1))])
    with pytest.raises(RuntimeError):
        HybridAdam([torch.nn.Parameter(torch.zeros(1))]).step()    # not wrapped: no chunk engine to step through


def test_scaler_state_dict_round_trip(host_backend):
    from elixir_b200 import kernels as K
    from elixir_b200.scaler import DynamicGradScaler
    scaler = DynamicGradScaler(initial_scale=1024.0, growth_interval=3, hysteresis=1)
    scaler.attach(K.ControlBlock('cpu', scaler.initial_scale))
    for found in (0, 0, 1, 0, 0, 0):
        scaler.ctl.found_inf.fill_(found)
        K.step_begin(scaler.ctl, scaler.cfg)
    saved = scaler.state_dict()
    assert saved == dict(scale=1024.0, growth_step=0, hysteresis_step=0, step=5, skipped_steps=1)
    other = DynamicGradScaler(initial_scale=1.0)
    other.attach(K.ControlBlock('cpu', 1.0))
    other.load_state_dict(saved)
    assert other.state_dict() == saved
    assert float(other.scale) == 1024.0
    with pytest.raises(ValueError):
        DynamicGradScaler(growth_factor=1.0)
    with pytest.raises(ValueError):
        DynamicGradScaler(backoff_factor=1.5)


def test_simple_plan_equals_the_reference_simple_search():
    """tests/golden/plans.json holds what the reference's SearchSimple.search + generate_chunk_plans produce for
    two small models over group sizes, split numbers and allocate factors (tests/golden/make_golden.py):
    same name lists, same chunk sizes, same private chunks, same number and size of public blocks."""
    import json
    import os
    import sys
    import torch
    sys.path.insert(0, W.GOLDEN)
    from make_golden import PLAN_GRID, PLAN_MODELS
    from elixir_b200.wrapper import simple_plan
    cases = json.load(open(os.path.join(W.GOLDEN, 'plans.json')))
    assert len(cases) == len(PLAN_MODELS) * len(PLAN_GRID)
    for case in cases:
        torch.manual_seed(3)
        model = PLAN_MODELS[case['model']]()
        sr = simple_plan(model, case['group_size'], split_number=case['split_number'],
                         allocate_factor=case['allocate_factor'], unified_dtype=torch.float16, rcache_device='cpu',
                         shard_device=torch.device('cpu'))
        got = [dict(names=list(p.name_list), chunk_size=p.chunk_size, fused=bool(p.kwargs.get('rcache_fused', False)))
               for p in sr.param_chunk_plans]
        key = (case['model'], case['group_size'], case['split_number'], case['allocate_factor'])
        assert got == case['plans'], key
        pool = sr.chunk_group.rcache
        assert pool.public_free_cnt == case['public_block_number'], key
        if any(not p['fused'] for p in got):
            assert pool.public_block_size == case['public_block_size'], key


def test_tensor_state_machine_equals_the_reference():
    """tests/golden/states.json: the reference's legal transitions; every other pair must raise."""
    import json
    import os
    from elixir_b200.chunk import TensorState, ts_update_sanity_check
    from elixir_b200.chunk.states import legal_ts_update_list
    legal = json.load(open(os.path.join(W.GOLDEN, 'states.json')))
    assert sorted([old.name, new.name] for old, new in legal_ts_update_list) == legal
    assert [s.name for s in TensorState] == ['FREE', 'COMPUTE', 'HOLD', 'HOLD_AFTER_BWD', 'READY_FOR_REDUCE']
    for old in TensorState:
        for new in TensorState:
            if [old.name, new.name] in legal:
                assert ts_update_sanity_check(old, new)
            else:
                with pytest.raises(RuntimeError):
                    ts_update_sanity_check(old, new)


@pytest.mark.parametrize('world', [1, 2])
def test_chunk_group_and_memory_pool_bookkeeping(world):
    import torch.multiprocessing as mp
    mp.spawn(W.group_worker, args=(world, free_port()), nprocs=world)


def test_single_pass_step_bookkeeping_equals_the_two_phase_step(host_backend):
    """Host-side logic of the single-pass step (two state sets, optimistic decision, commit or take-back, repair)
    on the host-memory shim: over applied, overflowing and already-flagged steps the control block, the masters of
    the current set and the working copies equal those of the probe-then-update step."""
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler

    def build(single_pass):
        torch.manual_seed(0)
        eng = ChunkStepEngine('cpu', torch.float16, DynamicGradScaler(initial_scale=64.0, hysteresis=1, growth_interval=2))
        for n, nv in ((9000, 9000), (5000, 3000), (4096, 0)):
            p, _, _, lowp = _shard(n)
            eng.add_shard(p, lowp, nv, [(0, nv // 2, 0), (nv // 2, nv, 1)] if nv else [])
        eng.finalize()
        eng.set_hyper([K.hyper(weight_decay=0.01), K.hyper(lr=3e-3)])
        if single_pass:
            eng.enable_single_pass()
        return eng

    a, b = build(False), build(True)
    for step in range(7):
        gen = torch.Generator().manual_seed(100 + step)
        for k in range(a.n_chunks):
            g = (torch.randn(a.shards[k][3].numel(), generator=gen) * 1e-3 * 64).half()
            if step in (2, 5) and k == 1:
                g[10] = float('inf')
            a.shards[k][3].copy_(g)
            b.shards[k][3].copy_(g)
        if step == 4:    # an overflow already known before the step (a probe with no step after it)
            a.ctl.found_inf.fill_(1)
            b.ctl.found_inf.fill_(1)
        a.probe()
        a.step()
        b.step_single_pass()
        ca, cb = a.read_control(), b.read_control()
        for field in ('scale', 'growth_step', 'hysteresis_step', 'step', 'skip', 'skipped_steps', 'found_inf', 'status'):
            assert getattr(ca, field) == getattr(cb, field), (step, field)
        assert bool(cb.skip) == (step in (2, 4, 5))
        assert cb.repair == int(step in (2, 5)) and cb.spec_state == 0
        assert b.chunk_flags.tolist() == [0, 0, 0]
        for sa, sb in zip(a.shards, b.current_shards()):
            for x, y in zip(sa[:4], sb[:4]):
                assert torch.equal(x, y), step
    assert b.read_control().cur_set == 4 % 2    # four applied steps: the sets changed roles four times
    # one more applied step leaves set 1 current; normalize_sets makes the live state "set 0" again, after which
    # the in-place step continues from it exactly as the reference engine does
    for eng in (a, b):
        for k in range(eng.n_chunks):
            eng.shards[k][3].fill_(0.01)
    a.probe()
    a.step()
    b.step_single_pass()
    assert b.read_control().cur_set == 1
    b.normalize_sets()
    assert b.read_control().cur_set == 0
    for sa, sb in zip(a.shards, b.shards):
        for x, y in zip(sa[:4], sb[:4]):
            assert torch.equal(x, y)
    for eng in (a, b):
        for k in range(eng.n_chunks):
            eng.shards[k][3].fill_(-0.02)
        eng.probe()
        eng.step()
    for sa, sb in zip(a.shards, b.shards):
        for x, y in zip(sa[:4], sb[:4]):
            assert torch.equal(x, y)


def test_near_gpu_narrows_the_affinity_and_restores_it(monkeypatch):
    """``numa.near_gpu``: inside the block the thread runs on the CPUs of the GPU's NUMA node, afterwards on those it
    had before; with the node unknown nothing changes.  The sysfs lookup is replaced by a fake."""
    import os
    from elixir_b200 import numa
    assert numa._parse_cpulist('0-3,8,10-11\n') == {0, 1, 2, 3, 8, 10, 11}
    assert numa._parse_cpulist('') == set()
    before = os.sched_getaffinity(0)
    one = {min(before)}
    monkeypatch.setattr(numa, 'gpu_numa_cpus', lambda device: one)
    with numa.near_gpu(0) as cpus:
        assert cpus == one and os.sched_getaffinity(0) == one
    assert os.sched_getaffinity(0) == before
    monkeypatch.setattr(numa, 'gpu_numa_cpus', lambda device: set())
    with numa.near_gpu(0) as cpus:
        assert cpus == set() and os.sched_getaffinity(0) == before
    assert os.sched_getaffinity(0) == before
