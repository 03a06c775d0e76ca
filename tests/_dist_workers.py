"""Worker functions of the multi-process (gloo) tests.  They run in spawned children, so everything they
need is imported inside them.  The children route the elx_* ABI to the oracle's host-memory shim."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, 'tests', 'golden')


def use_host_shim():
    """Replace the CUDA library by the oracle's host-memory implementation of the same ABI (tests only)."""
    import ctypes
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    from elixir_b200 import _abi, _lib
    from oracle import oracle
    cdll = ctypes.CDLL(oracle.build_host_shim())
    _abi.apply_prototypes(cdll)
    _lib._LIB = cdll
    _lib._HOST_MEMORY = True


def init_gloo(rank, world, port):
    import torch.distributed as dist
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR='127.0.0.1',
                      MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    return dist


def bits_equal(a, b):
    view = {2: torch.int16, 4: torch.int32}[a.element_size()]
    return a.shape == b.shape and torch.equal(a.contiguous().view(view), b.contiguous().view(view))


def chunk_worker(rank, world, port):
    """Replay tests/golden/make_golden.py::run_chunk with this package's Chunk and compare bit for bit."""
    use_host_shim()
    dist = init_gloo(rank, world, port)
    sys.path.insert(0, GOLDEN)
    from make_golden import CHUNK_SIZE, chunk_inputs
    from elixir_b200.chunk import Chunk, MemoryPool, TensorState
    golden = torch.load(os.path.join(GOLDEN, f'chunk_w{world}.pt'))['ranks'][rank]
    cpu = torch.device('cpu')
    tensors, grads = chunk_inputs(world)
    for case in ('clean', 'inf'):
        want = golden[case]
        pool = MemoryPool('cpu')
        pool.allocate(public_dtype=torch.float16, public_block_size=CHUNK_SIZE, public_block_number=1)
        chunk = Chunk(pool, CHUNK_SIZE, torch.float16, dist.GroupMember.WORLD, temp_device=cpu, shard_device=cpu)
        held = [t.clone() for t in tensors]
        originals = [t.clone() for t in tensors]
        for t in held:
            chunk.append_tensor(t)
        chunk.close_chunk()
        assert (chunk.shard_begin, chunk.shard_size) == (want['shard_begin'], want['shard_size'])
        assert chunk.valid_end == min(want['valid_end'], want['shard_size'])
        assert bits_equal(chunk.shard, want['shard_after_close'])
        block = pool.get_public_block()
        chunk.access_chunk(block)
        assert bits_equal(block.payload, want['payload_after_access'])
        for t, o in zip(held, originals):
            assert bits_equal(t.data, o)    # tensors point into the gathered block again
        for t, g in zip(held, grads[rank]):
            g = g.clone()
            if case == 'inf' and rank == world - 1 and t is held[0]:
                g.view(-1)[3] = float('inf')
            for state in (TensorState.COMPUTE, TensorState.HOLD_AFTER_BWD, TensorState.READY_FOR_REDUCE):
                chunk.tensor_trans_state(t, state)
            chunk.copy_tensor_to_chunk_slice(t, g)
        assert chunk.reduce_check
        chunk.reduce_chunk()
        assert not chunk.is_replica and chunk.tensor_state_cnter[TensorState.HOLD] == 4
        assert bits_equal(chunk.shard, want['shard_after_reduce']), (case, rank)
        assert chunk.overflow == want['overflow'], (case, rank)
    dist.barrier()
    dist.destroy_process_group()


def optim_worker(rank, world, port, sync_overflow):
    """Replay make_golden.py::run_optim with this package's ElixirModule / ElixirOptimizer."""
    use_host_shim()
    dist = init_gloo(rank, world, port)
    sys.path.insert(0, GOLDEN)
    sys.path.insert(0, os.path.join(ROOT, 'tests'))
    from _util import close_1e6
    from make_golden import INF_STEP, OPTIM_CFG, OPTIM_CHUNK, OPTIM_HYPER, OPTIM_STEPS, optim_inputs
    from elixir_b200.optim import HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    golden = torch.load(os.path.join(GOLDEN, f'optim_w{world}.pt'))['ranks'][rank]
    cpu = torch.device('cpu')
    model, grads = optim_inputs(world, OPTIM_STEPS)
    sr = simple_plan(model, world, unified_dtype=torch.float16, shard_device=cpu, chunk_size=OPTIM_CHUNK,
                     rcache_device='cpu')
    assert [list(p.name_list) for p in sr.param_chunk_plans] == golden['plans']
    inner = HybridAdam(model.parameters(), adamw_mode=True, **OPTIM_HYPER)
    emodel = ElixirModule(model, sr, dist.GroupMember.WORLD, dtype=torch.float16)
    eoptim = ElixirOptimizer(emodel, inner, sync_overflow=sync_overflow, **OPTIM_CFG)
    chunks = emodel.param_chunks
    assert [c.valid_end for c in chunks] == [min(v, c.shard_size) for v, c in zip(golden['valid_end'], chunks)]
    for c, want in zip(chunks, golden['init_master']):
        assert bits_equal(c.paired_chunk.shard, want)
    any_rank_overflow = []
    for s in range(OPTIM_STEPS):
        want = golden['steps'][s]
        scale = eoptim.loss_scale
        if not sync_overflow:
            assert scale == want['scale_before'], (s, rank)
        named = {}
        for n, g in grads[s][rank].items():
            g = (g * scale).half()
            if s == INF_STEP and rank == world - 1 and n == 'fc2.weight':
                g.view(-1)[5] = float('inf')
            named[n] = g
        emodel.inject_gradients(named)
        flags = [c.overflow for c in chunks]
        if not sync_overflow:
            assert flags == want['chunk_overflow'], (s, rank)
            for c, g in zip(chunks, want['grad_shards']):
                assert bits_equal(c.shard, g), (s, rank)
        eoptim.step()
        ctl = eoptim.engine.read_control()
        assert ctl.status == 0
        if not sync_overflow:
            # the reference decides per rank: trajectories (and masters) follow the fixture of THIS rank
            assert eoptim.loss_scale == want['scale_after'], (s, rank)
            assert bool(ctl.skip) == any(want['chunk_overflow'])
            for c, m in zip(chunks, want['master']):
                ok, ratio = close_1e6(c.paired_chunk.shard, m.double(), rtol=2e-6)
                assert ok, (s, rank, ratio)
        else:
            # with the agreement all-reduce every rank skips exactly when any rank overflowed
            t = torch.tensor([float(any(flags))])
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            assert bool(ctl.skip) == bool(t.item())
            any_rank_overflow.append(bool(t.item()))
            scales = [torch.zeros(1) for _ in range(world)]
            dist.all_gather(scales, torch.tensor([eoptim.loss_scale]))
            assert all(x.item() == scales[0].item() for x in scales)
        # the low-precision shard is the rounded master again
        for c in chunks:
            assert bits_equal(c.shard, c.paired_chunk.shard.half())
    if sync_overflow:
        assert any_rank_overflow == [s == INF_STEP for s in range(OPTIM_STEPS)]
    dist.barrier()
    dist.destroy_process_group()


def _residency_model():
    import torch.nn as nn

    class TransposedLinear(nn.Module):
        """Uses a VIEW of its parameter, which autograd saves for backward in place of the parameter."""

        def __init__(self, n_in, n_out):
            super().__init__()
            self.weight = nn.Parameter(torch.randn(n_out, n_in) * 0.1)

        def forward(self, x):
            return x @ self.weight.t()

    class Net(nn.Module):

        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(50, 32)
            self.blocks = nn.ModuleList()
            for _ in range(4):
                self.blocks.append(nn.Sequential(nn.LayerNorm(32), nn.Linear(32, 64), nn.Tanh(), TransposedLinear(64, 32)))
            self.head = nn.Linear(32, 50, bias=False)
            self.head.weight = self.embed.weight    # tied: a private chunk

        def forward(self, ids):
            x = self.embed(ids)
            for block in self.blocks:
                x = x + block(x)
            return self.head(x).float().log_softmax(-1).mean().neg()

    torch.manual_seed(11)
    return Net()


def residency_check(group, rank, world, prefetch, dtype, device):
    """Scheduled residency (fewer blocks than public chunks) against everything-resident on the same model,
    data and steps: same loss, same reduced gradients, same parameters after the steps, bit for bit."""
    import copy
    from elixir_b200.chunk import FIFOScheduler, PrefetchScheduler
    from elixir_b200.optim import HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    base = _residency_model()
    torch.manual_seed(100 + rank)
    batches = [torch.randint(0, 50, (3, 7)).to(device) for _ in range(3)]
    on_host = device.type == 'cpu'

    def build(blocks):
        model = copy.deepcopy(base)
        sr = simple_plan(model, world, unified_dtype=dtype, shard_device=device, chunk_size=2400,
                         rcache_device='cpu' if on_host else None, public_block_number=blocks)
        emodel = ElixirModule(model, sr, group, prefetch=prefetch, dtype=dtype)
        eoptim = ElixirOptimizer(emodel, HybridAdam(model.parameters(), lr=1e-2, weight_decay=0.01), initial_scale=4.0)
        return emodel, eoptim

    full, full_opt = build(None)
    n_public = len(full.param_chunk_group.float_chunks)
    assert n_public >= 5 and not full.scheduled
    lean, lean_opt = build(2)
    assert lean.scheduled and lean.param_chunk_group.rcache.public_free_cnt == 2
    assert isinstance(lean.fetcher.scheduler, PrefetchScheduler if prefetch else FIFOScheduler)

    with torch.no_grad():
        assert bits_equal(full(batches[0]), lean(batches[0]))
    assert lean.param_chunk_group.rcache.public_free_cnt == 2    # everything went back

    for it, ids in enumerate(batches):
        l_full, l_lean = full(ids), lean(ids)
        assert bits_equal(l_full.detach(), l_lean.detach()), (it, rank)
        full_opt.backward(l_full)
        lean_opt.backward(l_lean)
        stats = dict(lean.fetcher.stats)
        assert stats['released'] > 0    # the replica cache really was too small
        if prefetch and it > 0:
            assert stats['ahead'] > 0 and stats['ahead_hit'] == stats['ahead'], stats    # the learnt trace was right
        assert lean.param_chunk_group.rcache.public_free_cnt == 2
        for a, b in zip(full.param_chunks, lean.param_chunks):
            assert bits_equal(a.shard, b.shard), (it, rank, a.chunk_id)    # reduced gradients
        full_opt.step()
        lean_opt.step()
        for a, b in zip(full.param_chunks, lean.param_chunks):
            assert bits_equal(a.shard, b.shard) and bits_equal(a.paired_chunk.shard, b.paired_chunk.shard)
        if not on_host:
            assert lean_opt.engine.read_control().status == 0
    if prefetch:
        assert not lean.fetcher.scheduler.learning and lean.fetcher.scheduler.total_steps > 0


def residency_worker(rank, world, port, prefetch, dtype_name):
    """The check above on gloo ranks in host memory."""
    use_host_shim()
    dist = init_gloo(rank, world, port)
    residency_check(dist.GroupMember.WORLD, rank, world, prefetch, getattr(torch, dtype_name), torch.device('cpu'))
    dist.barrier()
    dist.destroy_process_group()


def residency_worker_gpu(rank, world, port, prefetch, dtype_name):
    """The same on one GPU per rank over NCCL (gathers ahead and reduces on side streams)."""
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR='127.0.0.1',
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    residency_check(dist.group.WORLD, rank, world, prefetch, getattr(torch, dtype_name), dev)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def gpt2_check(group, device, dtype):
    """A micro GPT-2 (Hugging Face implementation, random weights, tied embedding) trained three steps:
    plain torch AdamW, the wrapper with everything resident, the wrapper with two replica-cache blocks and
    gathers ahead.  The two wrappers agree bit for bit; in fp32 they follow the plain run within the
    tolerance of the reference's own wrapper test (rtol 2e-6, atol 2e-5; test/wrapper/test_optimizer.py:49)."""
    import copy
    import torch.nn as nn
    from transformers import GPT2Config, GPT2LMHeadModel
    from elixir_b200.optim import HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan

    class Lm(nn.Module):

        def __init__(self):
            super().__init__()
            cfg = GPT2Config(n_embd=64, n_layer=3, n_head=4, n_positions=32, vocab_size=128, resid_pdrop=0.0,
                             embd_pdrop=0.0, attn_pdrop=0.0)
            self.module = GPT2LMHeadModel(cfg)

        def forward(self, input_ids, attention_mask):
            logits = self.module(input_ids=input_ids, attention_mask=attention_mask).logits
            return nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.size(-1)).float(),
                                               input_ids[:, 1:].reshape(-1))

    torch.manual_seed(0)
    plain = Lm().to(device)
    on_host = device.type == 'cpu'

    def build(blocks, prefetch):
        model = copy.deepcopy(plain)
        sr = simple_plan(model, 1, unified_dtype=dtype, shard_device=device, chunk_size=40000,
                         rcache_device='cpu' if on_host else None, public_block_number=blocks)
        emodel = ElixirModule(model, sr, group, prefetch=prefetch, dtype=dtype)
        return emodel, ElixirOptimizer(emodel, HybridAdam(model.parameters(), lr=1e-2, weight_decay=0.0),
                                       initial_scale=128.0)

    full, full_opt = build(None, False)
    lean, lean_opt = build(2, True)
    assert len(full.param_chunk_group.float_chunks) >= 4 and len(full.param_chunk_group.fused_chunks) == 1
    assert lean.scheduled and not full.scheduled
    opt = torch.optim.AdamW(plain.parameters(), lr=1e-2, weight_decay=0.0)
    for it in range(3):
        ids = torch.randint(0, 128, (4, 32), device=device)
        mask = torch.ones_like(ids)
        if dtype == torch.float:
            opt.zero_grad()
            loss = plain(ids, mask)
            loss.backward()
            opt.step()
        l_full = full(input_ids=ids, attention_mask=mask)
        l_lean = lean(input_ids=ids, attention_mask=mask)
        assert bits_equal(l_full.detach(), l_lean.detach())
        if dtype == torch.float:
            torch.testing.assert_close(l_full.detach(), loss.detach(), rtol=1e-5, atol=1e-5)
        full_opt.backward(l_full)
        lean_opt.backward(l_lean)
        stats = lean.fetcher.stats
        assert stats['released'] > 0
        if it > 0:
            assert stats['ahead'] > 0 and stats['ahead_hit'] == stats['ahead'], stats
        full_opt.step()
        lean_opt.step()
    got_full, got_lean = full.state_dict(), lean.state_dict()
    for name, ref in plain.state_dict().items():
        if name not in full.grad_state_dict:
            continue
        assert torch.equal(got_full[name], got_lean[name]), name
        if dtype == torch.float:
            a, b = got_full[name].to(device), ref
            if name.endswith('c_attn.bias'):
                # the key bias has no influence on the loss (softmax is shift-invariant): its gradient is
                # rounding noise, which Adam normalises into steps of +-lr; compare the query and value parts
                n = a.numel() // 3
                a, b = torch.cat([a[:n], a[2 * n:]]), torch.cat([b[:n], b[2 * n:]])
            torch.testing.assert_close(a, b, rtol=2e-6, atol=2e-5, msg=name)


def gpt2_worker(rank, world, port):
    use_host_shim()
    dist = init_gloo(rank, world, port)
    gpt2_check(dist.GroupMember.WORLD, torch.device('cpu'), torch.float)
    dist.destroy_process_group()


def abandoned_pass_worker(rank, world, port):
    """A forward with gradients enabled that no backward follows must not cost replica-cache blocks."""
    use_host_shim()
    dist = init_gloo(rank, world, port)
    import copy
    from elixir_b200.wrapper import ElixirModule, simple_plan
    cpu = torch.device('cpu')
    model = copy.deepcopy(_residency_model())
    sr = simple_plan(model, world, unified_dtype=torch.float, shard_device=cpu, chunk_size=2400, rcache_device='cpu',
                     public_block_number=2)
    emodel = ElixirModule(model, sr, dist.GroupMember.WORLD, dtype=torch.float)
    ids = torch.randint(0, 50, (3, 7))
    first = emodel(ids)    # leaves up to two chunks resident
    assert emodel.param_chunk_group.rcache.public_free_cnt < 2
    again = emodel(ids)
    assert bits_equal(first.detach(), again.detach())
    emodel.backward(again)
    assert emodel.param_chunk_group.rcache.public_free_cnt == 2
    dist.destroy_process_group()


def lifetime_worker(rank, world, port):
    """Dropping the wrapper frees the model: no parameter -> hook -> wrapper cycle survives a collection."""
    use_host_shim()
    dist = init_gloo(rank, world, port)
    import gc
    import weakref
    from elixir_b200.optim import HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    cpu = torch.device('cpu')

    def train(blocks):
        model = _residency_model()
        sr = simple_plan(model, 1, unified_dtype=torch.float, shard_device=cpu, chunk_size=2400, rcache_device='cpu',
                         public_block_number=blocks)
        emodel = ElixirModule(model, sr, dist.GroupMember.WORLD, prefetch=True, dtype=torch.float)
        eoptim = ElixirOptimizer(emodel, HybridAdam(model.parameters(), lr=1e-2), initial_scale=4.0)
        ids = torch.randint(0, 50, (3, 7))
        for _ in range(2):
            eoptim.zero_grad()
            eoptim.backward(emodel(ids))
            eoptim.step()
        chunk = emodel.param_chunks[0]
        return [weakref.ref(o) for o in (emodel, eoptim, eoptim.engine, chunk, chunk.paired_chunk.shard)]

    for blocks in (None, 2):
        refs = train(blocks)
        gc.collect()
        assert all(r() is None for r in refs), (blocks, [r() is None for r in refs])
    dist.destroy_process_group()


def fetcher_scenario_worker(rank, world, port):
    """Four chunks, two blocks, the access trace A B C A D: every decision of the fetcher spelled out."""
    use_host_shim()
    dist = init_gloo(rank, world, port)
    from elixir_b200.chunk import ChunkFetcher, ChunkGroup, FIFOScheduler, MemoryPool, PrefetchScheduler
    cpu = torch.device('cpu')

    def build(scheduler_of):
        pool = MemoryPool('cpu')
        pool.allocate(public_dtype=torch.float, public_block_size=64, public_block_number=2)
        group = ChunkGroup(pool)
        tensors = [torch.full((64,), float(i + 1)) for i in range(4)]
        chunks = [group.allocate_chunk([t], 64, torch.float, dist.GroupMember.WORLD,
                                       dict(shard_device=cpu, temp_device=cpu)) for t in tensors]
        fetcher = ChunkFetcher(scheduler_of(chunks), group, overlap=True)
        return pool, group, tensors, chunks, fetcher

    order = [0, 1, 2, 0, 3]

    def run(fetcher, group, tensors, chunks, log):
        with torch.no_grad():
            fetcher.reset()
            for i in order:
                got = fetcher.trans_to_compute([tensors[i]])
                assert got == [chunks[i]]
                fetcher.fetch_chunks(got)
                assert group.is_accessed(chunks[i]) and float(tensors[i][0]) == i + 1    # the data is there
                log.append((i, dict(fetcher.stats), sorted(c.chunk_id - chunks[0].chunk_id
                                                          for c in group.accessed_float_chunks)))
                fetcher.trans_to_hold([tensors[i]], phase='f')
            fetcher.release_all()
            fetcher.clear()

    # Belady on the known trace, gathers ahead
    pool, group, tensors, chunks, fetcher = build(lambda cs: PrefetchScheduler([[cs[i]] for i in order]))
    log = []
    run(fetcher, group, tensors, chunks, log)
    resident = [entry[2] for entry in log]
    #            after fetch of A: B gathered ahead; C cannot come (A is in use, nothing to release)
    assert resident == [[0, 1], [1, 2], [0, 2], [0, 3], [0, 3]], resident
    #            B: A (next use 3) leaves for C (use 2);  C: B (never again) leaves for A;  A: C leaves for D
    final = log[-1][1]
    assert final == dict(fetched=1, released=3, ahead=4, ahead_hit=4), final
    assert pool.public_free_cnt == 2

    # FIFO, nothing known about the future: every chunk is fetched on demand, the oldest releasable one leaves
    pool, group, tensors, chunks, fetcher = build(lambda cs: FIFOScheduler())
    log = []
    run(fetcher, group, tensors, chunks, log)
    assert [entry[2] for entry in log] == [[0], [0, 1], [1, 2], [0, 2], [0, 3]], [entry[2] for entry in log]
    assert log[-1][1] == dict(fetched=5, released=3, ahead=0, ahead_hit=0), log[-1][1]
    assert pool.public_free_cnt == 2

    # a replica cache that cannot hold what one fetch asks for
    pool, group, tensors, chunks, fetcher = build(lambda cs: FIFOScheduler())
    with torch.no_grad():
        fetcher.reset()
        both = fetcher.trans_to_compute(tensors[:3])
        try:
            fetcher.fetch_chunks(both)
        except RuntimeError as err:
            assert 'R cache is not enough' in str(err)
        else:
            raise AssertionError('three chunks in use at once fitted two blocks')
    dist.destroy_process_group()


def inject_worker(rank, world, port):
    """Gradients handed over by name (no autograd pass) land identically with a replica cache of two blocks."""
    use_host_shim()
    dist = init_gloo(rank, world, port)
    import copy
    from elixir_b200.wrapper import ElixirModule, simple_plan
    cpu = torch.device('cpu')
    base = _residency_model()
    gen = torch.Generator().manual_seed(9 + rank)
    grads = {n: torch.randn(p.shape, generator=gen) * 1e-2 for n, p in base.named_parameters()}

    def build(blocks, prefetch):
        model = copy.deepcopy(base)
        sr = simple_plan(model, world, unified_dtype=torch.float, shard_device=cpu, chunk_size=2400, rcache_device='cpu',
                         public_block_number=blocks)
        return ElixirModule(model, sr, dist.GroupMember.WORLD, prefetch=prefetch, dtype=torch.float)

    full, lean, ahead = build(None, False), build(2, False), build(2, True)
    for emodel in (full, lean, ahead):
        emodel.inject_gradients(grads)
    for a, b, c in zip(full.param_chunks, lean.param_chunks, ahead.param_chunks):
        assert bits_equal(a.shard, b.shard) and bits_equal(a.shard, c.shard)
        assert not b.is_replica and not c.is_replica
    assert lean.param_chunk_group.rcache.public_free_cnt == 2 and ahead.param_chunk_group.rcache.public_free_cnt == 2
    assert ahead.fetcher.scheduler.learning    # handing gradients over is not the model's access trace
    dist.barrier()
    dist.destroy_process_group()


def group_worker(rank, world, port):
    """ChunkGroup / MemoryPool bookkeeping the way the reference's test/chunk/test_group.py and test_block.py
    exercise it: lookups, gathers into public and private blocks, block accounting, release, reduce."""
    use_host_shim()
    dist = init_gloo(rank, world, port)
    from elixir_b200.chunk import BlockRequire, ChunkGroup, MemoryPool, PrivateBlock, PublicBlock, TensorState
    cpu = torch.device('cpu')
    block = PublicBlock(123, torch.float16, 'cpu')
    assert block.payload.numel() == 123 and block.payload.dtype == torch.float16 and block.memo_occ == 246
    assert PrivateBlock(77, torch.float, 'cpu').memo_occ == 308

    gen = torch.Generator().manual_seed(77)
    shapes = dict(a=(5, 48), b=(3, 16), c=(288,), d=(2, 3, 48), e=(2, 35))
    tensors = {k: torch.randn(s, generator=gen) for k, s in shapes.items()}
    originals = {k: t.clone() for k, t in tensors.items()}
    pool = MemoryPool('cpu')
    pool.allocate(public_block_size=288, public_block_number=2, private_block_list=[BlockRequire(72, torch.float)])
    assert (pool.public_free_cnt, pool.public_used_cnt) == (2, 0)
    group = ChunkGroup(rcache=pool)
    config = dict(shard_device=cpu, temp_device=cpu)
    c0 = group.allocate_chunk([tensors['a'], tensors['b']], 288, torch.float, dist.GroupMember.WORLD, dict(config))
    c1 = group.allocate_chunk([tensors['c']], 288, torch.float, dist.GroupMember.WORLD, dict(config))
    c2 = group.allocate_chunk([tensors['d']], 288, torch.float, dist.GroupMember.WORLD, dict(config))
    c3 = group.allocate_chunk([tensors['e']], 72, torch.float, dist.GroupMember.WORLD, dict(config, rcache_fused=True))
    assert group.float_chunks == {c0, c1, c2} and group.fused_chunks == {c3}
    assert group.tensors_to_chunks([tensors['e'], tensors['a'], tensors['b']]) == [c0, c3]    # by chunk id, once each

    def intact(*names):
        return all(torch.equal(tensors[n], originals[n]) for n in names)

    def hollow(name):    # shape kept, one element of storage: the data lives in the shards
        return tensors[name].shape == originals[name].shape and tensors[name].untyped_storage().nbytes() == 4

    assert hollow('a') and hollow('e')
    assert group.access_chunk(c0) and group.access_chunk(c1) and not group.access_chunk(c1)
    assert intact('a', 'b', 'c') and (pool.public_free_cnt, pool.public_used_cnt) == (0, 2)
    assert not group.rcache_enough_check(c2) and group.rcache_enough_check(c3)
    group.access_chunk(c3)    # private block: always there
    assert intact('e') and (pool.public_free_cnt, pool.public_used_cnt) == (0, 2)
    group.release_chunk(c1)
    assert hollow('c') and not group.is_accessed(c1) and group.rcache_enough_check(c2)
    group.access_chunk(c2)
    assert intact('d')
    try:
        group.access_chunk(c1)
    except IndexError:
        pass    # no free public block
    else:
        raise AssertionError('a third public chunk fitted two blocks')
    for state in (TensorState.COMPUTE, TensorState.HOLD_AFTER_BWD, TensorState.READY_FOR_REDUCE):
        group.tensor_trans_state(tensors['e'], state)
    assert c3.reduce_check
    group.reduce_chunk(c3)
    assert not c3.is_replica and not group.is_accessed(c3)
    group.release_chunk(c0)
    group.release_chunk(c2)
    assert (pool.public_free_cnt, pool.public_used_cnt) == (2, 0)
    for chunk, names in ((c0, 'ab'), (c1, 'c'), (c2, 'd')):    # everything survives a round trip through the shards
        group.access_chunk(chunk)
        assert intact(*names)
        group.release_chunk(chunk)
    dist.barrier()
    dist.destroy_process_group()
