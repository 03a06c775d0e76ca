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
