"""Sharded step over NCCL on 2+ GPUs of one box (skipped when fewer are visible): pre-multiplied-sum
reduce-scatter, probe, overflow agreement, fused update and all-gather, against the CPU oracle."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR='127.0.0.1',
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, 'tests'))
    import torch.distributed as dist
    from _util import bits_equal, close_1e6
    from elixir_b200 import comm
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    from oracle import oracle as orc
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    dtype, scale = torch.float16, 256.0
    chunk_sizes = [world * 4096 * 3, world * (4096 + 8), world * 4096 * 5]
    used = [chunk_sizes[0], chunk_sizes[1], chunk_sizes[2] // 2 + 7]
    engine = ChunkStepEngine(dev, dtype, DynamicGradScaler(initial_scale=scale, hysteresis=1, growth_interval=3),
                             process_group=dist.group.WORLD)
    host = orc.ChunkSet(dtype)
    host_ctl = orc.new_ctl(scale)
    hypers = [K.hyper(weight_decay=0.01)]
    host_state, full_masters = [], []
    for c, (C, u) in enumerate(zip(chunk_sizes, used)):
        S = C // world
        gen = torch.Generator().manual_seed(c)
        full = torch.randn(C, generator=gen) * 0.02
        full[u:] = 0
        full_masters.append(full)
        mine = full[rank * S:(rank + 1) * S].clone()
        nv = max(0, min(S, u - rank * S))
        lowp = torch.zeros(S, dtype=dtype)
        host.add_chunk(mine, torch.zeros(S), torch.zeros(S), lowp, nv, [(0, nv, 0)] if nv else [])
        host_state.append((mine, lowp, nv))
        engine.add_shard(mine.to(dev), torch.zeros(S, dtype=dtype, device=dev), nv, [(0, nv, 0)] if nv else [])
    engine.finalize()
    engine.set_hyper(hypers)
    gather = [torch.empty(C, dtype=dtype, device=dev) for C in chunk_sizes]
    for step in range(5):
        blocks, per_rank = [], []
        for c, C in enumerate(chunk_sizes):
            rank_grads = []
            for r in range(world):
                gen = torch.Generator().manual_seed(1000 * step + 10 * c + r)
                g = (torch.randn(C, generator=gen) * 1e-3 * host_ctl.scale).to(dtype)
                if step == 2 and c == 1 and r == world - 1:
                    g[5] = float('inf')    # lands in rank 0's shard only
                rank_grads.append(g)
            per_rank.append(rank_grads)
            blocks.append(rank_grads[rank].to(dev))
        # NCCL's fp16 summation order is its own, so parity of the step is defined GIVEN the reduced gradients:
        # capture them with the same collective first, then run the pipelined step on the same inputs
        reduced = []
        for c, C in enumerate(chunk_sizes):
            S = C // world
            out = torch.empty(S, dtype=dtype, device=dev)
            comm.reduce_scatter_avg(out, blocks[c].clone(), dist.group.WORLD)
            reduced.append(out.cpu())
            # ... and they agree with the reference's divide-then-sum to fp16 rounding
            want = orc.reduce_avg([g[rank * S:(rank + 1) * S].contiguous() for g in per_rank[c]])
            finite = torch.isfinite(want.float()) & torch.isfinite(reduced[c].float())
            assert torch.equal(torch.isfinite(want.float()), torch.isfinite(reduced[c].float()))
            err = (reduced[c].float() - want.float()).abs()[finite]
            assert float(err.max()) <= 2 * 2.0**-10 * float(want.float().abs()[finite].max())
        engine.step_sharded(blocks, gather)
        torch.cuda.synchronize()
        for c in range(len(chunk_sizes)):
            host_state[c][1].copy_(reduced[c])
        any_inf = step == 2
        if any_inf:
            host_ctl.found_inf = 1    # agreement: every rank skips, also those whose shards are clean
        skipped = host.step(host_ctl, engine.scaler.cfg, hypers, probe=True, f64=True)
        ctl = engine.read_control()
        assert bool(ctl.skip) == skipped == any_inf, (step, rank)
        assert (ctl.scale, ctl.step) == (host_ctl.scale, host_ctl.step)
        for c, C in enumerate(chunk_sizes):
            S = C // world
            ok, ratio = close_1e6(engine.shards[c][0], host_state[c][0].double(), rtol=2e-6)
            assert ok, (step, rank, c, ratio)
            # the gathered block holds every rank's refreshed shard
            mine16 = engine.shards[c][3]
            assert bits_equal(gather[c][rank * S:(rank + 1) * S], mine16)
            others = [torch.empty_like(mine16) for _ in range(world)]
            dist.all_gather(others, mine16)
            assert bits_equal(gather[c], torch.cat(others))
    assert engine.read_control().status == 0
    dist.barrier()
    dist.destroy_process_group()


def _p2p_worker(rank, world, port, dtype_name='float16', pool=None, staged=False, pull_variant=1, overlapped=False,
                probe_first=False, host_buffers=False, pull_push=False):
    """The NVLink path: pull reduce-scatter + probe, overflow agreement inside the barrier, fused update with
    push all-gather — no NCCL collective in the step."""
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR='127.0.0.1',
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, 'tests'))
    import torch.distributed as dist
    from _util import bits_equal, close_1e6
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    from oracle import oracle as orc
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    dtype, scale = getattr(torch, dtype_name), 256.0
    chunk_sizes = [world * 4096 * 40, world * (4096 + 16), world * 4096 * 5, world * 24]
    used = [chunk_sizes[0], chunk_sizes[1], chunk_sizes[2] // 2 + 7, 9]
    if pool:
        # pooled blocks: equal-sized chunks, chunk k lives in block k % pool
        chunk_sizes = [world * (4096 * 6 + 32)] * 5
        used = [chunk_sizes[0], chunk_sizes[0], chunk_sizes[0] // 2 + 7, chunk_sizes[0], 9]
    engine = ChunkStepEngine(dev, dtype, DynamicGradScaler(initial_scale=scale, hysteresis=1, growth_interval=3),
                             process_group=dist.group.WORLD)
    host = orc.ChunkSet(dtype)
    host_ctl = orc.new_ctl(scale)
    hypers = [K.hyper(weight_decay=0.01)]
    host_state = []
    for c, (C, u) in enumerate(zip(chunk_sizes, used)):
        S = C // world
        gen = torch.Generator().manual_seed(c)
        full = torch.randn(C, generator=gen) * 0.02
        full[u:] = 0
        mine = full[rank * S:(rank + 1) * S].clone()
        nv = max(0, min(S, u - rank * S))
        lowp = torch.zeros(S, dtype=dtype)
        host.add_chunk(mine, torch.zeros(S), torch.zeros(S), lowp, nv, [(0, nv, 0)] if nv else [])
        host_state.append((mine, lowp, nv))
        engine.add_shard(mine.to(dev), torch.zeros(S, dtype=dtype, device=dev), nv, [(0, nv, 0)] if nv else [])
    engine.finalize()
    engine.set_hyper(hypers)
    engine.enable_p2p(chunk_sizes, timeout_ms=5000, pool=pool)
    K.set_tuning(pull_variant=pull_variant)
    if staged:
        engine.enable_staging(pool=2)
    if overlapped:
        engine.enable_single_pass()

    host_in = [torch.empty(C, dtype=dtype).pin_memory() for C in chunk_sizes] if host_buffers else None
    host_out = [torch.empty(C // world, dtype=dtype).pin_memory() for C in chunk_sizes] if host_buffers else None

    def fill(step, into_blocks=not host_buffers):
        per_rank = []
        for c, C in enumerate(chunk_sizes):
            rank_grads = []
            if pool and c >= pool:
                # the block is shared with chunk c - pool: same gradients (the engine reads what is in the block)
                per_rank.append(per_rank[c - pool])
                continue
            for r in range(world):
                gen = torch.Generator().manual_seed(1000 * step + 10 * c + r)
                g = (torch.randn(C, generator=gen) * 1e-3 * host_ctl.scale).to(dtype)
                if step == 2 and c == 1 and r == world - 1:
                    g[5] = float('inf')    # lands in rank 0's shard only
                rank_grads.append(g)
            per_rank.append(rank_grads)
            if into_blocks:
                engine.grad_block(c).copy_(rank_grads[rank])
            else:
                host_in[c].copy_(rank_grads[rank])
        if not into_blocks:
            for c in range(len(chunk_sizes)):
                if pool and c >= pool:
                    host_in[c].copy_(host_in[c - pool])
        return per_rank

    # the pull alone: bit-exact against the oracle's fp32-accumulated average
    per_rank = fill(0, into_blocks=True)
    engine.peer_barrier(engine.ctl)
    K.pull_reduce_multi(engine.table, engine.grad_slab.table, engine.block_off, engine.ctl,
                        chunk_flags=engine.chunk_flags)
    engine.peer_barrier(engine.ctl)
    torch.cuda.synchronize()
    for c, C in enumerate(chunk_sizes):
        S = C // world
        want = orc.reduce_avg_f32acc([g[rank * S:(rank + 1) * S].contiguous() for g in per_rank[c]])
        assert bits_equal(engine.shards[c][3], want), (rank, c)
    assert engine.chunk_flags.sum().item() == 0

    for step in range(5):
        per_rank = fill(step)
        if staged:
            engine.step_sharded_staged()
        elif host_buffers:
            engine.step_sharded_p2p(host_grads=host_in, host_params=host_out)
        elif overlapped:
            engine.step_sharded_overlapped(pull_ctas=40)
        elif probe_first:
            engine.step_sharded_probe_first(pull_ctas=40)
        elif pull_push:
            engine.step_sharded_pull_push()
        else:
            engine.step_sharded_p2p()
        torch.cuda.synchronize()
        shards = engine.current_shards()
        for c, C in enumerate(chunk_sizes):
            S = C // world
            host_state[c][1].copy_(orc.reduce_avg_f32acc([g[rank * S:(rank + 1) * S].contiguous()
                                                          for g in per_rank[c]]))
        any_inf = step == 2
        if any_inf:
            host_ctl.found_inf = 1    # agreement: every rank skips
        skipped = host.step(host_ctl, engine.scaler.cfg, hypers, probe=True, f64=True)
        ctl = engine.read_control()
        assert ctl.status == 0, (step, rank, ctl.status)
        assert bool(ctl.skip) == skipped == any_inf, (step, rank)
        assert (ctl.scale, ctl.step) == (host_ctl.scale, host_ctl.step)
        for c, C in enumerate(chunk_sizes):
            S = C // world
            ok, ratio = close_1e6(shards[c][0], host_state[c][0].double(), rtol=2e-6)
            assert ok, (step, rank, c, ratio)
            mine16 = shards[c][3]
            others = [torch.empty_like(mine16) for _ in range(world)]
            dist.all_gather(others, mine16)
            if not pool or c + pool >= len(chunk_sizes):    # a pooled gather block holds its LAST chunk
                assert bits_equal(engine.gather_block(c), torch.cat(others)), (step, rank, c)
            if host_buffers:
                assert bits_equal(host_out[c], mine16), (step, rank, c)
    dist.barrier()
    dist.destroy_process_group()


def _mm_worker(rank, world, port, dtype_name='float16', host_buffers=False):
    """The single-pass sharded step: reduce-scatter, update and all-gather in one kernel through the NVLink switch
    (multimem.ld_reduce / multimem.st on symmetric memory).  The switch forms the sum of the ranks' values with an
    arithmetic of its own (for more than two ranks not the rank-order fp32 sum rounded once), exactly as NCCL's
    order is its own, so parity of the step is defined GIVEN the reduced gradients: they are captured first with
    ``elx_multimem_reduce`` (the same switch operation, stored instead of consumed), checked against the exact
    average to the rounding of the 16-bit format, and the oracle then steps on them."""
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR='127.0.0.1',
                      MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, 'tests'))
    import torch.distributed as dist
    from _util import bits_equal, close_1e6
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    from oracle import oracle as orc
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    dtype, scale = getattr(torch, dtype_name), 256.0
    ulp = 2.0**-10 if dtype == torch.float16 else 2.0**-7
    chunk_sizes = [world * 4096 * 40, world * (4096 + 16), world * 4096 * 5, world * 24]
    used = [chunk_sizes[0], chunk_sizes[1], chunk_sizes[2] // 2 + 7, 9]
    engine = ChunkStepEngine(dev, dtype, DynamicGradScaler(initial_scale=scale, hysteresis=1, growth_interval=3),
                             process_group=dist.group.WORLD)
    host = orc.ChunkSet(torch.float32)    # the oracle steps on the averaged gradients as fp32 values: float(sum) / W
    host_ctl = orc.new_ctl(scale)
    hypers = [K.hyper(weight_decay=0.01)]
    host_state = []
    for c, (C, u) in enumerate(zip(chunk_sizes, used)):
        S = C // world
        gen = torch.Generator().manual_seed(c)
        full = torch.randn(C, generator=gen) * 0.02
        full[u:] = 0
        mine = full[rank * S:(rank + 1) * S].clone()
        nv = max(0, min(S, u - rank * S))
        grad32 = torch.zeros(S)
        host.add_chunk(mine, torch.zeros(S), torch.zeros(S), grad32, nv, [(0, nv, 0)] if nv else [])
        host_state.append((mine, grad32, nv))
        engine.add_shard(mine.to(dev), torch.zeros(S, dtype=dtype, device=dev), nv, [(0, nv, 0)] if nv else [])
    engine.finalize()
    engine.set_hyper(hypers)
    engine.enable_single_pass()
    engine.enable_multicast(chunk_sizes, timeout_ms=5000)
    host_in = [torch.empty(C, dtype=dtype).pin_memory() for C in chunk_sizes] if host_buffers else None
    host_out = [torch.empty(C // world, dtype=dtype).pin_memory() for C in chunk_sizes] if host_buffers else None

    def one_step(step):
        per_rank = []
        for c, C in enumerate(chunk_sizes):
            rank_grads = []
            for r in range(world):
                gen = torch.Generator().manual_seed(1000 * step + 10 * c + r)
                g = (torch.randn(C, generator=gen) * 1e-3 * host_ctl.scale).to(dtype)
                if step == 2 and c == 1 and r == world - 1:
                    g[5] = float('inf')    # lands in rank 0's shard only
                rank_grads.append(g)
            per_rank.append(rank_grads)
            engine.grad_block(c).copy_(rank_grads[rank])
            if host_buffers:
                host_in[c].copy_(rank_grads[rank])
        # every rank's blocks are in place; what the switch makes of them, seen before the step consumes it
        torch.cuda.synchronize()
        dist.barrier()
        sums = [t.cpu() for t in engine.switch_reduced_gradients()]
        torch.cuda.synchronize()
        dist.barrier()
        for c, C in enumerate(chunk_sizes):
            S = C // world
            exact = torch.stack([g[rank * S:(rank + 1) * S].double() for g in per_rank[c]]).sum(0)
            got = sums[c].double()
            finite = torch.isfinite(exact)
            assert torch.equal(torch.isfinite(got), finite), (step, rank, c)
            # a few roundings to the 16-bit format on the way, each at most one unit in the last place of a partial sum
            bound = world * ulp * torch.stack([g[rank * S:(rank + 1) * S].double().abs() for g in per_rank[c]]).sum(0)
            assert bool(((got - exact).abs()[finite] <= bound[finite]).all()), (step, rank, c)
            host_state[c][1].copy_(sums[c].float() * (1.0 / world))    # exact in fp32: what the kernel feeds to Adam
        if host_buffers:    # blocks filled from pinned memory chunk by chunk, shards copied out behind their update
            engine.step_sharded_single_pass(host_grads=host_in, host_params=host_out)
        else:
            engine.step_sharded_single_pass()
        torch.cuda.synchronize()
        any_inf = step == 2
        if any_inf:
            host_ctl.found_inf = 1    # agreement: every rank skips
        skipped = host.step(host_ctl, engine.scaler.cfg, hypers, probe=True, f64=True)
        ctl = engine.read_control()
        assert ctl.status == 0, (step, rank, ctl.status)
        assert bool(ctl.skip) == skipped == any_inf, (step, rank)
        assert (ctl.scale, ctl.step, ctl.repair) == (host_ctl.scale, host_ctl.step, int(any_inf))
        shards = engine.current_shards()
        for c, C in enumerate(chunk_sizes):
            S = C // world
            ok, ratio = close_1e6(shards[c][0], host_state[c][0].double(), rtol=2e-6)
            assert ok, (step, rank, c, ratio)
            want16 = torch.empty(S, dtype=dtype)
            orc.cast(shards[c][0].cpu(), want16)
            assert bits_equal(shards[c][3], want16), (step, rank, c)
            if host_buffers:    # also after the overflow step, when the rebuilt working copies are sent again
                assert bits_equal(host_out[c], want16), (step, rank, c)

    def agree(failure):
        verdict = torch.tensor([0 if failure is None else 1], device=dev)
        dist.all_reduce(verdict, op=dist.ReduceOp.MAX)
        return bool(verdict.item())

    # A rank that fails must not leave while the others still use memory bound to the multicast object: every
    # rank learns of a failure between steps, all stop together, and the error is raised after an orderly teardown.
    failure = None
    for step in range(5):
        try:
            one_step(step)    # its two host-side barriers come before anything that can raise
        except Exception as exc:    # noqa: BLE001
            failure = f'{type(exc).__name__}: {exc}'
        if agree(failure):
            break
        shards = engine.current_shards()
        for c in range(len(chunk_sizes)):    # the gathered block holds every rank's refreshed shard
            others = [torch.empty_like(shards[c][3]) for _ in range(world)]
            dist.all_gather(others, shards[c][3])
            if not bits_equal(engine.gather_block(c), torch.cat(others)):
                failure = failure or f'step {step} rank {rank} chunk {c}: gathered block differs from the shards'
        if agree(failure):
            break
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    assert failure is None, failure


@pytest.mark.parametrize('world,dtype_name', [(2, 'float16'), (2, 'bfloat16'), (4, 'float16'), (8, 'float16')])
def test_sharded_single_pass_step_through_the_switch(world, dtype_name):
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_mm_worker, args=(world, 29900 + world + (10 if dtype_name == 'bfloat16' else 0), dtype_name), nprocs=world)


def test_sharded_single_pass_step_fed_from_host_buffers():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    mp.spawn(_mm_worker, args=(2, 29935, 'float16', True), nprocs=2)


@pytest.mark.parametrize('world', [2, 4])
def test_sharded_step_staged_copy_engines(world):
    """The same step with the copy engines moving the slices (local staging + reduce kernel on local memory,
    copies of the refreshed shards into the gather blocks): same oracle, same bits."""
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_p2p_worker, args=(world, 29870 + world, 'float16', None, True), nprocs=world)


@pytest.mark.parametrize('world,dtype_name', [(2, 'float16'), (2, 'bfloat16'), (4, 'float16')])
def test_sharded_step_p2p_per_lane_pull(world, dtype_name):
    """pull_variant=0: the slices are read with per-lane 256-bit peer loads instead of bulk copies into shared
    memory (the default); same rank-order fp32 accumulation, so the same bits as the oracle."""
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_p2p_worker, args=(world, 29880 + world, dtype_name, None, False, 0), nprocs=world)


def test_sharded_step_with_the_reduction_overlapping_the_update():
    """Out-of-place update, so chunk k may be updated while chunk k + 1 is still being reduced on another stream
    (the SMs split between the two kernels): same oracle, same bits as the two-phase step."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    mp.spawn(_p2p_worker, args=(2, 29865, 'float16', None, False, 1, True), nprocs=2)


@pytest.mark.parametrize('world,dtype_name', [(2, 'float16'), (2, 'bfloat16'), (4, 'float16')])
def test_sharded_step_decided_on_the_inputs_with_the_reduction_overlapping_the_update(world, dtype_name):
    """The overflow word formed from every rank's own gradient blocks before the reduction (the fp32-accumulated
    average is non-finite exactly when an input is), so that the in-place update of chunk k runs while chunk
    k + 1 is still being reduced: same oracle, same bits as the two-phase step."""
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_p2p_worker, args=(world, 29920 + world + (10 if dtype_name == 'bfloat16' else 0), dtype_name, None, False, 1,
                                False, True), nprocs=world)


@pytest.mark.parametrize('pool', [None, 2])
def test_sharded_step_p2p_fed_from_host_buffers(pool):
    """Gradient blocks filled from pinned host memory chunk by chunk while earlier chunks are reduced, refreshed
    shards copied out behind their update; with a pool of two blocks a block is refilled only once every rank is
    done reading its previous tenant."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    mp.spawn(_p2p_worker, args=(2, 29940 + (pool or 0), 'float16', pool, False, 1, False, False, True), nprocs=2)


@pytest.mark.parametrize('dtype_name', ['float16', 'bfloat16'])
def test_sharded_step_with_both_collectives_inside_the_update_kernel(dtype_name):
    """Two ranks: per tile the update kernel fetches both ranks' gradient slices, averages them as the pull kernel
    does, updates in place and stores the refreshed tile to both gather blocks; the decision comes from a probe of
    the inputs.  Same oracle, same bits as the two-phase step."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    mp.spawn(_p2p_worker, args=(2, 29950 + (1 if dtype_name == 'bfloat16' else 0), dtype_name, None, False, 1, False, False,
                                False, True), nprocs=2)


def test_sharded_step_p2p_pooled_blocks():
    """Chunk-by-chunk NVLink step over a pool of 2 replicated blocks for 5 chunks."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    mp.spawn(_p2p_worker, args=(2, 29860, 'float16', 2), nprocs=2)


@pytest.mark.parametrize('world', [2, 4, 8])
def test_sharded_step_p2p_kernels(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_p2p_worker, args=(world, 29820 + world), nprocs=world)


def _wrapper_worker(rank, world, port, nvlink=False, host_shards=False):
    """ElixirModule + ElixirOptimizer over NCCL with a real forward / backward, against plain data-parallel
    training (gradients averaged by hand, torch.optim.AdamW): the reference's test/wrapper/test_optimizer.py
    in spirit, tolerance included."""
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR='127.0.0.1',
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, 'tests'))
    import copy
    import torch.distributed as dist
    import torch.nn as nn
    from elixir_b200.optim import HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    torch.manual_seed(0)
    plain = nn.Sequential(nn.Linear(40, 72), nn.GELU(), nn.Linear(72, 72), nn.GELU(), nn.Linear(72, 6)).to(dev)
    wrapped = copy.deepcopy(plain)
    opt = torch.optim.AdamW(plain.parameters(), lr=1e-2, betas=(0.875, 0.99609375), weight_decay=0.0)
    sr = simple_plan(wrapped, world, split_number=3, unified_dtype=torch.float,
                     peer_group=dist.group.WORLD if nvlink else None,
                     shard_device=torch.device('cpu') if host_shards else None)
    inner = HybridAdam(wrapped.parameters(), lr=1e-2, betas=(0.875, 0.99609375), weight_decay=0.0)
    emodel = ElixirModule(wrapped, sr, dist.group.WORLD, dtype=torch.float)
    eopt = ElixirOptimizer(emodel, inner)
    assert emodel.nvlink_step == nvlink
    assert all(c.host_resident == host_shards for c in emodel.param_chunks)
    for step in range(3):
        torch.manual_seed(100 * step + rank)    # every rank its own batch
        x = torch.randn(16, 40, device=dev)
        opt.zero_grad()
        plain(x).pow(2).mean().backward()
        for p in plain.parameters():
            dist.all_reduce(p.grad)
            p.grad /= world
        opt.step()
        eopt.zero_grad()
        eopt.backward(emodel(x).pow(2).mean())
        eopt.step()
    got = emodel.state_dict()
    for name, ref in plain.state_dict().items():
        torch.testing.assert_close(got[name].to(dev), ref, rtol=2e-6, atol=2e-5)
    assert eopt.engine.read_control().status == 0
    # sharded checkpoint round trip: only rank 0 supplies the tensors, every rank ends with its shard
    zeros = {k: torch.zeros_like(v) for k, v in got.items()}
    emodel.load_state_dict(zeros if rank == 0 else None, only_rank_0=True)
    assert all(float(v.abs().max()) == 0.0 for v in emodel.state_dict().values())
    emodel.load_state_dict(got if rank == 0 else None, only_rank_0=True)
    again = emodel.state_dict()
    for name in got:
        assert torch.equal(again[name], got[name])
    dist.barrier()
    dist.destroy_process_group()


def test_wrapper_data_parallel_training_matches_plain_ddp():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    mp.spawn(_wrapper_worker, args=(2, 29840), nprocs=2)


def _amp_worker(rank, world, port):
    """fp16 working copies, fp32 gradient accumulation across ranks (reduce_always_fp32), loss scale 1: the
    setting of the reference's test/wrapper/test_amp.py.  Compared with hand-written mixed precision: fp16
    replica refreshed from fp32 masters, fp16 backward, gradients averaged in fp32, torch AdamW on the masters."""
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR='127.0.0.1',
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    sys.path.insert(0, ROOT)
    import copy
    import torch.distributed as dist
    import torch.nn as nn
    from elixir_b200.optim import HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    torch.manual_seed(0)
    masters = nn.Sequential(nn.Linear(40, 72), nn.GELU(), nn.Linear(72, 72), nn.GELU(), nn.Linear(72, 6)).to(dev)
    replica = copy.deepcopy(masters).half()
    wrapped = copy.deepcopy(masters)
    opt = torch.optim.AdamW(masters.parameters(), lr=1e-2, betas=(0.875, 0.99609375), weight_decay=0.0)
    sr = simple_plan(wrapped, world, split_number=3, unified_dtype=torch.float16)
    inner = HybridAdam(wrapped.parameters(), lr=1e-2, betas=(0.875, 0.99609375), weight_decay=0.0)
    emodel = ElixirModule(wrapped, sr, dist.group.WORLD, dtype=torch.float16, reduce_always_fp32=True, output_fp32=True)
    eopt = ElixirOptimizer(emodel, inner, initial_scale=1.0)
    for step in range(2):
        torch.manual_seed(100 * step + rank)
        x = torch.randn(16, 40, device=dev)
        with torch.no_grad():
            for h, m in zip(replica.parameters(), masters.parameters()):
                h.copy_(m)
        replica.zero_grad()
        replica(x.half()).float().pow(2).mean().backward()
        for h, m in zip(replica.parameters(), masters.parameters()):
            g = h.grad.float() / world    # divide, then sum, in fp32 (elixir/chunk/core/chunk.py:292-303)
            dist.all_reduce(g)
            m.grad = g.half().float()     # the averaged gradient goes back to the fp16 chunk (chunk.py:306-308)
        opt.step()
        eopt.zero_grad()
        eopt.backward(emodel(x).pow(2).mean())
        eopt.step()
    got = emodel.state_dict()
    for name, ref in masters.state_dict().items():
        torch.testing.assert_close(got[name].to(dev), ref)
    assert eopt.engine.read_control().status == 0
    dist.barrier()
    dist.destroy_process_group()


def test_wrapper_amp_with_fp32_gradient_reduction():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    mp.spawn(_amp_worker, args=(2, 29845), nprocs=2)


def test_wrapper_training_with_the_nvlink_step_matches_plain_ddp():
    """The same training with the replica cache in peer-mapped memory: no NCCL collective after the first
    gather; reduce-scatter and all-gather happen inside the optimizer's kernels."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    mp.spawn(_wrapper_worker, args=(2, 29850, True), nprocs=2)


def test_sharded_step_p2p_kernels_bf16():
    """The OPT-66B configuration's dtype (bf16 chunks) through the same NVLink path, on two ranks."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    mp.spawn(_p2p_worker, args=(2, 29830, 'bfloat16'), nprocs=2)


@pytest.mark.parametrize('world', [2, 4])
def test_sharded_step_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    mp.spawn(_worker, args=(world, 29800 + world), nprocs=world)


@pytest.mark.parametrize('prefetch', [False, True])
def test_scheduled_residency_over_nccl(prefetch):
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    import _dist_workers as W
    mp.spawn(W.residency_worker_gpu, args=(2, 29860 + int(prefetch), prefetch, 'float16'), nprocs=2)


def test_wrapper_data_parallel_training_with_shards_in_host_memory():
    """shard_device=cpu over NCCL: the reduce-scatter leaves the average in the block, the landing kernel moves
    it to the pinned shard over PCIe, the update runs on the pinned arrays, the gather starts from them."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    mp.spawn(_wrapper_worker, args=(2, 29845, False, True), nprocs=2)
