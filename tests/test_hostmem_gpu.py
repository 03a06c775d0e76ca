"""Shards kept in pinned host memory (the reference's shard_device=cpu placement): the same GPU kernels
update them in place over PCIe.  Results must equal the device-resident run bit for bit (the load/store
variant of the update is bit-identical to the bulk-copy pipeline), and therefore the oracle's within the
same bounds."""
import copy

import pytest
import torch

from _util import bits_equal, close_1e6, make_chunk

pytestmark = pytest.mark.gpu


def _engine(device, dtype, shards, host, segments, scaler_kw=None):
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    scaler = DynamicGradScaler(**(scaler_kw or dict(initial_scale=64.0, growth_interval=2, hysteresis=1)))
    eng = ChunkStepEngine(device, dtype, scaler)
    held = []
    for k, ((master, m, v, lowp), (n_valid, segs)) in enumerate(zip(shards, segments)):
        if host is True or (host == 'mixed' and k % 2 == 0):
            arrays = [t.clone().pin_memory() for t in (master, m, v, lowp)]
        else:
            arrays = [t.clone().to(device) for t in (master, m, v, lowp)]
        eng.add_shard(arrays[0], arrays[3], n_valid, segs, exp_avg=arrays[1], exp_avg_sq=arrays[2])
        held.append(arrays)
    eng.finalize()
    return eng, held


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16, torch.float32])
def test_host_resident_step_equals_device_resident_step(cuda, oracle, dtype):
    import elixir_b200.kernels as K
    sizes = [3 * 4096 + 17, 8 * 4096, 4096 - 5, 40000]
    shards = [make_chunk(n, dtype, seed=50 + i) for i, n in enumerate(sizes)]
    segments = [(sizes[0] - 9, [(0, 5000, 0), (5000, sizes[0] - 9, 1)]), (sizes[1], [(0, sizes[1], 0)]),
                (sizes[2], [(3, sizes[2], 1)]), (30000, [(0, 12345, 1), (12345, 30000, 0)])]
    hypers = [K.hyper(lr=1e-3, weight_decay=0.01), K.hyper(lr=3e-3, betas=(0.8, 0.95), weight_decay=0.0, adamw_mode=False)]
    on_dev, dev_arrays = _engine(cuda, dtype, shards, False, segments)
    on_host, host_arrays = _engine(cuda, dtype, shards, True, segments)
    streamed, streamed_arrays = _engine(cuda, dtype, shards, True, segments)
    streamed.enable_streaming(slots=3)    # copy engines + staging sets instead of kernel accesses over PCIe
    mixed, mixed_arrays = _engine(cuda, dtype, shards, 'mixed', segments)    # shards 0 and 2 on the host, 1 and 3 not
    mixed.enable_streaming(slots=2)
    assert on_host.table.host_resident and not on_dev.table.host_resident
    assert all(K.is_mapped_host(t) for t in on_host.shards[0][:4])    # moments included
    gen = torch.Generator().manual_seed(3)
    for step in range(4):
        for eng in (on_dev, on_host, streamed, mixed):
            eng.set_hyper(hypers)
        grads = []
        for n in sizes:
            g = (torch.randn(n, generator=gen) * 1e-3 * 64).to(dtype)
            if step == 2 and n == sizes[1]:
                g[777] = float('inf')    # one overflow: the whole step is skipped, the scale backs off
            grads.append(g)
        for eng in (on_dev, on_host, streamed, mixed):
            for k, g in enumerate(grads):
                eng.land(k, g.to(cuda))    # device block -> shard (host shard: written over PCIe) + probe
            if eng in (streamed, mixed):
                eng.step_streamed()
            else:
                eng.step()
        torch.cuda.synchronize()
        a = on_dev.read_control()
        assert a.status == 0 and bool(a.skip) == (step == 2)
        for eng, arrays in ((on_host, host_arrays), (streamed, streamed_arrays), (mixed, mixed_arrays)):
            b = eng.read_control()
            assert (a.skip, a.scale, a.step, a.status) == (b.skip, b.scale, b.step, b.status)
            for da, ha in zip(dev_arrays, arrays):
                for x, y in zip(da, ha):
                    assert bits_equal(x, y), step
    # and the host-resident result is the oracle's, within the usual bounds, for the last clean step
    # (both engines agree bit for bit, so one comparison covers them)
    assert on_host.read_control().step == 3


def test_probe_and_refresh_work_on_host_resident_shards(cuda):
    import elixir_b200.kernels as K
    n = 5 * 4096 + 123
    g = (torch.randn(n) * 3).half().pin_memory()
    flag = torch.zeros(1, dtype=torch.int32, device=cuda)
    K.grad_check(g, flag=flag)
    assert int(flag.item()) == 0
    g[n - 1] = float('nan')
    K.grad_check(g, n_valid=n - 1, flag=flag)
    assert int(flag.item()) == 0    # outside the probed prefix
    K.grad_check(g, flag=flag)
    assert int(flag.item()) == 1
    master = torch.randn(n).pin_memory()
    out = torch.empty(n, dtype=torch.bfloat16).pin_memory()
    K.cast_copyback(master, out)
    torch.cuda.synchronize()
    assert bits_equal(out, master.bfloat16())


def test_pageable_host_memory_and_collective_paths_are_refused(cuda):
    import elixir_b200.kernels as K
    from elixir_b200.engine import ChunkStepEngine
    flag = torch.zeros(1, dtype=torch.int32, device=cuda)
    with pytest.raises(RuntimeError, match='no CPU path'):
        K.grad_check(torch.zeros(4096, dtype=torch.float16), flag=flag)
    eng = ChunkStepEngine(cuda, torch.float16)
    with pytest.raises(RuntimeError, match='no CPU path'):
        eng.add_shard(torch.zeros(4096), torch.zeros(4096, dtype=torch.float16), 4096, [(0, 4096, 0)])
    eng.add_shard(torch.zeros(4096).pin_memory(), torch.zeros(4096, dtype=torch.float16).pin_memory(), 4096,
                  [(0, 4096, 0)])
    eng.finalize()
    with pytest.raises(RuntimeError, match='device-resident'):
        eng.step_sharded([torch.zeros(4096, dtype=torch.float16, device=cuda)], [None])


class _Net(torch.nn.Module):

    def __init__(self):
        super().__init__()
        self.net = torch.nn.Sequential(torch.nn.Linear(48, 96), torch.nn.GELU(), torch.nn.Linear(96, 96), torch.nn.GELU(),
                                       torch.nn.Linear(96, 8))

    def forward(self, x):
        return self.net(x).float().pow(2).mean()


@pytest.mark.parametrize('blocks', [None, 1])
def test_wrapper_with_shards_in_host_memory_trains_identically(cuda, blocks):
    """ElixirModule / ElixirOptimizer with shard_device=cpu against shard_device=cuda: same losses, same
    parameters, same optimizer state after three steps; also with a replica cache of a single block."""
    import torch.distributed as dist
    from elixir_b200.optim import HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    if not dist.is_initialized():
        dist.init_process_group('gloo', init_method='tcp://127.0.0.1:29791', rank=0, world_size=1)
    torch.manual_seed(0)
    base = _Net().to(cuda)

    def build(shard_device):
        model = copy.deepcopy(base)
        sr = simple_plan(model, 1, split_number=3, unified_dtype=torch.float16, shard_device=shard_device,
                         public_block_number=blocks)
        emodel = ElixirModule(model, sr, dist.GroupMember.WORLD, dtype=torch.float16)
        return emodel, ElixirOptimizer(emodel, HybridAdam(model.parameters(), lr=1e-2, weight_decay=0.01),
                                       initial_scale=256.0)

    dev, dev_opt = build(cuda)
    host, host_opt = build(torch.device('cpu'))
    assert all(c.host_resident and c.shard.is_pinned() and c.paired_chunk.shard.is_pinned() for c in host.param_chunks)
    assert host_opt.engine.table.host_resident and host_opt.engine.device == cuda
    for step in range(3):
        x = torch.randn(16, 48, device=cuda)
        la, lb = dev(x), host(x)
        assert bits_equal(la.detach(), lb.detach())
        dev_opt.backward(la)
        host_opt.backward(lb)
        dev_opt.step()
        host_opt.step()
    torch.cuda.synchronize()
    assert host_opt.engine.read_control().status == 0
    for a, b in zip(dev.param_chunks, host.param_chunks):
        assert bits_equal(a.shard, b.shard) and bits_equal(a.paired_chunk.shard, b.paired_chunk.shard)
    # the chunk-level norm (Chunk.set_l2_norm, elixir/chunk/core/chunk.py:218-221) also works on a shard in host
    # memory: result and scratch live on the device that runs the kernel
    for a, b in zip(dev.param_chunks, host.param_chunks):
        for chunk in (a, b):
            chunk.l2_norm = None
            chunk.set_l2_norm(chunk.shard[:chunk.valid_end])
        assert a.l2_norm == b.l2_norm
        want = float(b.shard[:b.valid_end].float().pow(2).sum())
        assert abs(b.l2_norm - want) <= 1e-5 * max(want, 1e-30)
    sa, sb = dev_opt.state_dict(), host_opt.state_dict()
    for x, y in zip(sa['shards'], sb['shards']):
        assert bits_equal(x['exp_avg'], y['exp_avg']) and bits_equal(x['exp_avg_sq'], y['exp_avg_sq'])
    got_a, got_b = dev.state_dict(), host.state_dict()
    for name in got_a:
        assert torch.equal(got_a[name], got_b[name])
    ok, ratio = close_1e6(got_b['net.0.weight'], got_a['net.0.weight'].double())
    assert ok
    # checkpoint round trip with the shards in host memory: zero everything, load it back, train on identically
    saved_model, saved_opt = host.state_dict(), host_opt.state_dict()
    host.load_state_dict({k: torch.zeros_like(v) for k, v in saved_model.items()})
    assert all(float(v.abs().max()) == 0.0 for v in host.state_dict().values())
    host.load_state_dict(saved_model)
    host_opt.load_state_dict(saved_opt)
    x = torch.randn(16, 48, device=cuda)
    la, lb = dev(x), host(x)
    assert bits_equal(la.detach(), lb.detach())
    dev_opt.backward(la)
    host_opt.backward(lb)
    dev_opt.step()
    host_opt.step()
    torch.cuda.synchronize()
    for a, b in zip(dev.param_chunks, host.param_chunks):
        assert bits_equal(a.shard, b.shard) and bits_equal(a.paired_chunk.shard, b.paired_chunk.shard)
