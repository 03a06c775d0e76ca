"""The benchmark configurations of this path as parity cases (the single-GPU ones; sharded ones:
test_sharded_gpu.py).

config 1  4 chunks x 4 194 304 elements, fp16 gradients N(0,1e-3)*64, Adam lr 1e-3 b(0.9,0.999) eps 1e-8 wd 0,
          10 steps, seed 0 — full size, every step against the CPU oracle.
config 4  overflow path: fp16 chunk set, inf/nan injected at rate 1e-6 in a random 1 of 20 steps, dynamic scale
          2^16 / backoff 0.5 / growth 2 every 1000 steps.  Full size (1 G parameters) through size-independent
          properties (bit patterns of master and moments untouched on the skipped step, working copy restored,
          decision and scale trajectory equal to the oracle's); a 16 M-parameter instance element by element,
          with hysteresis 1 and 2, and with growth interval 5 so that growth is exercised too.
"""
import pytest
import torch

from _util import bits_equal, close_1e6, lowp_within_1ulp

pytestmark = pytest.mark.gpu


def _ctl_tuple(c):
    return (c.scale, c.found_inf, c.growth_step, c.hysteresis_step, c.step, c.skip, c.div_scale, c.skipped_steps)


@pytest.mark.parametrize('single_pass', [False, True])
def test_config1_ten_steps_full_size(cuda, oracle, single_pass):
    """single_pass: the step as ONE launch that detects inf/nan itself and updates out of place between two state
    sets, reading the gradients from blocks of their own (what bench.py times on one GPU)."""
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    n_chunks, n, scale = 4, 4194304, 64.0
    hyper = [K.hyper(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)]
    engine = ChunkStepEngine(cuda, torch.float16, DynamicGradScaler(initial_scale=scale))
    host = oracle.ChunkSet(torch.float16)
    host_ctl = oracle.new_ctl(scale)
    gen = torch.Generator().manual_seed(0)
    hs, blocks = [], []
    for c in range(n_chunks):
        master = torch.randn(n, generator=gen) * 0.02
        lowp = torch.zeros(n, dtype=torch.float16)
        hm = (master.clone(), torch.zeros(n), torch.zeros(n), lowp)
        host.add_chunk(*hm, n, [(0, n, 0)])
        hs.append(hm)
        block = torch.zeros(n, dtype=torch.float16, device=cuda) if single_pass else None
        blocks.append(block)
        engine.add_shard(master.to(cuda), torch.zeros(n, dtype=torch.float16, device=cuda), n, [(0, n, 0)], grad_src=block)
    engine.finalize()
    engine.set_hyper(hyper)
    if single_pass:
        engine.enable_single_pass()
    for step in range(10):
        for c in range(n_chunks):
            g = (torch.randn(n, generator=gen) * 1e-3 * scale).half()
            hs[c][3].copy_(g)
            if single_pass:
                blocks[c].copy_(g)
            else:
                engine.land(c, g.to(cuda))
        if single_pass:
            engine.step_single_pass()
        else:
            engine.step()
        assert not host.step(host_ctl, engine.scaler.cfg, hyper, probe=True, f64=True)
        assert _ctl_tuple(engine.read_control()) == _ctl_tuple(host_ctl)
        shards = engine.current_shards()
        for c in range(n_chunks):
            for name, got, want in zip(('master', 'exp_avg', 'exp_avg_sq'), shards[c][:3], hs[c][:3]):
                ok, ratio = close_1e6(got, want.double())
                assert ok, (step, c, name, ratio)
            want16 = torch.empty(n, dtype=torch.float16)
            oracle.cast(shards[c][0].cpu(), want16)
            assert bits_equal(shards[c][3], want16)
            assert lowp_within_1ulp(shards[c][3], hs[c][3], hs[c][0])[0]
    assert engine.read_control().status == 0 and engine.read_control().step == 10


def _inject(g, gen, rate):
    """Replace elements by +inf / -inf / nan with probability `rate` (Bernoulli mask from `gen`)."""
    mask = torch.rand(g.numel(), generator=gen, device=g.device) < rate
    kinds = torch.randint(0, 3, (g.numel(),), generator=gen, device=g.device)
    vals = torch.tensor([float('inf'), -float('inf'), float('nan')], device=g.device)[kinds].to(g.dtype)
    out = torch.where(mask, vals, g)
    return out, int(mask.sum().item())


@pytest.mark.parametrize('single_pass', [False, True])
@pytest.mark.parametrize('hysteresis,growth_interval', [(1, 1000), (2, 1000), (1, 5), (2, 5)])
def test_config4_overflow_trajectory_16m_elementwise(cuda, oracle, hysteresis, growth_interval, single_pass):
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    n_chunks, n = 4, 4194304
    hyper = [K.hyper(lr=1e-3, weight_decay=0.0)]
    scaler = DynamicGradScaler(initial_scale=2.0**16, backoff_factor=0.5, growth_factor=2, growth_interval=growth_interval,
                               min_scale=1, max_scale=2**24, hysteresis=hysteresis)
    engine = ChunkStepEngine(cuda, torch.float16, scaler)
    host = oracle.ChunkSet(torch.float16)
    host_ctl = oracle.new_ctl(2.0**16)
    gen = torch.Generator().manual_seed(4)
    bad_steps = {int(torch.randint(0, 20, (1,), generator=gen)), 11, 12}    # the drawn one plus two in a row
    hs = []
    for c in range(n_chunks):
        master = torch.randn(n, generator=gen) * 0.02
        hm = (master.clone(), torch.zeros(n), torch.zeros(n), torch.zeros(n, dtype=torch.float16))
        host.add_chunk(*hm, n, [(0, n, 0)])
        hs.append(hm)
        engine.add_shard(master.to(cuda), torch.zeros(n, dtype=torch.float16, device=cuda), n, [(0, n, 0)])
    engine.finalize()
    engine.set_hyper(hyper)
    if single_pass:
        engine.enable_single_pass()
    skipped_steps = []
    for step in range(20):
        for c in range(n_chunks):
            g = (torch.randn(n, generator=gen) * 1e-3 * host_ctl.scale).half()
            if step in bad_steps:
                g, count = _inject(g, gen, 1e-6 if c else 2e-6)
            hs[c][3].copy_(g)
            if single_pass:
                engine.shards[c][3].copy_(g)    # no probe beforehand: the update kernel finds what there is to find
            else:
                engine.land(c, g.to(cuda))
        if single_pass:
            engine.step_single_pass()
        else:
            flags = engine.chunk_flags.tolist()
            assert flags == [int(oracle.probe(hs[c][3])) for c in range(n_chunks)]
            engine.step()
        skipped = host.step(host_ctl, engine.scaler.cfg, hyper, probe=True, f64=True)
        assert _ctl_tuple(engine.read_control()) == _ctl_tuple(host_ctl), step
        if skipped:
            skipped_steps.append(step)
        if step % 5 == 4 or skipped:
            shards = engine.current_shards()
            for c in range(n_chunks):
                for got, want in zip(shards[c][:3], hs[c][:3]):
                    assert close_1e6(got, want.double())[0], (step, c)
    assert set(skipped_steps) <= bad_steps and len(skipped_steps) >= 1
    assert engine.read_control().status == 0


def _bit_checksum(t):
    return int(t.view(torch.int32).to(torch.int64).sum().item())


def test_config4_overflow_trajectory_full_size_properties(cuda, oracle):
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    free, _ = torch.cuda.mem_get_info(cuda)
    n_chunks, n = 32, 33554432    # 1 073 741 824 parameters
    if free < n_chunks * n * 20:
        pytest.skip('not enough free device memory for the 1 G-parameter instance')
    hyper = [K.hyper(lr=1e-3, weight_decay=0.0)]
    scaler = DynamicGradScaler(initial_scale=2.0**16, backoff_factor=0.5, growth_factor=2, growth_interval=1000,
                               min_scale=1, max_scale=2**24, hysteresis=2)
    engine = ChunkStepEngine(cuda, torch.float16, scaler)
    host_ctl = oracle.new_ctl(2.0**16)
    dgen = torch.Generator(device=cuda).manual_seed(44)
    for c in range(n_chunks):
        master = torch.empty(n, device=cuda).normal_(0.0, 0.02, generator=dgen)
        engine.add_shard(master, torch.zeros(n, dtype=torch.float16, device=cuda), n, [(0, n, 0)])
    engine.finalize()
    engine.set_hyper(hyper)
    bad_step = int(torch.randint(0, 20, (1,), generator=torch.Generator().manual_seed(44)))
    block = torch.empty(n, dtype=torch.float16, device=cuda)
    tmp = torch.empty(n, device=cuda)
    for step in range(20):
        before = None
        if step == bad_step:
            before = [[_bit_checksum(t) for t in engine.shards[c][:3]] for c in range(n_chunks)]
        injected = 0
        for c in range(n_chunks):
            block.copy_(tmp.normal_(0.0, 1e-3, generator=dgen).mul_(host_ctl.scale))
            if step == bad_step:
                dirty, count = _inject(block, dgen, 1e-6)
                block.copy_(dirty)
                injected += count
            engine.land(c, block)
        if step == bad_step:
            assert injected > 0
            host_ctl.found_inf = 1
        assert bool(engine.read_control().found_inf) == (step == bad_step)
        engine.step()
        oracle.step_begin(host_ctl, engine.scaler.cfg)
        assert _ctl_tuple(engine.read_control()) == _ctl_tuple(host_ctl), step
        if step == bad_step:
            after = [[_bit_checksum(t) for t in engine.shards[c][:3]] for c in range(n_chunks)]
            assert after == before    # master and both moments untouched, bit for bit
        # the working copy is the rounded master after every step, skipped or not (checked with torch's cast,
        # which the oracle's cast is pinned to bit for bit)
        c = step % n_chunks
        assert torch.equal(engine.shards[c][3].view(torch.int16), engine.shards[c][0].half().view(torch.int16))
    ctl = engine.read_control()
    assert (ctl.skipped_steps, ctl.step, ctl.status) == (1, 19, 0)
    assert ctl.scale == 2.0**16    # hysteresis 2: a single overflow does not back off


def test_shard_larger_than_2_31_elements(cuda, oracle):
    """Index arithmetic past 2^31: one shard of 2^31 + 3 * 4096 + 5 elements (the OPT-66B configuration holds
    8.2 G elements per rank).  Slices at the start, around 2^31 and at the ragged tail are compared with the
    oracle element by element; everything in between through checksums of a second, identical run."""
    from elixir_b200 import kernels as K
    n = 2**31 + 3 * 4096 + 5
    free, _ = torch.cuda.mem_get_info(cuda)
    if free < n * 16:
        pytest.skip('not enough free device memory')
    n_valid = n - 3
    gen = torch.Generator(device=cuda).manual_seed(7)
    master = torch.empty(n, device=cuda).normal_(0.0, 0.02, generator=gen)
    exp_avg = torch.zeros(n, device=cuda)
    exp_avg_sq = torch.zeros(n, device=cuda)
    lowp = torch.empty(n, dtype=torch.float16, device=cuda)
    step_size = 1 << 28
    for b in range(0, n, step_size):    # gradients generated piecewise to bound temporaries
        e = min(n, b + step_size)
        lowp[b:e] = torch.empty(e - b, device=cuda).normal_(0.0, 1e-3, generator=gen).mul_(64.0).half()
    windows = [(0, 70000), (2**31 - 40000, 2**31 + 6000), (n - 5000, n)]
    assert all(0 <= b < e <= n for b, e in windows)
    before = [(master[b:e].cpu(), lowp[b:e].cpu()) for b, e in windows]
    lowp[2**31 + 77] = float('inf')
    flag = torch.zeros(1, dtype=torch.int32, device=cuda)
    K.grad_check(lowp, n_valid=n_valid, flag=flag)
    assert flag.item() == 1                      # an inf beyond index 2^31 is found
    lowp[2**31 + 77] = before[1][1][40000 + 77].item()
    flag.zero_()
    lowp[n - 2] = float('nan')                   # padding (>= n_valid): ignored
    K.grad_check(lowp, n_valid=n_valid, flag=flag)
    assert flag.item() == 0
    h = K.hyper(lr=1e-3, weight_decay=0.01)
    ctl = K.ControlBlock(cuda, 64.0)
    K.step_begin(ctl, K.scaler_cfg(False))
    K.adam_chunk(master, exp_avg, exp_avg_sq, lowp, h, ctl, n_valid=n_valid)
    c = ctl.read()
    assert c.status == 0 and c.step == 1
    for (b, e), (m0, g0) in zip(windows, before):
        hi = min(e, n_valid)
        rm, r1, r2 = m0.clone(), torch.zeros(e - b), torch.zeros(e - b)
        oracle.adam(rm, r1, r2, g0, h, 1, 64.0, 0, hi - b, f64=True)
        for got, want in ((master[b:e], rm), (exp_avg[b:e], r1), (exp_avg_sq[b:e], r2)):
            ok, ratio = close_1e6(got, want.double())
            assert ok, (b, e, ratio)
        want16 = torch.empty(e - b, dtype=torch.float16)
        oracle.cast(master[b:e].cpu(), want16)
        assert bits_equal(lowp[b:e], want16)
    assert torch.equal(master[n_valid:].cpu(), before[2][0][-3:])    # padding untouched
    # every element was updated exactly once: no moment is still zero where the gradient was not
    assert int((exp_avg_sq[:n_valid] == 0).sum().item()) < 2048


def test_gradient_clipping_by_global_norm(cuda, oracle):
    """max_norm > 0: the global L2 norm of the (still scaled) gradients feeds the combined divisor
    (elixir/wrapper/optimizer.py:149-183; dead code in the reference, live here).  Norm bit-reproducible,
    divisor and masters against the oracle."""
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    sizes = [9 * 4096 + 3, 4096, 20 * 4096]
    valid = [9 * 4096 + 3, 1000, 20 * 4096]
    scale = 1024.0
    hyper = [K.hyper(lr=1e-3, weight_decay=0.01)]
    results = []
    for attempt in range(2):
        engine = ChunkStepEngine(cuda, torch.float16, DynamicGradScaler(initial_scale=scale), max_norm=0.05)
        host = oracle.ChunkSet(torch.float16)
        host_ctl = oracle.new_ctl(scale)
        gen = torch.Generator().manual_seed(3)
        hs = []
        for n, nv in zip(sizes, valid):
            master = torch.randn(n, generator=gen) * 0.02
            hm = (master.clone(), torch.zeros(n), torch.zeros(n), torch.zeros(n, dtype=torch.float16))
            host.add_chunk(*hm, nv, [(0, nv, 0)])
            hs.append(hm)
            engine.add_shard(master.to(cuda), torch.zeros(n, dtype=torch.float16, device=cuda), nv, [(0, nv, 0)])
        engine.finalize()
        engine.set_hyper(hyper)
        for step in range(3):
            for c, n in enumerate(sizes):
                g = (torch.randn(n, generator=gen) * (1e-3 if step else 1e-5) * scale).half()
                hs[c][3].copy_(g)
                engine.land(c, g.to(cuda))
            engine.step()
            host.step(host_ctl, engine.scaler.cfg, hyper, probe=True, f64=True)
            ctl = engine.read_control()
            assert ctl.skip == 0 and ctl.status == 0
            assert abs(ctl.grad_norm - host_ctl.grad_norm) <= 1e-5 * host_ctl.grad_norm
            assert abs(ctl.div_scale - host_ctl.div_scale) <= 2e-6 * host_ctl.div_scale
            assert (ctl.clip_coef > 1.0) == (host_ctl.clip_coef > 1.0) == (step > 0)    # first step is below the threshold
            for c in range(len(sizes)):
                for got, want in zip(engine.shards[c][:3], hs[c][:3]):
                    ok, ratio = close_1e6(got, want.double(), rtol=4e-6)
                    assert ok, (step, c, ratio)
        results.append([t.cpu() for sh in engine.shards for t in sh[:3]] + [engine.total_l2sq.cpu()])
    for a, b in zip(*results):
        assert bits_equal(a, b)    # two runs, same bits: the norm reduction order is fixed
