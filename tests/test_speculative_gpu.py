"""The out-of-place update (elx_adam_multi_shadow) and the host-buffer form of the single-pass step: same
results as the step that waits for every gradient, bit for bit, including the step in which an overflow turns
up after earlier chunks were already updated."""
import pytest
import torch

from _util import bits_equal, make_chunk

pytestmark = pytest.mark.gpu

SIZES = [3 * 4096 + 17, 8 * 4096, 4096 - 5, 40000, 16 * 4096]


def _segments():
    return [(SIZES[0] - 9, [(0, 5000, 0), (5000, SIZES[0] - 9, 1)]), (SIZES[1], [(0, SIZES[1], 0)]),
            (SIZES[2], [(3, SIZES[2], 1)]), (30000, [(0, 12345, 1), (12345, 30000, 0)]), (SIZES[4], [(0, SIZES[4], 1)])]


def _engine(cuda, dtype):
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    eng = ChunkStepEngine(cuda, dtype, DynamicGradScaler(initial_scale=64.0, growth_interval=2, hysteresis=1))
    for i, (n, (n_valid, segs)) in enumerate(zip(SIZES, _segments())):
        master, m, v, lowp = (t.to(cuda) for t in make_chunk(n, dtype, seed=70 + i))
        eng.add_shard(master, lowp, n_valid, segs, exp_avg=m, exp_avg_sq=v)
    eng.finalize()
    return eng


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_out_of_place_update_equals_in_place_and_leaves_its_input_alone(cuda, dtype):
    import elixir_b200.kernels as K
    hypers = [K.hyper(lr=1e-3, weight_decay=0.01), K.hyper(lr=3e-3, betas=(0.8, 0.95), weight_decay=0.0, adamw_mode=False)]
    a, b = _engine(cuda, dtype), _engine(cuda, dtype)
    b.enable_speculation()
    twin_table, twin_shards = b._sets[1]
    for eng in (a, b):
        eng.set_hyper(hypers)
        eng.probe()
        eng.begin_step()
    before = [[t.clone() for t in shard[:3]] for shard in b.shards]
    a.update()
    twin_table.set_hyper_from(b.table)
    K.adam_multi_shadow(b.table, twin_table, b.ctl)
    torch.cuda.synchronize()
    assert a.read_control().status == 0 and b.read_control().status == 0
    for in_place, source, kept, out in zip(a.shards, b.shards, before, twin_shards):
        for x, y in zip(source[:3], kept):
            assert bits_equal(x, y)    # the set that was read is unchanged
        for x, y in zip(in_place[:3], out[:3]):
            assert bits_equal(x, y)    # the set that was written holds what the in-place update produces
        assert bits_equal(in_place[3], source[3])    # the working copy (shared by both sets)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_speculative_host_step_equals_the_step_that_waits(cuda, dtype):
    import elixir_b200.kernels as K
    hypers = [K.hyper(lr=1e-3, weight_decay=0.01), K.hyper(lr=3e-3, betas=(0.8, 0.95), weight_decay=0.0, adamw_mode=False)]
    waits, spec = _engine(cuda, dtype), _engine(cuda, dtype)
    spec.enable_speculation()
    gen = torch.Generator().manual_seed(5)
    outs_w = [torch.empty(n, dtype=dtype).pin_memory() for n in SIZES]
    outs_s = [torch.empty(n, dtype=dtype).pin_memory() for n in SIZES]
    applied = []
    for step in range(6):
        grads = []
        for i, n in enumerate(SIZES):
            g = (torch.randn(n, generator=gen) * 1e-3 * 64).to(dtype)
            if step in (2, 4) and i == 3:
                g[111] = float('inf') if step == 2 else float('nan')    # turns up after chunks 0-2 were updated
            grads.append(g.pin_memory())
        for eng in (waits, spec):
            eng.set_hyper(hypers)
        waits.step_from_host(grads, outs_w)
        applied.append(spec.step_from_host(grads, outs_s, speculative=True))
        torch.cuda.synchronize()
        cw, cs = waits.read_control(), spec.read_control()
        assert cw.status == 0 and cs.status == 0
        for field in ('scale', 'found_inf', 'growth_step', 'hysteresis_step', 'step', 'skip', 'div_scale', 'late_inf'):
            assert getattr(cw, field) == getattr(cs, field), (step, field)
        for sw, ss, ow, os_ in zip(waits.shards, spec.current_shards(), outs_w, outs_s):
            for x, y in zip(sw[:4], ss[:4]):
                assert bits_equal(x, y), step
            assert bits_equal(ow, os_), step
    assert applied == [True, True, False, True, False, True]


def test_speculation_is_refused_where_it_cannot_hold(cuda):
    from elixir_b200.engine import ChunkStepEngine
    eng = ChunkStepEngine(cuda, torch.float16, max_norm=1.0)    # the clip factor needs every gradient first
    eng.add_shard(torch.zeros(4096, device=cuda), torch.zeros(4096, dtype=torch.float16, device=cuda), 4096, [(0, 4096, 0)])
    eng.finalize()
    with pytest.raises(RuntimeError, match='single-pass'):
        eng.enable_speculation()
