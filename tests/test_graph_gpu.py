"""A whole step captured as one CUDA graph: because the overflow decision, the loss scale and the step count
never leave the device, applied and skipped steps replay from the same graph.  Compared bit for bit with the
eager step on config 1's shape (4 chunks of 4 Mi elements)."""
import pytest
import torch

from _util import bits_equal, make_chunk

pytestmark = pytest.mark.gpu


def _engine(cuda, n_chunks, n):
    import elixir_b200.kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    eng = ChunkStepEngine(cuda, torch.float16, DynamicGradScaler(initial_scale=64.0, growth_interval=2, hysteresis=1))
    for i in range(n_chunks):
        master, m, v, lowp = (t.to(cuda) for t in make_chunk(n, torch.float16, seed=90 + i))
        eng.add_shard(master, lowp, n - 100 * i, [(0, n - 100 * i, 0)], exp_avg=m, exp_avg_sq=v)
    eng.finalize()
    eng.set_hyper([K.hyper(lr=1e-3, weight_decay=0.0)])
    return eng


def test_captured_step_replays_applied_and_skipped_steps_bit_exactly(cuda):
    n_chunks, n = 4, 4 * 1024 * 1024
    eager, captured = _engine(cuda, n_chunks, n), _engine(cuda, n_chunks, n)
    blocks = [torch.zeros(n, dtype=torch.float16, device=cuda) for _ in range(n_chunks)]
    graph = captured.capture_step(blocks)
    torch.cuda.synchronize()
    for a, b in zip(eager.shards, captured.shards):    # the capture itself changed nothing
        for x, y in zip(a[:4], b[:4]):
            assert bits_equal(x, y)
    assert captured.read_control().step == 0
    gen = torch.Generator().manual_seed(17)
    for step in range(5):
        for k, block in enumerate(blocks):
            g = (torch.randn(n, generator=gen) * 1e-3 * 64).half()
            if step == 2 and k == 1:
                g[12345] = float('inf')
            block.copy_(g)
        eager.land_all(blocks, streams=1)
        eager.step()
        graph.replay()
        torch.cuda.synchronize()
        ca, cb = eager.read_control(), captured.read_control()
        assert ca.status == 0 and cb.status == 0
        fields = ('scale', 'step', 'skip', 'growth_step', 'hysteresis_step')
        assert [getattr(ca, f) for f in fields] == [getattr(cb, f) for f in fields], step
        assert bool(ca.skip) == (step == 2)
        for a, b in zip(eager.shards, captured.shards):
            for x, y in zip(a[:4], b[:4]):
                assert bits_equal(x, y), step
    assert eager.read_control().step == 4
