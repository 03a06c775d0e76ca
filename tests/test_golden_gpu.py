"""The CUDA step against fixtures produced by the reference's own ElixirOptimizer (tests/golden): every
(world, rank) trajectory is replayed on one GPU by feeding the engine the reduced gradient shards the
reference produced.  Decisions and scales bit-exact; masters within 1e-6-class tolerance of the
reference's fp32 torch.optim.AdamW results."""
import os

import pytest
import torch

from _util import bits_equal, close_1e6

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')


@pytest.mark.parametrize('world', [1, 2, 4])
def test_engine_replays_reference_trajectories(cuda, oracle, world):
    from elixir_b200 import kernels as K
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    from make_golden_constants import OPTIM_CFG, OPTIM_HYPER
    for rank, golden in enumerate(torch.load(os.path.join(GOLDEN, f'optim_w{world}.pt'))['ranks']):
        scaler = DynamicGradScaler(**{k: v for k, v in OPTIM_CFG.items()})
        engine = ChunkStepEngine(cuda, torch.float16, scaler)
        masters = []
        for init, nv in zip(golden['init_master'], golden['valid_end']):
            nv = min(nv, init.numel())
            m = init.to(cuda)
            engine.add_shard(m, torch.zeros(init.numel(), dtype=torch.float16, device=cuda), nv,
                             [(0, nv, 0)] if nv else [])
            masters.append(m)
        engine.finalize()
        engine.set_hyper([K.hyper(adamw_mode=True, **OPTIM_HYPER)])
        for s, want in enumerate(golden['steps']):
            assert engine.read_control().scale == want['scale_before']
            for c, g in enumerate(want['grad_shards']):
                engine.land(c, g.to(cuda))
            assert engine.chunk_flags.tolist()[:len(masters)] == [int(f) for f in want['chunk_overflow']]
            engine.step()
            ctl = engine.read_control()
            assert bool(ctl.skip) == any(want['chunk_overflow'])
            assert ctl.scale == want['scale_after'] and ctl.status == 0
            for c, (m, ref) in enumerate(zip(masters, want['master'])):
                ok, ratio = close_1e6(m, ref.double(), rtol=2e-6)
                assert ok, (world, rank, s, c, ratio)
                want16 = torch.empty(m.numel(), dtype=torch.float16)
                oracle.cast(m.cpu(), want16)
                assert bits_equal(engine.shards[c][3], want16)
