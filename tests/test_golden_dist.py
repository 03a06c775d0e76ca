"""Host-side logic against fixtures produced by the reference's own code (tests/golden/make_golden.py).

Runs on CPU: 1, 2 and 4 gloo ranks; the elx_* ABI is served by the oracle's host-memory shim, so what
is under test is this package's Python — chunk geometry, gather / reduce call sequence, probe domain,
ElixirOptimizer state machine — not the CUDA kernels (those are compared with the same oracle in the
`-m gpu` tests)."""
import pytest
import torch
import torch.multiprocessing as mp

import _dist_workers as W
from _util import free_port


@pytest.mark.parametrize('world', [1, 2, 4])
def test_chunk_geometry_gather_reduce_match_reference(world):
    mp.spawn(W.chunk_worker, args=(world, free_port()), nprocs=world)


@pytest.mark.parametrize('world', [1, 2, 4])
def test_optimizer_trajectory_matches_reference_per_rank(world):
    """sync_overflow=False reproduces the reference decision rule (each rank looks at its own shards only),
    including the ranks drifting apart after an overflow that only one rank's shard holds."""
    mp.spawn(W.optim_worker, args=(world, free_port(), False), nprocs=world)


@pytest.mark.parametrize('world', [2, 4])
def test_overflow_agreement_keeps_ranks_in_lockstep(world):
    mp.spawn(W.optim_worker, args=(world, free_port(), True), nprocs=world)


def test_oracle_replays_reference_steps(oracle):
    """The CPU oracle alone, fed the reduced gradient shards the reference produced: decisions and scales
    bit-exact, masters within 1e-6 (the reference side computed them with torch.optim.AdamW in fp32)."""
    import os
    from _util import close_1e6
    from elixir_b200 import kernels as K
    from make_golden_constants import OPTIM_CFG, OPTIM_HYPER
    for world in (1, 2, 4):
        data = torch.load(os.path.join(W.GOLDEN, f'optim_w{world}.pt'))['ranks']
        for rank, golden in enumerate(data):
            cs = oracle.ChunkSet(torch.float16)
            masters, lowps = [], []
            for init, nv in zip(golden['init_master'], golden['valid_end']):
                n = init.numel()
                nv = min(nv, n)
                m, lp = init.clone(), torch.zeros(n, dtype=torch.float16)
                cs.add_chunk(m, torch.zeros(n), torch.zeros(n), lp, nv, [(0, nv, 0)] if nv else [])
                masters.append(m)
                lowps.append(lp)
            ctl = oracle.new_ctl(OPTIM_CFG['initial_scale'])
            cfg = K.scaler_cfg(True, OPTIM_CFG['growth_factor'], OPTIM_CFG['backoff_factor'], OPTIM_CFG['min_scale'],
                               OPTIM_CFG['max_scale'], OPTIM_CFG['growth_interval'], OPTIM_CFG['hysteresis'])
            hyper = [K.hyper(adamw_mode=True, **OPTIM_HYPER)]
            for s, want in enumerate(golden['steps']):
                assert ctl.scale == want['scale_before']
                for lp, g in zip(lowps, want['grad_shards']):
                    lp.copy_(g)
                skipped = cs.step(ctl, cfg, hyper, probe=True, f64=True)
                assert skipped == any(want['chunk_overflow'])
                assert ctl.scale == want['scale_after']
                for m, ref in zip(masters, want['master']):
                    ok, ratio = close_1e6(m, ref.double(), rtol=2e-6)
                    assert ok, (world, rank, s, ratio)


def _same(a, b):
    if torch.is_tensor(a):
        return torch.is_tensor(b) and a.dtype == b.dtype and W.bits_equal(a, b)
    if isinstance(a, dict):
        return a.keys() == b.keys() and all(_same(a[k], b[k]) for k in a)
    if isinstance(a, (list, tuple)):
        return len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    return a == b


def test_committed_fixtures_are_what_the_reference_produces(tmp_path):
    """Where a checkout of hpcaitech/Elixir is at hand (ELIXIR_REFERENCE, or a directory `reference` beside
    this repository), rerun the generator and compare with the committed fixtures bit for bit."""
    import os
    import subprocess
    import sys
    ref = os.environ.get('ELIXIR_REFERENCE') or os.path.join(os.path.dirname(W.ROOT), 'reference')
    if not os.path.isdir(os.path.join(ref, 'elixir')):
        pytest.skip('no checkout of the reference')
    script = os.path.join(W.GOLDEN, 'make_golden.py')
    subprocess.run([sys.executable, script, ref, str(tmp_path)], check=True, capture_output=True, timeout=900)
    for world in (1, 2, 4):
        for kind in ('chunk', 'optim'):
            fresh = torch.load(os.path.join(str(tmp_path), f'{kind}_w{world}.pt'))
            committed = torch.load(os.path.join(W.GOLDEN, f'{kind}_w{world}.pt'))
            assert _same(fresh, committed), (kind, world)
    import json
    for name in ('scheduler.json', 'plans.json', 'states.json'):
        assert json.load(open(os.path.join(str(tmp_path), name))) == json.load(open(os.path.join(W.GOLDEN, name))), name
