"""The single-pass step (unscale + inf/nan detection + Adam/AdamW + working copy in ONE kernel, out of place
between two sets of state) against the probe-then-update step on the same inputs: same bits everywhere."""
import pytest
import torch

from _util import bits_equal

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16, torch.float32]


def _build(K, cuda, dtype, single_pass, separate_sources):
    from elixir_b200.engine import ChunkStepEngine
    from elixir_b200.scaler import DynamicGradScaler
    torch.manual_seed(0)
    eng = ChunkStepEngine(cuda, dtype, DynamicGradScaler(initial_scale=128.0, hysteresis=1, growth_interval=2))
    sizes = [300 * 4096, 5 * 4096 + 100, 4096, 3, 12 * 4096]
    valid = [300 * 4096 - 5, 5 * 4096 + 100, 1000, 0, 7 * 4096 + 1]
    # chunk 0 has a gap of whole tiles between two segments: valid, not updated, but still probed
    segs = [[(0, 100, 0), (100, 40 * 4096 + 7, 1), (90 * 4096, valid[0], 0)],
            [(0, 2 * 4096, 1), (2 * 4096, valid[1], 0)], [(0, 1000, 2)], [], [(0, 3 * 4096 + 5, 0), (3 * 4096 + 5, valid[4], 2)]]
    srcs = []
    for n, nv, sg in zip(sizes, valid, segs):
        master = (torch.randn(n) * 0.02).to(cuda)
        lowp = torch.zeros(n, dtype=dtype, device=cuda)
        src = torch.zeros(n, dtype=dtype, device=cuda) if separate_sources else None
        eng.add_shard(master, lowp, nv, sg, grad_src=src)
        srcs.append(src if src is not None else lowp)
    eng.finalize()
    eng.set_hyper([K.hyper(weight_decay=0.01), K.hyper(lr=3e-3, betas=(0.9, 0.98)), K.hyper(weight_decay=0.05, adamw_mode=False)])
    if single_pass:
        eng.enable_single_pass()
    return eng, srcs, sizes, valid


@pytest.mark.parametrize('separate_sources', [False, True])
@pytest.mark.parametrize('dtype', DTYPES)
def test_single_pass_step_equals_probe_then_update(cuda, dtype, separate_sources):
    from elixir_b200 import kernels as K
    a, a_src, sizes, valid = _build(K, cuda, dtype, False, separate_sources)
    b, b_src, _, _ = _build(K, cuda, dtype, True, separate_sources)
    # step: what goes wrong in it
    events = {2: ('inf', 0, 10), 4: ('nan in a gap between segments', 0, 60 * 4096 + 3), 5: ('pending', None, None),
              7: ('inf past valid_end (ignored)', 4, 7 * 4096 + 1), 8: ('nan in the last valid element', 1, valid[1] - 1)}
    skipped = []
    for step in range(10):
        gen = torch.Generator().manual_seed(100 + step)
        for k, n in enumerate(sizes):
            g = (torch.randn(n, generator=gen) * 1e-3 * 128).to(dtype)
            what, chunk, pos = events.get(step, (None, None, None))
            if chunk == k:
                g[pos] = float('nan') if 'nan' in what else float('inf')
            a_src[k].copy_(g)
            b_src[k].copy_(g)
        if events.get(step, ('',))[0] == 'pending':
            a.ctl.found_inf.fill_(1)
            b.ctl.found_inf.fill_(1)
        a.probe()
        a.step()
        b.step_single_pass()
        ca, cb = a.read_control(), b.read_control()
        for field in ('scale', 'growth_step', 'hysteresis_step', 'step', 'skip', 'skipped_steps', 'found_inf', 'status'):
            assert getattr(ca, field) == getattr(cb, field), (step, field)
        skipped.append(bool(cb.skip))
        assert b.chunk_flags.sum().item() == 0 and cb.spec_state == 0
        for k, (sa, sb) in enumerate(zip(a.shards, b.current_shards())):
            for x, y in zip(sa[:4], sb[:4]):
                assert bits_equal(x, y), (step, k)
    assert skipped == [s in (2, 4, 5, 8) for s in range(10)]
    assert b.read_control().status == 0


def test_single_pass_step_launched_chunk_by_chunk(cuda):
    """The update may be issued per chunk (gradients that arrive one chunk at a time): same result as one launch."""
    from elixir_b200 import kernels as K
    a, a_src, sizes, _ = _build(K, cuda, torch.float16, True, True)
    b, b_src, _, _ = _build(K, cuda, torch.float16, True, True)
    for step in range(3):
        gen = torch.Generator().manual_seed(7 + step)
        for k, n in enumerate(sizes):
            g = (torch.randn(n, generator=gen) * 1e-3 * 128).half()
            if step == 1 and k == 2:
                g[5] = float('inf')
            a_src[k].copy_(g)
            b_src[k].copy_(g)
        a.step_single_pass()
        (t0, _), (t1, _) = b._sets
        K.step_begin_optimistic(b.ctl, b.scaler.cfg, b.chunk_flags)
        for k in range(b.n_chunks):
            K.adam_multi_single_pass(t0, t1, b.ctl, b.chunk_flags, first=k, count=1)
        flags = b.chunk_flags.tolist()
        assert flags == [0, 0, int(step == 1), 0, 0]
        K.step_commit(b.ctl, b.scaler.cfg, b.chunk_flags)
        for k in range(b.n_chunks):
            K.adam_multi_repair(t0, t1, b.ctl, first=k, count=1)
        assert a.read_control().cur_set == b.read_control().cur_set
        for sa, sb in zip(a.current_shards(), b.current_shards()):
            for x, y in zip(sa[:4], sb[:4]):
                assert bits_equal(x, y), step
