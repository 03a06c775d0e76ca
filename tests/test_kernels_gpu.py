"""Parity of the CUDA kernels (called through the C ABI) against the CPU oracle on the same seeded inputs.

Bars: overflow flag, skip decision, scaler state and the low-precision copy of the kernel's own
master: bit-exact.  fp32 master / exp_avg / exp_avg_sq: within 1e-6 (relative to max(|x|, rms)) of
the double-precision oracle.  Low-precision working copy vs the oracle's: within 1 ulp of the format.
"""
import ctypes

import pytest
import torch

from _util import bits_equal, close_1e6, lowp_within_1ulp, make_chunk

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16, torch.float32]
SIZES = [1, 7, 8, 9, 1023, 4096, 4097, 3 * 4096 + 15, 70001, (1 << 20) + 3]


@pytest.fixture(scope='module')
def K(cuda):
    from elixir_b200 import kernels
    return kernels


def _inject(g, positions, values):
    for pos, val in zip(positions, values):
        g[pos] = val
    return g


# --------------------------------------------------------------------------------------------------
# probe
# --------------------------------------------------------------------------------------------------


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('n', SIZES)
def test_probe_clean_and_dirty(K, oracle, cuda, dtype, n):
    gen = torch.Generator().manual_seed(n)
    g = (torch.randn(n, generator=gen) * 100).to(dtype)
    cases = [('clean', [], [])]
    for name, val in (('inf', float('inf')), ('ninf', -float('inf')), ('nan', float('nan'))):
        cases.append((name + '_first', [0], [val]))
        cases.append((name + '_last', [n - 1], [val]))
        cases.append((name + '_mid', [n // 2], [val]))
    for name, pos, vals in cases:
        gc = _inject(g.clone(), pos, vals)
        want = oracle.probe(gc)
        assert want == (name != 'clean')
        flag = torch.zeros(1, dtype=torch.int32, device=cuda)
        ctl = K.ControlBlock(cuda, 1.0)
        K.grad_check(gc.to(cuda), flag=flag, ctl=ctl)
        assert bool(flag.item()) == want, (name, n, dtype)
        assert bool(ctl.read().found_inf) == want


@pytest.mark.parametrize('dtype', DTYPES)
def test_probe_respects_valid_end(K, oracle, cuda, dtype):
    n = 5 * 4096 + 100
    g = torch.ones(n, dtype=dtype)
    for n_valid in (0, 1, 4095, 4096, 4097, 3 * 4096, n - 1):
        gc = g.clone()
        gc[n_valid] = float('nan')    # first element of the padding: must not count
        flag = torch.zeros(1, dtype=torch.int32, device=cuda)
        K.grad_check(gc.to(cuda), n_valid=n_valid, flag=flag)
        assert flag.item() == 0 and not oracle.probe(gc, n_valid)
        if n_valid > 0:
            gc[n_valid - 1] = float('inf')    # last valid element: must count
            K.grad_check(gc.to(cuda), n_valid=n_valid, flag=flag)
            assert flag.item() == 1 and oracle.probe(gc, n_valid)


@pytest.mark.parametrize('dtype', DTYPES)
def test_probe_and_epilogue_on_views_off_the_vector_alignment(K, oracle, cuda, dtype):
    """A shard slice inside a replicated block starts wherever the shard size puts it: element-aligned views
    take the scalar path and give the same answers."""
    n = 3 * 4096 + 11
    gen = torch.Generator().manual_seed(17)
    base = (torch.randn(n + 5, generator=gen) * 10).to(dtype)
    for off in (1, 3, 5):
        src = base[off:off + n].clone()
        src[n - 2] = float('inf')
        block = torch.zeros(n + 8, dtype=dtype, device=cuda)
        block[off:off + n].copy_(src)
        dst_store = torch.zeros(n + 8, dtype=dtype, device=cuda)
        flag = torch.zeros(1, dtype=torch.int32, device=cuda)
        K.reduce_epilogue(block[off:off + n], dst_store[off + 2:off + 2 + n], n_valid=n - 2, flag=flag)
        assert flag.item() == 0 and bits_equal(dst_store[off + 2:off + 2 + n], src)
        K.grad_check(block[off:off + n], n_valid=n - 1, flag=flag)
        assert flag.item() == 1 and oracle.probe(src, n - 1)


def test_probe_largest_finite_values_do_not_flag(K, cuda):
    for dtype, big in ((torch.float16, 65504.0), (torch.bfloat16, 3.3895e38), (torch.float32, 3.4028e38)):
        g = torch.full((8192,), big, dtype=dtype, device=cuda)
        g[1::2] = -big
        assert torch.isfinite(g.float()).all()
        flag = torch.zeros(1, dtype=torch.int32, device=cuda)
        K.grad_check(g, flag=flag)
        assert flag.item() == 0


@pytest.mark.parametrize('dtype', DTYPES)
def test_probe_through_the_bulk_copy_ring(K, oracle, cuda, dtype):
    """The single-array probe has a second form for long arrays (a ring of bulk copies through shared memory);
    ``probe_variant=2`` sends every size there.  Sizes around its 32 KiB stage, 16-byte piece and ring length, an
    inf/nan at every kind of position, ``n_valid`` cutting the array, and the same answers as the loads form."""
    size = torch.empty(0, dtype=dtype).element_size()
    per_stage = 32768 // size
    sizes = [1, 7, 8, 9, per_stage - 1, per_stage, per_stage + 1, 6 * per_stage, 6 * per_stage + 3,
             148 * 6 * per_stage + 5 * per_stage + 11, 148 * 13 * per_stage - 1]
    K.set_tuning(probe_variant=2)
    try:
        for n in sizes:
            g = torch.ones(n, dtype=dtype, device=cuda)
            flag = torch.zeros(1, dtype=torch.int32, device=cuda)
            ctl = K.ControlBlock(cuda, 1.0)
            K.grad_check(g, flag=flag, ctl=ctl)
            assert flag.item() == 0 and ctl.read().found_inf == 0 and ctl.read().status == 0, n
            spots = sorted({0, n - 1, n // 2, max(0, n - 8), max(0, n - 9), min(n - 1, per_stage), min(n - 1, per_stage - 1)})
            for pos in spots:
                for val in (float('inf'), float('nan')):
                    g[pos] = val
                    flag.zero_()
                    K.grad_check(g, flag=flag)
                    assert flag.item() == 1, (n, pos, val)
                    # the same array cut just before the bad element is clean
                    flag.zero_()
                    K.grad_check(g, n_valid=pos, flag=flag)
                    assert flag.item() == 0, (n, pos, 'cut')
                    g[pos] = 1.0
        # a view that starts off the 16-byte boundary goes to the loads form and gives the same answer
        g = torch.ones(3 * per_stage + 9, dtype=dtype, device=cuda)
        g[-1] = float('-inf')
        flag = torch.zeros(1, dtype=torch.int32, device=cuda)
        K.grad_check(g[1:], flag=flag)
        assert flag.item() == 1
        # random data against the oracle and against the loads form
        gen = torch.Generator().manual_seed(5)
        h = (torch.randn(5 * per_stage + 123, generator=gen) * 1e4).to(dtype)
        want = oracle.probe(h)
        hd = h.to(cuda)
        got = []
        for variant in (2, 0):
            K.set_tuning(probe_variant=variant)
            flag.zero_()
            K.grad_check(hd, flag=flag)
            got.append(bool(flag.item()))
        assert got == [want, want]
    finally:
        K.set_tuning(probe_variant=-1)


def test_probe_of_a_long_array_takes_the_ring_by_default(K, cuda):
    """From 16 MiB on the ring is the default form: same answers on a 96 MiB array."""
    n = 48 * (1 << 20) + 5
    g = torch.zeros(n, dtype=torch.float16, device=cuda)
    flag = torch.zeros(1, dtype=torch.int32, device=cuda)
    K.grad_check(g, flag=flag)
    assert flag.item() == 0
    for pos in (0, n // 3, n - 1):
        g[pos] = float('nan')
        flag.zero_()
        K.grad_check(g, flag=flag)
        assert flag.item() == 1, pos
        g[pos] = 0


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('n', [1, 4095, 4096, 70001, (1 << 22) + 17])
def test_probe_l2_norm(K, oracle, cuda, dtype, n):
    gen = torch.Generator().manual_seed(n + 1)
    g = (torch.randn(n, generator=gen) * 3).to(dtype)
    n_valid = max(0, n - 5)
    want = oracle.l2sq(g, n_valid)
    gd = g.to(cuda)
    out = torch.full((1,), -1.0, device=cuda)
    scratch = torch.empty(K.n_tiles(n), device=cuda)
    K.grad_check(gd, n_valid=n_valid, l2sq=out, scratch=scratch)
    got = out.item()
    assert abs(got - want) <= 1e-5 * max(want, 1e-30), (got, want)
    # bit-reproducible, also under another grid size
    K.set_tuning(probe_ctas_per_sm=1)
    try:
        out2 = torch.full((1,), -1.0, device=cuda)
        K.grad_check(gd, n_valid=n_valid, l2sq=out2, scratch=scratch)
    finally:
        K.set_tuning(probe_ctas_per_sm=-1)
    assert bits_equal(out, out2)


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('n,n_valid', [(1, 1), (4096, 4096), (4097, 100), (70001, 69000), (1 << 20, 0), ((1 << 20) + 8, 1 << 19)])
def test_reduce_epilogue_copy_and_probe(K, oracle, cuda, dtype, n, n_valid):
    gen = torch.Generator().manual_seed(n)
    src = (torch.randn(n, generator=gen) * 10).to(dtype)
    for dirty in (False, True):
        s = src.clone()
        if dirty and n_valid > 0:
            s[n_valid - 1] = float('inf')
        if n_valid < n:
            s[n_valid] = float('nan')    # padding is copied but never probed
        dst = torch.zeros(n, dtype=dtype, device=cuda)
        flag = torch.zeros(1, dtype=torch.int32, device=cuda)
        K.reduce_epilogue(s.to(cuda), dst, n_valid=n_valid, flag=flag)
        assert bits_equal(dst, s)
        assert bool(flag.item()) == oracle.probe(s, n_valid) == (dirty and n_valid > 0)


# --------------------------------------------------------------------------------------------------
# control block: decision + loss scaler
# --------------------------------------------------------------------------------------------------


def _ctl_fields(c):
    return (c.scale, c.found_inf, c.growth_step, c.hysteresis_step, c.step, c.skip, c.div_scale, c.inv_div,
            c.skipped_steps)


@pytest.mark.parametrize('hysteresis', [1, 2, 3])
@pytest.mark.parametrize('initial', [65536.0, 1.0, 3.0])
def test_scaler_trajectory_bit_exact(K, oracle, cuda, hysteresis, initial):
    cfg = K.scaler_cfg(True, 2.0, 0.5, 1.0, 2.0**24, growth_interval=5, hysteresis=hysteresis)
    gen = torch.Generator().manual_seed(hysteresis * 100 + int(initial))
    pattern = (torch.rand(400, generator=gen) < 0.15).tolist()
    dev = K.ControlBlock(cuda, initial)
    host = oracle.new_ctl(initial)
    for found in pattern:
        if found:
            dev.found_inf.fill_(1)
            host.found_inf = 1
        K.step_begin(dev, cfg)
        oracle.step_begin(host, cfg)
        assert _ctl_fields(dev.read()) == _ctl_fields(host)
    assert host.skipped_steps == sum(pattern)


def test_constant_scaler_and_clip(K, oracle, cuda):
    cfg = K.scaler_cfg(False, max_norm=1.0)
    dev = K.ControlBlock(cuda, 1.0)
    host = oracle.new_ctl(1.0)
    for norm_sq in (0.25, 4.0, 1.0, 123.456):
        ns = torch.tensor([norm_sq], device=cuda)
        K.step_begin(dev, cfg, ns)
        oracle.step_begin(host, cfg, norm_sq)
        d = dev.read()
        assert _ctl_fields(d) == _ctl_fields(host)
        assert (d.clip_coef, d.grad_norm) == (host.clip_coef, host.grad_norm)
    # scale 1 and no clipping: the divisor is the -1 sentinel
    K.step_begin(dev, K.scaler_cfg(False))
    assert dev.read().div_scale == -1.0


# --------------------------------------------------------------------------------------------------
# fused Adam, single shard
# --------------------------------------------------------------------------------------------------

HYPERS = [
    dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adamw_mode=True),
    dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, adamw_mode=True),
    dict(lr=1e-3, betas=(0.8, 0.95), eps=1e-8, weight_decay=0.1, adamw_mode=False),
    dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adamw_mode=True, bias_correction=False),
]


def _run_single(K, oracle, cuda, n, dtype, hyper_kw, scale, steps, n_valid=None, math_mode=1):
    n_valid = n if n_valid is None else n_valid
    h = K.hyper(**hyper_kw)
    cfg = K.scaler_cfg(False)
    p, m, v, g = make_chunk(n, dtype, seed=n + steps, scale=scale)
    dp, dm, dv = p.to(cuda), m.to(cuda), v.to(cuda)
    ref = [t.clone() for t in (p, m, v)]
    f32 = [t.clone() for t in (p, m, v)]
    dev_ctl = K.ControlBlock(cuda, scale)
    host_ctl = oracle.new_ctl(scale)
    K.set_tuning(math_mode=math_mode)
    try:
        for s in range(steps):
            gen = torch.Generator().manual_seed(1000 * s + n)
            g = (torch.randn(n, generator=gen) * 1e-3 * scale).to(dtype)
            dg = g.to(cuda)
            K.step_begin(dev_ctl, cfg)
            oracle.step_begin(host_ctl, cfg)
            K.adam_chunk(dp, dm, dv, dg, h, dev_ctl, n_valid=n_valid)
            oracle.adam(ref[0], ref[1], ref[2], g, h, host_ctl.step, host_ctl.div_scale, 0, n_valid, f64=True)
            oracle.adam(f32[0], f32[1], f32[2], g, h, host_ctl.step, host_ctl.div_scale, 0, n_valid, f64=False)
    finally:
        K.set_tuning(math_mode=-1)
    return (dp, dm, dv, dg), ref, f32, dev_ctl


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('n', SIZES)
def test_adam_chunk_sizes(K, oracle, cuda, dtype, n):
    (dp, dm, dv, dg), ref, _, ctl = _run_single(K, oracle, cuda, n, dtype, HYPERS[1], 64.0, steps=2)
    for name, got, want in (('master', dp, ref[0]), ('exp_avg', dm, ref[1]), ('exp_avg_sq', dv, ref[2])):
        ok, ratio = close_1e6(got, want)
        assert ok, (name, n, dtype, ratio)
    # the working copy is the kernel's own master rounded to nearest even: bit-exact
    want16 = torch.empty(n, dtype=dtype)
    oracle.cast(dp.cpu(), want16)
    assert bits_equal(dg, want16)
    if dtype != torch.float32:
        ref16 = torch.empty(n, dtype=dtype)
        oracle.cast(ref[0], ref16)
        assert lowp_within_1ulp(dg, ref16, ref[0])[0]
    assert ctl.read().status == 0 and ctl.read().late_inf == 0


@pytest.mark.parametrize('math_mode', [1, 2])
@pytest.mark.parametrize('hyper_kw', HYPERS)
@pytest.mark.parametrize('scale', [1.0, 64.0, 65536.0, 3.7])
def test_adam_chunk_hypers_scales(K, oracle, cuda, hyper_kw, scale, math_mode):
    n = 5 * 4096 + 77
    (dp, dm, dv, dg), ref, f32, ctl = _run_single(K, oracle, cuda, n, torch.float16, hyper_kw, scale, steps=3,
                                                  math_mode=math_mode)
    for name, got, want in (('master', dp, ref[0]), ('exp_avg', dm, ref[1]), ('exp_avg_sq', dv, ref[2])):
        ok, ratio = close_1e6(got, want)
        assert ok, (name, hyper_kw, scale, ratio)
    want_div = -1.0 if scale == 1.0 else scale
    assert abs(ctl.read().div_scale - want_div) < 1e-6 * abs(want_div)


def test_adam_chunk_ill_conditioned_update_no_worse_than_strict_fp32(K, oracle, cuda):
    """With a large lr and eps, elements whose effective gradient is of the order of eps amplify fp32
    rounding beyond 1e-6 in ANY fp32 evaluation.  There the kernel must stay within a small multiple
    of the error the strict-fp32 oracle itself makes against the double-precision one."""
    hyper_kw = dict(lr=3e-2, betas=(0.8, 0.95), eps=1e-6, weight_decay=0.1, adamw_mode=False)
    n = 5 * 4096 + 77
    (dp, dm, dv, dg), ref, f32, _ = _run_single(K, oracle, cuda, n, torch.float16, hyper_kw, 1.0, steps=3)
    for got, want64, want32 in zip((dp, dm, dv), ref, f32):
        err_gpu = (got.cpu().double() - want64.double()).abs()
        err_f32 = (want32.double() - want64.double()).abs()
        rms = want64.double().pow(2).mean().sqrt()
        bound = 1e-6 * torch.maximum(want64.double().abs(), rms.expand_as(err_gpu))
        bad = err_gpu > bound
        assert bad.double().mean().item() < 0.02
        assert (err_gpu[bad] <= 8 * err_f32[bad] + bound[bad]).all()


@pytest.mark.parametrize('hyper_kw', [HYPERS[0], HYPERS[-1], dict(lr=1e-3, betas=(0.9, 0.999), eps=0.0, weight_decay=0.0)])
def test_adam_elements_whose_state_and_gradient_are_zero(K, oracle, cuda, hyper_kw):
    """Exact zeros (+0 and -0) in gradient and moments take a short cut around the IEEE division and square root
    (whose zero operands cost a slow path): the results must be what the plain operations give -- zero moments stay
    zero, everything within the tolerance of the double-precision oracle, and with eps = 0 the
    0 / 0 of such an element is the NaN it is in the reference arithmetic."""
    n = 3 * 4096 + 50
    gen = torch.Generator().manual_seed(11)
    p = torch.randn(n, generator=gen) * 0.05
    m = torch.randn(n, generator=gen) * 1e-3
    v = torch.rand(n, generator=gen) * 1e-6
    g = (torch.randn(n, generator=gen) * 1e-3).to(torch.float16)
    mask = torch.rand(n, generator=gen) < 0.5
    neg = mask & (torch.rand(n, generator=gen) < 0.3)
    m[mask], v[mask], g[mask] = 0.0, 0.0, 0.0
    m[neg] = -0.0
    g[neg] = -0.0
    h = K.hyper(**hyper_kw)
    cfg = K.scaler_cfg(False)
    dp, dm, dv, dg = (t.to(cuda) for t in (p, m, v, g))
    ref = [t.clone() for t in (p, m, v)]
    f32 = [t.clone() for t in (p, m, v)]
    dev_ctl, host_ctl = K.ControlBlock(cuda, 1.0), oracle.new_ctl(1.0)
    # with eps = 0 the zero elements turn into NaN in the first step (and everything they touch in the second)
    for _ in range(1 if hyper_kw['eps'] == 0.0 else 2):
        K.step_begin(dev_ctl, cfg)
        oracle.step_begin(host_ctl, cfg)
        K.adam_chunk(dp, dm, dv, dg.clone(), h, dev_ctl)
        oracle.adam(ref[0], ref[1], ref[2], g, h, host_ctl.step, host_ctl.div_scale, f64=True)
        oracle.adam(f32[0], f32[1], f32[2], g, h, host_ctl.step, host_ctl.div_scale, f64=False)
    got_p, got_m, got_v = dp.cpu(), dm.cpu(), dv.cpu()
    # zero moments stay exact zeros, as in the strict fp32 evaluation
    assert (got_m[mask] == 0).all() and (got_v[mask] == 0).all()
    assert (f32[1][mask] == 0).all() and (f32[2][mask] == 0).all()
    if hyper_kw['eps'] == 0.0:
        # 0 / (sqrt(0) + 0): NaN in the reference arithmetic, NaN here
        assert torch.isnan(got_p[mask]).all() and torch.isnan(f32[0][mask]).all()
        keep = ~mask
    else:
        keep = torch.ones(n, dtype=torch.bool)
    for name, got, want in (('master', got_p, ref[0]), ('exp_avg', got_m, ref[1]), ('exp_avg_sq', got_v, ref[2])):
        ok, ratio = close_1e6(got[keep], want[keep])
        assert ok, (name, ratio)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_adam_chunk_padding_is_only_refreshed(K, oracle, cuda, dtype):
    n, n_valid = 6 * 4096, 2 * 4096 + 33
    h = K.hyper(weight_decay=0.01)
    p, m, v, g = make_chunk(n, dtype, seed=5)
    m += 0.5
    v += 0.25
    dp, dm, dv, dg = (t.to(cuda) for t in (p, m, v, g))
    ctl = K.ControlBlock(cuda, 64.0)
    K.step_begin(ctl, K.scaler_cfg(False))
    K.adam_chunk(dp, dm, dv, dg, h, ctl, n_valid=n_valid)
    assert bits_equal(dp[n_valid:], p[n_valid:])
    assert bits_equal(dm[n_valid:], m[n_valid:])
    assert bits_equal(dv[n_valid:], v[n_valid:])
    want16 = torch.empty(n, dtype=dtype)
    oracle.cast(dp.cpu(), want16)
    assert bits_equal(dg, want16)
    assert not bits_equal(dp[:n_valid], p[:n_valid])


def test_adam_chunk_unaligned_views(K, oracle, cuda):
    """Views that start off a 32-byte boundary take the scalar path and still match."""
    n = 3 * 4096 + 5
    h = K.hyper(weight_decay=0.01)
    p, m, v, g = make_chunk(n + 3, torch.float16, seed=9)
    dp, dm, dv, dg = (t.to(cuda) for t in (p, m, v, g))
    ctl = K.ControlBlock(cuda, 64.0)
    host = oracle.new_ctl(64.0)
    K.step_begin(ctl, K.scaler_cfg(False))
    oracle.step_begin(host, K.scaler_cfg(False))
    K.adam_chunk(dp[3:], dm[3:], dv[3:], dg[3:], h, ctl)
    rp, rm, rv = p[3:].clone(), m[3:].clone(), v[3:].clone()
    oracle.adam(rp, rm, rv, g[3:].clone(), h, host.step, host.div_scale, f64=True)
    for got, want in ((dp[3:], rp), (dm[3:], rm), (dv[3:], rv)):
        assert close_1e6(got, want)[0]
    assert bits_equal(dp[:3], p[:3]) and bits_equal(dg[:3], g[:3])


@pytest.mark.parametrize('mode', ['adamw', 'l2'])
def test_adam_against_torch_fused_optimizer_on_the_gpu(K, cuda, mode):
    """A second, independent GPU implementation: torch's fused multi-tensor Adam/AdamW (the Apex lineage the
    reference's ColossalAI kernel also comes from), fed the unscaled fp32 gradients.  Dyadic betas keep
    (1 - beta) exact in either precision, so only rounding order differs."""
    n, scale, steps = 6 * 4096 + 123, 128.0, 4
    betas, lr, eps, wd = (0.875, 0.99609375), 0.0009765625, 1e-8, 0.0078125
    p, m, v, _ = make_chunk(n, torch.float16, seed=21)
    dp, dm, dv = p.to(cuda), m.to(cuda), v.to(cuda)
    ref = torch.nn.Parameter(p.to(cuda).clone())
    Opt = torch.optim.AdamW if mode == 'adamw' else torch.optim.Adam
    opt = Opt([ref], lr=lr, betas=betas, eps=eps, weight_decay=wd, fused=True)
    h = K.hyper(lr, betas, eps, wd, adamw_mode=(mode == 'adamw'))
    ctl = K.ControlBlock(cuda, scale)
    for s in range(steps):
        gen = torch.Generator().manual_seed(500 + s)
        g16 = (torch.randn(n, generator=gen) * 1e-3 * scale).half().to(cuda)
        ref.grad = g16.float() / scale
        opt.step()
        K.step_begin(ctl, K.scaler_cfg(False))
        K.adam_chunk(dp, dm, dv, g16, h, ctl)
    state = opt.state[ref]
    for name, got, want in (('master', dp, ref.data), ('exp_avg', dm, state['exp_avg']),
                            ('exp_avg_sq', dv, state['exp_avg_sq'])):
        ok, ratio = close_1e6(got, want.double(), rtol=2e-6)
        assert ok, (mode, name, ratio)


def test_skip_leaves_state_untouched_and_restores_params(K, oracle, cuda):
    n = 4 * 4096 + 9
    p, m, v, g = make_chunk(n, torch.float16, seed=11, scale=65536.0)
    m += 0.125
    g[n // 3] = float('inf')
    dp, dm, dv, dg = (t.to(cuda) for t in (p, m, v, g))
    ctl = K.ControlBlock(cuda, 65536.0)
    cfg = K.scaler_cfg(True, hysteresis=1)
    K.grad_check(dg, ctl=ctl)
    K.step_begin(ctl, cfg)
    K.adam_chunk(dp, dm, dv, dg, K.hyper(), ctl)
    c = ctl.read()
    assert (c.skip, c.step, c.scale, c.skipped_steps, c.found_inf) == (1, 0, 32768.0, 1, 0)
    assert bits_equal(dp, p) and bits_equal(dm, m) and bits_equal(dv, v)
    want16 = torch.empty(n, dtype=torch.float16)
    oracle.cast(p, want16)
    assert bits_equal(dg, want16)


def test_late_inf_is_reported(K, cuda):
    """A non-finite gradient on an applied step (probe not run) raises the sticky status bit."""
    n = 2 * 4096
    p, m, v, g = make_chunk(n, torch.float16, seed=13)
    g[17] = float('nan')
    dp, dm, dv, dg = (t.to(cuda) for t in (p, m, v, g))
    ctl = K.ControlBlock(cuda, 64.0)
    K.step_begin(ctl, K.scaler_cfg(False))
    K.adam_chunk(dp, dm, dv, dg, K.hyper(), ctl)
    c = ctl.read()
    assert c.late_inf == 1 and c.status & 1


def test_cast_copyback(K, oracle, cuda):
    for dtype in DTYPES:
        for n in (1, 4095, 4096, 70001):
            gen = torch.Generator().manual_seed(n)
            src = torch.randn(n, generator=gen) * torch.logspace(-8, 5, n)
            dst = torch.empty(n, dtype=dtype, device=cuda)
            K.cast_copyback(src.to(cuda), dst)
            want = torch.empty(n, dtype=dtype)
            oracle.cast(src, want)
            assert bits_equal(dst, want)


# --------------------------------------------------------------------------------------------------
# multi-chunk launches
# --------------------------------------------------------------------------------------------------


def _build_set(K, oracle, cuda, dtype, sizes, valid, seg_lists, seed, scale):
    table = K.ChunkTable(cuda, dtype)
    host = oracle.ChunkSet(dtype)
    dev_tensors, host_tensors = [], []
    for c, (n, nv, segs) in enumerate(zip(sizes, valid, seg_lists)):
        p, m, v, g = make_chunk(n, dtype, seed=seed + c, scale=scale)
        dts = tuple(t.to(cuda) for t in (p, m, v, g))
        table.add_chunk(*dts, n_valid=nv, segments=segs)
        host.add_chunk(p, m, v, g, nv, segs)
        dev_tensors.append(dts)
        host_tensors.append((p, m, v, g))
    table.finalize()
    return table, host, dev_tensors, host_tensors


def _segments(n_valid, cuts, groups):
    """Split [0, n_valid) at `cuts`; groups[i] < 0 leaves the piece uncovered."""
    edges = [0] + [c for c in cuts if 0 < c < n_valid] + [n_valid]
    out = []
    for i in range(len(edges) - 1):
        grp = groups[i % len(groups)]
        if grp >= 0 and edges[i] < edges[i + 1]:
            out.append((edges[i], edges[i + 1], grp))
    return out


@pytest.mark.parametrize('dtype', DTYPES)
def test_table_probe_through_the_bulk_copy_ring(K, oracle, cuda, dtype):
    """``elx_grad_check_multi`` without a norm has the ring form too (``probe_variant=2`` forces it at every size).
    Chunks whose tiles share stages with their neighbours, ragged tails, ``valid_end`` inside a tile, an empty
    chunk, a gradient source of its own that is off the 16-byte boundary: the per-chunk words and the control
    block's word must say the same as the oracle's probe of every chunk, for an inf/nan at any kind of position,
    and the same as the loads form."""
    sizes = [9 * 4096, 5 * 4096 + 100, 4096, 3, 12 * 4096 + 7, 40 * 4096]
    valid = [9 * 4096, 5 * 4096 + 100, 1000, 0, 7 * 4096 + 1, 40 * 4096 - 3]
    table = K.ChunkTable(cuda, dtype)
    grads = []
    for c, (n, nv) in enumerate(zip(sizes, valid)):
        p, m, v, g = make_chunk(n, dtype, seed=300 + c, scale=4.0)
        dts = [t.to(cuda) for t in (p, m, v, g)]
        kw = {}
        if c == 4:    # gradients in a block of their own, starting one element off the vector alignment
            store = torch.ones(n + 8, dtype=dtype, device=cuda)
            kw['grad_src'] = store[1:n + 1]
            dts.append(store)
        table.add_chunk(dts[0], dts[1], dts[2], dts[3], n_valid=nv, segments=[(0, nv, 0)] if nv else [], **kw)
        grads.append(kw.get('grad_src', dts[3]))
    table.finalize()
    flags = torch.zeros(table.n_chunks, dtype=torch.int32, device=cuda)

    def probe(variant):
        K.set_tuning(probe_variant=variant)
        try:
            flags.zero_()
            ctl = K.ControlBlock(cuda, 1.0)
            K.grad_check_multi(table, ctl, chunk_flags=flags)
            c = ctl.read()
            assert c.status == 0
            return flags.tolist(), int(c.found_inf)
        finally:
            K.set_tuning(probe_variant=-1)

    for g in grads:
        g.fill_(1.0)
    assert probe(2) == ([0] * len(sizes), 0)
    for c, nv in enumerate(valid):
        spots = sorted({p for p in (0, nv - 1, nv // 2, nv - 8, nv - 9, 4095, 4096, 4 * 4096 - 1, 4 * 4096) if 0 <= p < nv})
        for pos in spots:
            for val in (float('inf'), float('nan')):
                grads[c][pos] = val
                want = ([int(i == c) for i in range(len(sizes))], 1)
                assert oracle.probe(grads[c].cpu(), nv)
                assert probe(2) == want, (c, pos, val)
                assert probe(0) == want
                grads[c][pos] = 1.0
        if nv < sizes[c]:    # the first element past valid_end does not count
            grads[c][nv] = float('nan')
            assert probe(2) == ([0] * len(sizes), 0), c
            grads[c][nv] = 1.0
    # a sub-range of the table
    grads[1][7] = float('inf')
    grads[5][11] = float('inf')
    K.set_tuning(probe_variant=2)
    try:
        flags.zero_()
        ctl = K.ControlBlock(cuda, 1.0)
        K.grad_check_multi(table, ctl, chunk_flags=flags, first=2, count=3)
        assert flags.tolist() == [0] * len(sizes) and ctl.read().found_inf == 0
        K.grad_check_multi(table, ctl, chunk_flags=flags, first=1, count=5)
        assert flags.tolist() == [0, 1, 0, 0, 0, 1] and ctl.read().found_inf == 1
    finally:
        K.set_tuning(probe_variant=-1)


@pytest.mark.parametrize('dtype', DTYPES)
def test_adam_multi_segments_and_groups(K, oracle, cuda, dtype):
    sizes = [8 * 4096, 5 * 4096 + 100, 4096, 3, 12 * 4096]
    valid = [8 * 4096, 5 * 4096 + 100, 1000, 0, 7 * 4096 + 1]
    seg_lists = [
        _segments(valid[0], [100, 4096, 4096 + 7, 3 * 4096, 5 * 4096 + 2048], [0, 1, 2, -1, 0, 1]),
        _segments(valid[1], [2 * 4096], [1, 0]),
        _segments(valid[2], [], [2]),
        [],
        _segments(valid[4], [3 * 4096 + 5], [0, 2]),
    ]
    hypers = [
        K.hyper(1e-3, (0.9, 0.999), 1e-8, 0.01, True),
        K.hyper(5e-4, (0.9, 0.98), 1e-6, 0.0, True),
        K.hyper(2e-3, (0.85, 0.99), 1e-8, 0.05, False),
    ]
    scale = 1024.0
    table, host, dev_t, host_t = _build_set(K, oracle, cuda, dtype, sizes, valid, seg_lists, 77, scale)
    table.set_hyper(hypers)
    cfg = K.scaler_cfg(True, growth_interval=2, hysteresis=1)
    dev_ctl = K.ControlBlock(cuda, scale)
    host_ctl = oracle.new_ctl(scale)
    flags = torch.zeros(table.n_chunks, dtype=torch.int32, device=cuda)
    for step in range(4):
        for c, n in enumerate(sizes):
            gen = torch.Generator().manual_seed(31 * step + c)
            g = (torch.randn(n, generator=gen) * 1e-3 * host_ctl.scale).to(dtype)
            if step == 2 and c == 1:
                g[valid[c] - 1] = float('inf')
            host_t[c][3].copy_(g)
            dev_t[c][3].copy_(g)
        flags.zero_()
        K.grad_check_multi(table, dev_ctl, chunk_flags=flags)
        K.step_begin(dev_ctl, cfg)
        K.adam_multi(table, dev_ctl)
        skipped = host.step(host_ctl, cfg, hypers, probe=True, f64=True)
        assert skipped == (step == 2)
        assert flags.tolist() == [int(step == 2 and c == 1) for c in range(len(sizes))]
        assert _ctl_fields(dev_ctl.read()) == _ctl_fields(host_ctl)
        for c in range(len(sizes)):
            for name, got, want in zip(('master', 'exp_avg', 'exp_avg_sq'), dev_t[c][:3], host_t[c][:3]):
                ok, ratio = close_1e6(got, want)
                assert ok, (step, c, name, ratio)
            want16 = torch.empty(sizes[c], dtype=dtype)
            oracle.cast(dev_t[c][0].cpu(), want16)
            assert bits_equal(dev_t[c][3], want16), (step, c)
            if dtype != torch.float32:
                assert lowp_within_1ulp(dev_t[c][3], host_t[c][3], host_t[c][0])[0]
    assert dev_ctl.read().status == 0


def test_adam_multi_sub_ranges_equal_one_launch(K, oracle, cuda):
    """Launching chunk by chunk (as the sharded pipeline does) gives the same bits as one launch."""
    sizes = [4 * 4096, 4096 + 5, 9 * 4096]
    segs = [[(0, n, 0)] for n in sizes]
    hypers = [K.hyper(weight_decay=0.01)]
    results = []
    for per_chunk in (False, True):
        table, _, dev_t, _ = _build_set(K, oracle, cuda, torch.float16, sizes, sizes, segs, 5, 64.0)
        table.set_hyper(hypers)
        ctl = K.ControlBlock(cuda, 64.0)
        K.step_begin(ctl, K.scaler_cfg(False))
        if per_chunk:
            for c in range(len(sizes)):
                K.adam_multi(table, ctl, first=c, count=1)
        else:
            K.adam_multi(table, ctl)
        results.append([[t.cpu() for t in ts] for ts in dev_t])
    for a, b in zip(*results):
        for x, y in zip(a, b):
            assert bits_equal(x, y)


@pytest.mark.parametrize('threads,ctas', [(256, 1), (256, 3), (512, 2), (512, 4)])
def test_launch_shapes_give_identical_bits(K, oracle, cuda, threads, ctas):
    sizes = [16 * 4096, 4096 + 5]
    segs = [[(0, n, 0)] for n in sizes]
    hypers = [K.hyper(weight_decay=0.01)]

    def run():
        table, _, dev_t, _ = _build_set(K, oracle, cuda, torch.float16, sizes, sizes, segs, 3, 64.0)
        table.set_hyper(hypers)
        ctl = K.ControlBlock(cuda, 64.0)
        K.step_begin(ctl, K.scaler_cfg(False))
        K.adam_multi(table, ctl)
        return [[t.cpu() for t in ts] for ts in dev_t]

    base = run()
    K.set_tuning(adam_variant=0, adam_threads=threads, adam_ctas_per_sm=ctas)
    try:
        other = run()
    finally:
        K.set_tuning(adam_variant=-1, adam_threads=-1, adam_ctas_per_sm=-1)
    for a, b in zip(base, other):
        for x, y in zip(a, b):
            assert bits_equal(x, y)


@pytest.mark.parametrize('dtype', DTYPES)
def test_bulk_copy_pipeline_variant_is_bit_identical_to_direct(K, oracle, cuda, dtype):
    """adam_variant=1 stages tiles through shared memory with cp.async.bulk; the arithmetic is shared, so
    applied and skipped steps must give the same bits, over many tiles per CTA, ragged tiles and groups."""
    sizes = [700 * 4096, 5 * 4096 + 100, 4096, 3, 12 * 4096]
    valid = [700 * 4096 - 5, 5 * 4096 + 100, 1000, 0, 7 * 4096 + 1]
    seg_lists = [
        _segments(valid[0], [100, 4096, 4096 + 7, 300 * 4096, 500 * 4096 + 2048], [0, 1, 2, -1, 0, 1]),
        _segments(valid[1], [2 * 4096], [1, 0]),
        _segments(valid[2], [], [2]),
        [],
        _segments(valid[4], [3 * 4096 + 5], [0, 2]),
    ]
    hypers = [K.hyper(1e-3, (0.9, 0.999), 1e-8, 0.01, True), K.hyper(5e-4, (0.9, 0.98), 1e-6, 0.0, True),
              K.hyper(2e-3, (0.85, 0.99), 1e-8, 0.05, False)]
    outs = []
    # direct accesses; the ring at its default depth (four stages for 16-bit chunks); the ring with three stages
    for variant, stages in ((0, -1), (1, -1), (1, 3)):
        K.set_tuning(adam_variant=variant, adam_tma_stages=stages)
        try:
            table, _, dev_t, _ = _build_set(K, oracle, cuda, dtype, sizes, valid, seg_lists, 21, 512.0)
            table.set_hyper(hypers)
            ctl = K.ControlBlock(cuda, 512.0)
            cfg = K.scaler_cfg(True, hysteresis=1)
            for step in range(3):
                if step == 1:
                    ctl.found_inf.fill_(1)    # a skipped step in the middle
                K.step_begin(ctl, cfg)
                K.adam_multi(table, ctl)
                for ts in dev_t:    # next step's "gradients": something deterministic and finite
                    ts[3].copy_((ts[0] * 37.0).to(dtype))
            torch.cuda.synchronize()
            assert ctl.read().status == 0
            outs.append([[t.cpu() for t in ts] for ts in dev_t])
        finally:
            K.set_tuning(adam_variant=-1, adam_tma_stages=-1)
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            for x, y in zip(a, b):
                assert bits_equal(x, y)


def test_peer_barrier_wait_is_bounded(K, cuda):
    """A peer that never arrives: the barrier kernel gives up after its time limit, raises the sticky
    ELX_STAT_TIMEOUT bit and returns; the context stays usable.  The "missing peer" is a second flag region
    on the same GPU that nothing ever writes an epoch into — no other process, nothing hangs."""
    import time
    from elixir_b200 import _abi, _lib
    lib = _lib.get()
    mine = torch.zeros(256, dtype=torch.int32, device=cuda)
    silent_peer = torch.zeros(256, dtype=torch.int32, device=cuda)
    table = _abi.ElxPeerTable()
    table.base[0], table.base[1] = mine.data_ptr(), silent_peer.data_ptr()
    table.rank, table.world = 0, 2
    ctl = K.ControlBlock(cuda, 1.0)
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)
    t0 = time.time()
    assert lib.elx_peer_barrier(table, 1, ctl.ptr, 1, 200, stream) == _abi.OK
    torch.cuda.synchronize()
    elapsed = time.time() - t0
    assert 0.15 < elapsed < 5.0
    c = ctl.read()
    assert c.status & _abi.STAT_TIMEOUT
    # what this rank announced did arrive in both regions (slot of sender 0, parity of epoch 1)
    slot = (1 * _abi.MAX_PEERS + 0) * 2
    assert mine[slot].item() == 1 and silent_peer[slot].item() == 1
    # a world of one completes at once, and the device still works
    solo = _abi.ElxPeerTable()
    solo.base[0], solo.rank, solo.world = mine.data_ptr(), 0, 1
    ctl2 = K.ControlBlock(cuda, 1.0)
    assert lib.elx_peer_barrier(solo, 2, ctl2.ptr, 0, 200, stream) == _abi.OK
    torch.cuda.synchronize()
    assert ctl2.read().status == 0
    assert lib.elx_peer_barrier(solo, 0, ctl2.ptr, 0, 200, stream) == _abi.ERR_ARG    # epochs start at 1


def test_expired_wait_forces_a_skip_instead_of_an_update(K, oracle, cuda):
    """After a wait gave up (ELX_STAT_TIMEOUT, raised here by a barrier whose peer never arrives) the
    gradients may be incomplete: the next decision is "skip" although no overflow was seen, the loss scaler and
    the step count stay as they were, and the update launch only refreshes the working copy."""
    from elixir_b200 import _abi, _lib
    lib = _lib.get()
    mine = torch.zeros(256, dtype=torch.int32, device=cuda)
    silent_peer = torch.zeros(256, dtype=torch.int32, device=cuda)
    table = _abi.ElxPeerTable()
    table.base[0], table.base[1] = mine.data_ptr(), silent_peer.data_ptr()
    table.rank, table.world = 0, 2
    ctl = K.ControlBlock(cuda, 64.0)
    cfg = K.scaler_cfg(True, growth_interval=1, hysteresis=1)
    n = 3 * 4096 + 9
    p, m, v, g = (t.to(cuda) for t in make_chunk(n, torch.float16, seed=5))
    p0 = p.clone()
    flags = torch.ones(3, dtype=torch.int32, device=cuda)
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)
    assert lib.elx_peer_barrier(table, 1, ctl.ptr, 1, 100, stream) == _abi.OK
    K.step_begin(ctl, cfg, chunk_flags=flags)
    K.adam_chunk(p, m, v, g, K.hyper(), ctl)
    c = ctl.read()
    assert c.status & _abi.STAT_TIMEOUT
    assert (c.skip, c.forced_skips, c.skipped_steps, c.step, c.scale, c.growth_step) == (1, 1, 1, 0, 64.0, 0)
    assert flags.tolist() == [0, 0, 0]    # the decision clears the per-chunk overflow words
    assert bits_equal(p, p0) and float(m.abs().max()) == 0.0 and float(v.abs().max()) == 0.0
    want16 = torch.empty(n, dtype=torch.float16)
    oracle.cast(p0.cpu(), want16)
    assert bits_equal(g, want16)
    # the bit is sticky: the next step is skipped too, until the host has looked (engine.check_status raises)
    K.step_begin(ctl, cfg)
    assert ctl.read().forced_skips == 2
    from elixir_b200.engine import ChunkStepEngine
    engine = ChunkStepEngine(cuda, torch.float16)
    engine.ctl = ctl
    with pytest.raises(RuntimeError, match='bounded wait'):
        engine.check_status()


@pytest.mark.parametrize('variant', [0, 1])
@pytest.mark.parametrize('dtype', DTYPES)
def test_gradient_source_separate_from_the_working_copy(K, oracle, cuda, dtype, variant):
    """With ElxChunkDesc.grad_src the probe and the update read the gradient where it was produced and only
    write the working copy into the shard: same bits as copying the gradient into the shard first, and the
    source is left untouched.  Whole tiles that no segment covers (the tail past valid_end, a gap between two
    segments) take the refresh-only path of the pipelined kernel."""
    sizes = [40 * 4096, 5 * 4096 + 100, 4096, 3, 12 * 4096]
    valid = [40 * 4096 - 5, 5 * 4096 + 100, 1000, 0, 7 * 4096 + 1]
    seg_lists = [
        _segments(valid[0], [100, 4096, 4096 + 7, 20 * 4096, 30 * 4096 + 2048], [0, 1, 2, -1, 0, 1]),
        _segments(valid[1], [2 * 4096], [1, 0]),
        _segments(valid[2], [], [2]),
        [],
        _segments(valid[4], [3 * 4096 + 5], [0, 2]),
    ]
    hypers = [K.hyper(1e-3, (0.9, 0.999), 1e-8, 0.01, True), K.hyper(5e-4, (0.9, 0.98), 1e-6, 0.0, True),
              K.hyper(2e-3, (0.85, 0.99), 1e-8, 0.05, False)]
    scale = 512.0
    K.set_tuning(adam_variant=variant)
    try:
        # reference run: gradients copied into the shards
        table, host, dev_t, host_t = _build_set(K, oracle, cuda, dtype, sizes, valid, seg_lists, 91, scale)
        table.set_hyper(hypers)
        # run under test: same state, gradients in tensors of their own
        table2 = K.ChunkTable(cuda, dtype)
        dev2, srcs = [], []
        for c, (n, nv, segs) in enumerate(zip(sizes, valid, seg_lists)):
            p, m, v, _ = (t.clone() for t in dev_t[c])
            lowp = torch.full((n,), 3.0, dtype=dtype, device=cuda)    # stale parameters: must never be read
            src = torch.empty(n, dtype=dtype, device=cuda)
            table2.add_chunk(p, m, v, lowp, n_valid=nv, segments=segs, grad_src=src)
            dev2.append((p, m, v, lowp))
            srcs.append(src)
        table2.finalize()
        table2.set_hyper(hypers)
        cfg = K.scaler_cfg(True, growth_interval=2, hysteresis=1)
        ctl1, ctl2 = K.ControlBlock(cuda, scale), K.ControlBlock(cuda, scale)
        flags1 = torch.zeros(table.n_chunks, dtype=torch.int32, device=cuda)
        flags2 = torch.zeros(table.n_chunks, dtype=torch.int32, device=cuda)
        for step in range(3):
            for c, n in enumerate(sizes):
                gen = torch.Generator().manual_seed(17 * step + c)
                g = (torch.randn(n, generator=gen) * 1e-3 * scale).to(dtype)
                if step == 1 and c == 4:
                    g[valid[c] - 1] = float('nan')
                    g[valid[c]] = float('inf')    # past valid_end: not probed, not used
                dev_t[c][3].copy_(g)
                srcs[c].copy_(g)
            K.grad_check_multi(table, ctl1, chunk_flags=flags1)
            K.grad_check_multi(table2, ctl2, chunk_flags=flags2)
            assert flags1.tolist() == flags2.tolist() == [int(step == 1 and c == 4) for c in range(len(sizes))]
            K.step_begin(ctl1, cfg, chunk_flags=flags1)
            K.step_begin(ctl2, cfg, chunk_flags=flags2)
            kept = [s.clone() for s in srcs]
            K.adam_multi(table, ctl1)
            K.adam_multi(table2, ctl2)
            assert _ctl_fields(ctl1.read()) == _ctl_fields(ctl2.read())
            assert bool(ctl2.read().skip) == (step == 1)
            for c in range(len(sizes)):
                for x, y in zip(dev_t[c], dev2[c]):
                    assert bits_equal(x, y), (step, c)
                assert bits_equal(srcs[c], kept[c]), (step, c)
        assert ctl2.read().status == 0
    finally:
        K.set_tuning(adam_variant=-1)


# --------------------------------------------------------------------------------------------------
# argument validation: errors are status codes, nothing is launched
# --------------------------------------------------------------------------------------------------


def test_bad_arguments_are_rejected(K, cuda):
    from elixir_b200 import _abi, _lib
    lib = _lib.get()
    good = torch.zeros(4096, device=cuda)
    g16 = torch.zeros(4096, dtype=torch.float16, device=cuda)
    ctl = K.ControlBlock(cuda, 1.0)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    flag = torch.zeros(1, dtype=torch.int32, device=cuda)
    assert lib.elx_grad_check(None, 0, 10, P(flag), None, None, None, 0, None) == _abi.ERR_NULL
    assert lib.elx_grad_check(P(g16), 7, 10, P(flag), None, None, None, 0, None) == _abi.ERR_DTYPE
    assert lib.elx_grad_check(P(g16), 0, -1, P(flag), None, None, None, 0, None) == _abi.ERR_SIZE
    assert lib.elx_grad_check(ctypes.c_void_p(g16.data_ptr() + 1), 0, 10, P(flag), None, None, None, 0,
                              None) == _abi.ERR_ALIGN
    out = torch.zeros(1, device=cuda)
    assert lib.elx_grad_check(P(g16), 0, 4096, None, None, P(out), None, 0, None) == _abi.ERR_NULL
    assert lib.elx_grad_check(P(g16), 0, 4096, None, None, P(out), P(good), 0, None) == _abi.ERR_SIZE
    assert lib.elx_reduce_epilogue(P(g16), P(g16), 0, 4096, 4096, P(flag), None, None, None, 0, None) == _abi.ERR_ARG
    assert lib.elx_adam_chunk(P(good), P(good), P(good), P(g16), 0, 5000, 4096, K.hyper(), ctl.ptr,
                              None) == _abi.ERR_SIZE
    assert lib.elx_adam_chunk(P(good), None, P(good), P(g16), 0, 4096, 4096, K.hyper(), ctl.ptr, None) == _abi.ERR_NULL
    assert lib.elx_adam_multi(P(good), 0, 1, 1, 0, P(good), P(good), 65, ctl.ptr, None) == _abi.ERR_CAPACITY
    assert lib.elx_set_tuning(b'adam_threads', 300) == _abi.ERR_ARG
    assert lib.elx_set_tuning(b'no_such_knob', 1) == _abi.ERR_ARG
    assert lib.elx_strerror(_abi.ERR_ALIGN).decode().startswith('a pointer')
    with pytest.raises(RuntimeError):
        K.grad_check(torch.zeros(8, dtype=torch.float16), flag=flag.cpu())    # CPU tensor: no CPU path
    torch.cuda.synchronize()
