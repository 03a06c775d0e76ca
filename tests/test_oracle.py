"""Pins of the CPU oracle itself (no GPU).

* 16-bit conversions: bit-exact against torch's CPU casts over the whole fp32 exponent range.
* probe / sum of squares: against torch.isinf|isnan and float().norm(2)**2 — the expressions the
  reference uses (elixir/chunk/core/chunk.py:214-221).
* Adam / AdamW arithmetic: against torch.optim.Adam / AdamW evaluated in float64 from the same state
  (the stand-in for the ColossalAI optimizers, which cannot be installed offline).
* rank-average reduce: against the reference's sequence (divide in the chunk dtype, then sum).
"""
import pytest
import torch

from _util import bits_equal, close_1e6


def test_fp16_bf16_casts_bit_exact_vs_torch(oracle):
    gen = torch.Generator().manual_seed(0)
    n = 1 << 21
    x = torch.randn(n, generator=gen) * torch.logspace(-46, 39, n)
    edge = torch.tensor([0.0, -0.0, 65504.0, 65519.996, 65520.0, -65520.0, 5.9604645e-8, 2.9802322e-8, 2.9802326e-8,
                         8.940697e-8, 6.1035156e-5, 6.0975552e-5, 1e-45, 3.4028235e38, 3.3895314e38, 3.3961775e38,
                         float('inf'), -float('inf')])
    x = torch.cat([x, edge])
    for dtype in (torch.float16, torch.bfloat16):
        got = torch.empty(x.numel(), dtype=dtype)
        oracle.cast(x, got)
        assert bits_equal(got, x.to(dtype)), dtype
    nan = torch.tensor([float('nan')])
    for dtype in (torch.float16, torch.bfloat16):
        got = torch.empty(1, dtype=dtype)
        oracle.cast(nan, got)
        assert torch.isnan(got.float()).all()
    # every fp16 / bf16 bit pattern converts back to the same float torch gives
    lib = oracle.lib()
    pats = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16)
    for dtype, fn in ((torch.float16, lib.orc_f16_to_f32), (torch.bfloat16, lib.orc_bf16_to_f32)):
        want = pats.view(dtype).float()
        for i in range(0, 65536, 97):
            w = want[i].item()
            g = fn(i)
            assert (g != g and w != w) or g == w, (dtype, i)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16, torch.float32])
def test_probe_and_norm_vs_torch_expressions(oracle, dtype):
    gen = torch.Generator().manual_seed(1)
    g = (torch.randn(100003, generator=gen) * 50).to(dtype)
    assert not oracle.probe(g)
    ref = g.float().norm(2).item()**2
    assert abs(oracle.l2sq(g) - ref) <= 1e-5 * ref
    for val in (float('inf'), -float('inf'), float('nan')):
        for pos in (0, 50001, 100002):
            h = g.clone()
            h[pos] = val
            want = bool(torch.isinf(h).any().item() | torch.isnan(h).any().item())
            assert oracle.probe(h) == want is True
            assert oracle.probe(h, n_valid=pos) is False    # the bad element lies outside [0, valid_end)
            assert oracle.probe(h, n_valid=pos + 1) is True


def _torch_step64(Opt, p, m, v, g, step, lr, betas, eps, wd):
    """One step of torch.optim.Adam/AdamW in float64 from an injected state."""
    tp = torch.nn.Parameter(p.double().clone())
    opt = Opt([tp], lr=lr, betas=betas, eps=eps, weight_decay=wd)
    opt.state[tp] = {'step': torch.tensor(float(step - 1)), 'exp_avg': m.double().clone(),
                     'exp_avg_sq': v.double().clone()}
    tp.grad = g.double().clone()
    opt.step()
    st = opt.state[tp]
    return tp.data, st['exp_avg'], st['exp_avg_sq']


@pytest.mark.parametrize('mode', ['adam', 'adamw', 'l2'])
@pytest.mark.parametrize('step', [1, 2, 10, 1000])
def test_adam_formula_pinned_against_torch_optim(oracle, mode, step):
    """Dyadic betas make (1 - beta) exact in fp32, so the only differences left are roundings: the
    double-precision oracle must agree with torch.optim in double to fp32 resolution."""
    from elixir_b200 import kernels as K
    n = 50000
    gen = torch.Generator().manual_seed(step)
    p = torch.randn(n, generator=gen) * 0.02
    m = torch.randn(n, generator=gen) * 1e-4 if step > 1 else torch.zeros(n)
    v = torch.rand(n, generator=gen) * 1e-6 if step > 1 else torch.zeros(n)
    scale = 64.0
    g16 = (torch.randn(n, generator=gen) * 1e-3 * scale).half()
    betas, lr, eps = (0.875, 0.99609375), 0.0009765625, 1e-8
    wd = 0.0 if mode == 'adam' else 0.0078125
    Opt = torch.optim.AdamW if mode == 'adamw' else torch.optim.Adam
    want = _torch_step64(Opt, p, m, v, g16.double() / scale, step, lr, betas, eps, wd)
    h = K.hyper(lr, betas, eps, wd, adamw_mode=(mode != 'l2'))
    for f64, tol in ((True, 2e-7), (False, 1e-6)):
        po, mo, vo = p.clone(), m.clone(), v.clone()
        oracle.adam(po, mo, vo, g16, h, step, scale, f64=f64)
        for name, got, ref in (('p', po, want[0]), ('m', mo, want[1]), ('v', vo, want[2])):
            ok, ratio = close_1e6(got, ref, rtol=tol)
            assert ok, (mode, step, f64, name, ratio)


def test_adam_default_betas_differ_from_torch_only_by_the_fp32_one_minus_beta(oracle):
    """With beta2 = 0.999 the reference kernels form (1 - beta2) in fp32 (0.00099998713), torch in double:
    a known 1.3e-5 relative offset of exp_avg_sq, nothing else."""
    from elixir_b200 import kernels as K
    n = 20000
    gen = torch.Generator().manual_seed(3)
    p = torch.randn(n, generator=gen) * 0.02
    g16 = (torch.randn(n, generator=gen) * 1e-3).half()
    want = _torch_step64(torch.optim.Adam, p, torch.zeros(n), torch.zeros(n), g16.double(), 1, 1e-3, (0.9, 0.999), 1e-8,
                         0.0)
    po, mo, vo = p.clone(), torch.zeros(n), torch.zeros(n)
    oracle.adam(po, mo, vo, g16, K.hyper(), 1, -1.0, f64=True)
    nz = want[2] > 0
    rel_v = ((vo.double() - want[2]).abs() / want[2].clamp_min(1e-300))[nz].max().item()
    assert 1.0e-5 < rel_v < 1.6e-5
    assert close_1e6(po, want[0], rtol=2e-6)[0]


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize('world', [2, 4, 8])
def test_reduce_avg_follows_divide_then_sum(oracle, dtype, world):
    gen = torch.Generator().manual_seed(world)
    ranks = [(torch.randn(10007, generator=gen) * 300).to(dtype) for _ in range(world)]
    ranks[0][5] = 60000.0 if dtype == torch.float16 else 3e38
    ranks[1][5] = 60000.0 if dtype == torch.float16 else 3e38
    got = oracle.reduce_avg(ranks)
    acc = None
    for r in ranks:
        q = r.clone()
        q /= world    # rounded in the chunk dtype, as `reduce_buffer /= pg_size` does
        acc = q if acc is None else (acc + q)
    assert bits_equal(got, acc)
    assert torch.isfinite(got.float()[5])    # pre-division keeps a sum finite that post-division would overflow


def test_scaler_state_machine_against_a_python_restatement(oracle):
    """orc_step_begin vs a literal Python transcription of DynamicGradScaler.update plus the ElixirOptimizer.step
    ordering (scale read for the divisor BEFORE the update; the step counter moves only on applied steps)."""
    import numpy as np
    from elixir_b200 import kernels as K
    for hysteresis in (1, 2, 4):
        cfg = K.scaler_cfg(True, 2.0, 0.5, 1.0, 2.0**24, growth_interval=3, hysteresis=hysteresis)
        ctl = oracle.new_ctl(2.0**16)
        scale, growth, hyst, step = np.float32(2.0**16), 0, 0, 0
        gen = torch.Generator().manual_seed(hysteresis)
        for found in (torch.rand(500, generator=gen) < 0.2).tolist():
            ctl.found_inf = int(found)
            oracle.step_begin(ctl, cfg)
            if found:
                hyst += 1
                growth = 0
                if hyst >= hysteresis:
                    scale = max(np.float32(scale * np.float32(0.5)), np.float32(1.0))
                want_div, want_skip = -1.0, 1
            else:
                want_div = -1.0 if scale == 1 else float(scale)
                want_skip = 0
                step += 1
                growth += 1
                if growth == 3:
                    growth, hyst = 0, 0
                    scale = min(np.float32(scale * np.float32(2.0)), np.float32(2.0**24))
            assert (ctl.scale, ctl.growth_step, ctl.hysteresis_step, ctl.step, ctl.skip, ctl.div_scale,
                    ctl.found_inf) == (float(scale), growth, hyst, step, want_skip, want_div, 0)


def test_scaler_trajectory_equals_torch_amp_update_scale(oracle):
    """An implementation nobody here wrote: torch's own loss-scale update (`torch._amp_update_scale_`, what
    torch.amp.GradScaler.update runs).  With hysteresis 1 and no clamping in reach it is the same state machine:
    back off and reset the growth tracker on an overflow, grow after `growth_interval` clean steps."""
    from elixir_b200 import kernels as K
    for growth_interval, growth, backoff in ((2, 2.0, 0.5), (5, 2.0, 0.5), (3, 4.0, 0.25)):
        cfg = K.scaler_cfg(True, growth, backoff, 0.0, 0.0, growth_interval=growth_interval, hysteresis=1)
        ctl = oracle.new_ctl(2.0**10)
        scale, tracker = torch.full((1,), 2.0**10), torch.zeros(1, dtype=torch.int32)
        gen = torch.Generator().manual_seed(growth_interval)
        for found in (torch.rand(400, generator=gen) < 0.3).tolist():
            ctl.found_inf = int(found)
            oracle.step_begin(ctl, cfg)
            torch._amp_update_scale_(scale, tracker, torch.tensor([float(found)]), growth, backoff, growth_interval)
            assert ctl.scale == float(scale) and ctl.growth_step == int(tracker) and ctl.skip == int(found)


@pytest.mark.parametrize('p_overflow', [0.7, 0.05])
def test_scaler_trajectory_with_clamps_equals_torch_amp_update_scale_clamped(oracle, p_overflow):
    """The same pin on trajectories that reach the bounds: with many overflows the scale sits on `min_scale`,
    with few it sits on `max_scale`.  torch's update knows no bounds, so its scale tensor is clamped after every
    update, which is what `max(scale * backoff, min_scale)` / `min(scale * growth, max_scale)` amount to when the
    scale starts inside the bounds."""
    from elixir_b200 import kernels as K
    lo, hi = 1.0, 16.0
    for growth_interval, growth, backoff in ((2, 2.0, 0.5), (3, 4.0, 0.25)):
        cfg = K.scaler_cfg(True, growth, backoff, lo, hi, growth_interval=growth_interval, hysteresis=1)
        ctl = oracle.new_ctl(4.0)
        scale, tracker = torch.full((1,), 4.0), torch.zeros(1, dtype=torch.int32)
        gen = torch.Generator().manual_seed(int(p_overflow * 100) + growth_interval)
        hit_lo = hit_hi = 0
        for found in (torch.rand(300, generator=gen) < p_overflow).tolist():
            ctl.found_inf = int(found)
            oracle.step_begin(ctl, cfg)
            torch._amp_update_scale_(scale, tracker, torch.tensor([float(found)]), growth, backoff, growth_interval)
            scale.clamp_(lo, hi)
            assert ctl.scale == float(scale) and ctl.growth_step == int(tracker) and ctl.skip == int(found)
            hit_lo += ctl.scale == lo
            hit_hi += ctl.scale == hi
        assert (hit_lo if p_overflow > 0.5 else hit_hi) > 50    # the bound was really in play
