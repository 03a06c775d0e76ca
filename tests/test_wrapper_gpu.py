"""ElixirModule + ElixirOptimizer on a GPU, driven by a real forward / backward (world size 1)."""
import copy

import pytest
import torch
import torch.nn as nn

from _util import bits_equal, close_1e6

pytestmark = pytest.mark.gpu


class TiedNet(nn.Module):
    """Embedding tied to the output projection (a parameter used twice gets a private chunk)."""

    def __init__(self, vocab=64, hidden=32):
        super().__init__()
        self.embed = nn.Embedding(vocab, hidden)
        self.fc = nn.Linear(hidden, hidden)
        self.norm = nn.LayerNorm(hidden)
        self.head = nn.Linear(hidden, vocab, bias=False)
        self.head.weight = self.embed.weight

    def forward(self, ids):
        h = self.norm(torch.relu(self.fc(self.embed(ids))))
        return self.head(h).float().logsumexp(-1).mean()


class Mlp(nn.Module):

    def __init__(self):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(48, 96), nn.GELU(), nn.Linear(96, 96), nn.GELU(), nn.Linear(96, 8))

    def forward(self, x):
        return self.net(x).float().pow(2).mean()


@pytest.fixture(scope='module')
def single_group(cuda):
    import torch.distributed as dist
    if not dist.is_initialized():
        dist.init_process_group('gloo', init_method='tcp://127.0.0.1:29791', rank=0, world_size=1)
    yield dist.GroupMember.WORLD


def _wrap(model, group, dtype, **opt_kwargs):
    from elixir_b200.optim import HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    sr = simple_plan(model, 1, split_number=3, unified_dtype=dtype)
    inner = HybridAdam(model.parameters(), lr=opt_kwargs.pop('lr', 1e-3), weight_decay=opt_kwargs.pop('wd', 0.01))
    emodel = ElixirModule(model, sr, group, dtype=dtype)
    return emodel, ElixirOptimizer(emodel, inner, **opt_kwargs)


def test_fp32_mode_matches_plain_torch_training(cuda, single_group):
    """The reference's own acceptance test in spirit (test/wrapper/test_optimizer.py): one optimizer on a
    plain model, the same optimizer behind ElixirModule/ElixirOptimizer, fp32, a few steps, full state
    compared with rtol 2e-6 / atol 2e-5."""
    torch.manual_seed(0)
    plain = Mlp().to(cuda)
    wrapped_model = copy.deepcopy(plain)
    opt = torch.optim.AdamW(plain.parameters(), lr=1e-2, betas=(0.875, 0.99609375), weight_decay=0.0)
    emodel, eopt = _wrap(wrapped_model, single_group, torch.float, lr=1e-2, wd=0.0)
    for g in eopt.param_groups:
        g['betas'] = (0.875, 0.99609375)
    for step in range(3):
        x = torch.randn(16, 48, device=cuda)
        opt.zero_grad()
        loss_a = plain(x)
        loss_a.backward()
        opt.step()
        eopt.zero_grad()
        loss_b = emodel(x)
        eopt.backward(loss_b)
        eopt.step()
        torch.testing.assert_close(loss_a, loss_b)
    got = emodel.state_dict()
    for name, ref in plain.state_dict().items():
        torch.testing.assert_close(got[name].to(cuda), ref, rtol=2e-6, atol=2e-5)
    assert eopt.engine.read_control().status == 0


def test_an_optimizer_outside_the_available_list_is_stepped_unscaled(cuda, single_group):
    """The reference accepts any torch optimizer as long as the gradients need no division (fp32, scale 1, no
    clipping: elixir/wrapper/optimizer.py:52-56, 211-214) and steps it on the fp32 shard views.  SGD with
    momentum behind the wrapper must train like the same SGD on a plain model, also across a skipped step."""
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    torch.manual_seed(5)
    plain = Mlp().to(cuda)
    wrapped_model = copy.deepcopy(plain)
    opt = torch.optim.SGD(plain.parameters(), lr=5e-2, momentum=0.9, weight_decay=1e-3)
    sr = simple_plan(wrapped_model, 1, split_number=3, unified_dtype=torch.float)
    inner = torch.optim.SGD(wrapped_model.parameters(), lr=5e-2, momentum=0.9, weight_decay=1e-3)
    emodel = ElixirModule(wrapped_model, sr, single_group, dtype=torch.float)
    eopt = ElixirOptimizer(emodel, inner)
    assert not eopt.scaled_optimizer
    for step in range(4):
        x = torch.randn(16, 48, device=cuda)
        if step == 2:
            x[0, 0] = float('inf')    # non-finite gradients: both sides leave the parameters alone
        opt.zero_grad()
        plain(x).backward()
        if step != 2:
            opt.step()
        eopt.zero_grad()
        eopt.backward(emodel(x))
        eopt.step()
    ctl = eopt.engine.read_control()
    assert (ctl.step, ctl.skipped_steps, ctl.status) == (3, 1, 0)
    got = emodel.state_dict()
    for name, ref in plain.state_dict().items():
        torch.testing.assert_close(got[name].to(cuda), ref, rtol=2e-6, atol=2e-5)
    saved = eopt.state_dict()
    assert 'optim' in saved and len(saved['optim']['state']) > 0
    eopt.load_state_dict(saved)


def test_an_optimizer_outside_the_available_list_is_refused_when_gradients_are_scaled(cuda, single_group):
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    torch.manual_seed(6)
    model = Mlp().to(cuda)
    sr = simple_plan(model, 1, split_number=3, unified_dtype=torch.float16)
    emodel = ElixirModule(model, sr, single_group, dtype=torch.float16)
    eopt = ElixirOptimizer(emodel, torch.optim.SGD(model.parameters(), lr=1e-2), initial_scale=64.0)
    eopt.zero_grad()
    eopt.backward(emodel(torch.randn(8, 48, device=cuda)))
    with pytest.raises(AssertionError, match='available list'):
        eopt.step()


def test_per_parameter_step_counts_follow_the_device_counter(cuda, single_group):
    """state[p]['step'] is the number of applied updates (skipped steps do not count), as the reference's
    optimizers keep it; here it is read from the control block when the state is looked at."""
    torch.manual_seed(7)
    model = Mlp().to(cuda)
    emodel, eopt = _wrap(model, single_group, torch.float16, initial_scale=64.0, hysteresis=1)
    for step in range(4):
        x = torch.randn(8, 48, device=cuda)
        if step == 1:
            x[0, 0] = float('nan')
        eopt.zero_grad()
        eopt.backward(emodel(x))
        eopt.step()
    steps = {entry['step'] for entry in eopt.state.values()}
    assert steps == {3}
    assert eopt.state_dict()['scaler']['step'] == 3


@pytest.mark.parametrize('model_cls', [Mlp, TiedNet])
def test_fp16_step_matches_oracle_on_the_gradients_autograd_produced(cuda, oracle, single_group, model_cls):
    from elixir_b200 import kernels as K
    torch.manual_seed(1)
    model = model_cls().to(cuda)
    emodel, eopt = _wrap(model, single_group, torch.float16, initial_scale=128.0, hysteresis=1, growth_interval=2)
    chunks = emodel.param_chunks
    assert any(c.rcache_fused for c in chunks) == (model_cls is TiedNet)
    host_ctl = oracle.new_ctl(128.0)
    hyper = [K.hyper(lr=1e-3, weight_decay=0.01)]
    for step in range(4):
        if model_cls is Mlp:
            batch = torch.randn(8, 48, device=cuda)
        else:
            batch = torch.randint(0, 64, (8, 12), device=cuda)
        eopt.zero_grad()
        loss = emodel(batch)
        eopt.backward(loss)
        if step == 2:    # poison one reduced gradient: the whole step must be skipped
            chunks[0].shard[3] = float('inf')
            chunks[0].overflow = True
            eopt.engine.ctl.found_inf.fill_(1)
        # CPU replay on what is in the shards right now
        cs = oracle.ChunkSet(torch.float16)
        masters = []
        for i, c in enumerate(chunks):
            m, e1, e2, lowp, nv = (t.cpu().clone() if torch.is_tensor(t) else t for t in eopt.engine.shards[i])
            cs.add_chunk(m, e1, e2, lowp, nv, [(0, nv, 0)] if nv else [])
            masters.append((m, e1, e2))
        eopt.step()
        skipped = cs.step(host_ctl, eopt.grad_scaler.cfg, hyper, probe=True, f64=True)
        ctl = eopt.engine.read_control()
        assert bool(ctl.skip) == skipped == (step == 2)
        assert (ctl.scale, ctl.step, ctl.growth_step) == (host_ctl.scale, host_ctl.step, host_ctl.growth_step)
        for i, c in enumerate(chunks):
            for got, want in zip(eopt.engine.shards[i][:3], masters[i]):
                ok, ratio = close_1e6(got, want.double())
                assert ok, (step, i, ratio)
            want16 = torch.empty(c.shard_size, dtype=torch.float16)
            oracle.cast(c.paired_chunk.shard.cpu(), want16)
            assert bits_equal(c.shard, want16)
    assert eopt.engine.read_control().status == 0
    assert all(p.grad is None for p in model.parameters())


def test_training_reduces_the_loss_and_state_dict_round_trips(cuda, single_group):
    torch.manual_seed(2)
    model = Mlp().to(cuda)
    emodel, eopt = _wrap(model, single_group, torch.float16, lr=3e-3, wd=0.0, initial_scale=1024.0)
    x = torch.randn(64, 48, device=cuda)
    losses = []
    for _ in range(30):
        eopt.zero_grad()
        loss = emodel(x)
        eopt.backward(loss)
        eopt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.5 * losses[0]
    state = emodel.state_dict()
    ostate = eopt.state_dict()
    assert ostate['scaler']['step'] == 30 - ostate['scaler']['skipped_steps']
    zeros = {k: torch.zeros_like(v) for k, v in state.items()}
    emodel.load_state_dict(zeros)
    assert all(float(v.abs().max()) == 0.0 for v in emodel.state_dict().values())
    emodel.load_state_dict(state)
    again = emodel.state_dict()
    for k in state:
        assert bits_equal(again[k], state[k])
    with torch.no_grad():
        assert abs(emodel(x).item() - emodel(x).item()) == 0.0


def test_init_step_reproduces_the_reference_side_effects(cuda, single_group):
    """init_step=True takes one step with zero gradients: the step count becomes 1 and decoupled weight decay
    shrinks every weight once (elixir/wrapper/optimizer.py:94-113)."""
    torch.manual_seed(3)
    model = Mlp().to(cuda)
    before = {n: p.detach().clone().float() for n, p in model.named_parameters()}
    emodel, eopt = _wrap(model, single_group, torch.float16, lr=1e-2, wd=0.1, init_step=True)
    assert eopt.engine.read_control().step == 1
    after = emodel.state_dict()
    for n, ref in before.items():
        torch.testing.assert_close(after[n].to(cuda), ref * (1 - 1e-2 * 0.1), rtol=1e-6, atol=1e-9)


def test_lr_schedule_and_param_groups_are_picked_up_every_step(cuda, oracle, single_group):
    """Hyper-parameters are re-read from param_groups on every step (lr schedulers mutate them) and groups with
    different settings update their own ranges of the same chunks."""
    from elixir_b200 import kernels as K
    from elixir_b200.optim import HybridAdam
    from elixir_b200.wrapper import ElixirModule, ElixirOptimizer, simple_plan
    torch.manual_seed(5)
    model = Mlp().to(cuda)
    decay = [p for n, p in model.named_parameters() if n.endswith('weight')]
    no_decay = [p for n, p in model.named_parameters() if n.endswith('bias')]
    inner = HybridAdam([dict(params=decay, weight_decay=0.05), dict(params=no_decay, weight_decay=0.0, lr=2e-3)], lr=1e-3)
    sr = simple_plan(model, 1, split_number=2, unified_dtype=torch.float16)
    emodel = ElixirModule(model, sr, single_group, dtype=torch.float16)
    eopt = ElixirOptimizer(emodel, inner, initial_scale=256.0)
    sched = torch.optim.lr_scheduler.LambdaLR(inner, lambda step: 1.0 / (1 + step))
    host_ctl = oracle.new_ctl(256.0)
    chunks = emodel.param_chunks
    seg_lists = [[(b, e, g) for b, e, g in eopt.engine.table._segs_of(i)] for i in range(len(chunks))]
    assert any(len({g for _, _, g in segs}) == 2 for segs in seg_lists)    # both groups inside one chunk
    for step in range(3):
        x = torch.randn(8, 48, device=cuda)
        eopt.zero_grad()
        eopt.backward(emodel(x))
        hypers = [K.hyper(lr=g['lr'], weight_decay=g['weight_decay']) for g in inner.param_groups]
        cs = oracle.ChunkSet(torch.float16)
        masters = []
        for i in range(len(chunks)):
            m, e1, e2, lowp, nv = (t.cpu().clone() if torch.is_tensor(t) else t for t in eopt.engine.shards[i])
            cs.add_chunk(m, e1, e2, lowp, nv, seg_lists[i])
            masters.append(m)
        eopt.step()
        sched.step()
        cs.step(host_ctl, eopt.grad_scaler.cfg, hypers, probe=True, f64=True)
        for i in range(len(chunks)):
            ok, ratio = close_1e6(eopt.engine.shards[i][0], masters[i].double())
            assert ok, (step, i, ratio)
    assert inner.param_groups[0]['lr'] < 1e-3


def test_checkpoint_resume_continues_bit_identically(cuda, single_group):
    """Flat-state checkpoint (fp32 masters through ElixirModule.state_dict, moments + control block through
    ElixirOptimizer.state_dict): a run resumed from it takes exactly the steps the original run takes."""
    def fresh():
        torch.manual_seed(11)
        model = Mlp().to(cuda)
        return _wrap(model, single_group, torch.float16, lr=2e-3, wd=0.01, initial_scale=512.0, growth_interval=3,
                     hysteresis=1)

    def train(emodel, eopt, steps, first):
        for i in range(first, first + steps):
            gen = torch.Generator(device=cuda).manual_seed(1000 + i)
            x = torch.randn(8, 48, device=cuda, generator=gen)
            eopt.zero_grad()
            eopt.backward(emodel(x))
            if i == 2:    # an overflow before the checkpoint, so the scaler counters are not trivial
                eopt.engine.ctl.found_inf.fill_(1)
            eopt.step()

    emodel, eopt = fresh()
    train(emodel, eopt, 4, 0)
    model_state, optim_state = emodel.state_dict(), eopt.state_dict()
    train(emodel, eopt, 3, 4)
    want = [[t.cpu() for t in s[:4]] for s in eopt.engine.shards]
    want_ctl = eopt.grad_scaler.state_dict()

    emodel2, eopt2 = fresh()
    emodel2.load_state_dict(model_state)
    eopt2.load_state_dict(optim_state)
    assert eopt2.grad_scaler.state_dict() == optim_state['scaler']
    train(emodel2, eopt2, 3, 4)
    assert eopt2.grad_scaler.state_dict() == want_ctl
    for got, ref in zip(eopt2.engine.shards, want):
        for a, b in zip(got[:4], ref):
            assert bits_equal(a, b)


def test_bf16_module_runs_with_a_constant_scale_and_matches_the_oracle(cuda, oracle, single_group):
    """bfloat16 working copies (an extension: the reference accepts float and float16 only): constant loss scale
    1, no unscale, same fused step."""
    from elixir_b200 import kernels as K
    from elixir_b200.scaler import ConstantGradScaler
    torch.manual_seed(8)
    model = Mlp().to(cuda)
    emodel, eopt = _wrap(model, single_group, torch.bfloat16)
    assert isinstance(eopt.grad_scaler, ConstantGradScaler) and not emodel.use_amp
    host_ctl = oracle.new_ctl(1.0)
    hyper = [K.hyper(lr=1e-3, weight_decay=0.01)]
    chunks = emodel.param_chunks
    for step in range(2):
        eopt.zero_grad()
        eopt.backward(emodel(torch.randn(8, 48, device=cuda)))
        cs = oracle.ChunkSet(torch.bfloat16)
        masters = []
        for i in range(len(chunks)):
            m, e1, e2, lowp, nv = (t.cpu().clone() if torch.is_tensor(t) else t for t in eopt.engine.shards[i])
            cs.add_chunk(m, e1, e2, lowp, nv, [(0, nv, 0)] if nv else [])
            masters.append(m)
        eopt.step()
        assert not cs.step(host_ctl, eopt.grad_scaler.cfg, hyper, probe=True, f64=True)
        ctl = eopt.engine.read_control()
        assert (ctl.scale, ctl.div_scale, ctl.step) == (1.0, -1.0, step + 1)
        for i, c in enumerate(chunks):
            assert close_1e6(eopt.engine.shards[i][0], masters[i].double())[0]
            want16 = torch.empty(c.shard_size, dtype=torch.bfloat16)
            oracle.cast(c.paired_chunk.shard.cpu(), want16)
            assert bits_equal(c.shard, want16)


def test_wrapper_gradient_clipping(cuda, single_group):
    """max_norm at the wrapper level: the update is divided by clip x scale once the unscaled global norm exceeds
    max_norm (the reference's dead clipping branch, elixir/wrapper/optimizer.py:149-183, made to work)."""
    torch.manual_seed(9)
    model = Mlp().to(cuda)
    emodel, eopt = _wrap(model, single_group, torch.float16, initial_scale=256.0, max_norm=1e-3)
    x = torch.randn(8, 48, device=cuda)
    eopt.zero_grad()
    eopt.backward(emodel(x))
    eopt.step()
    ctl = eopt.engine.read_control()
    assert ctl.skip == 0 and ctl.status == 0
    assert ctl.grad_norm > 1e-3 and ctl.clip_coef > 1.0
    assert abs(ctl.div_scale - ctl.clip_coef * 256.0) <= 1e-5 * ctl.div_scale
    assert abs(ctl.clip_coef - (ctl.grad_norm + 1e-6) / 1e-3) <= 1e-5 * ctl.clip_coef


@pytest.mark.parametrize('prefetch', [False, True])
@pytest.mark.parametrize('dtype', [torch.float16, torch.float])
def test_scheduled_residency_equals_everything_resident(cuda, single_group, prefetch, dtype):
    """Two replica-cache blocks for five and more public chunks: chunks leave and come back during forward
    and backward (FIFO; Belady with gathers ahead on a side stream), results bit-identical."""
    import _dist_workers as W
    W.residency_check(single_group, 0, 1, prefetch, dtype, cuda)


@pytest.mark.parametrize('dtype', [torch.float, torch.float16])
def test_micro_gpt2_through_both_residency_modes(cuda, single_group, dtype):
    pytest.importorskip('transformers')
    import _dist_workers as W
    W.gpt2_check(single_group, cuda, dtype)
