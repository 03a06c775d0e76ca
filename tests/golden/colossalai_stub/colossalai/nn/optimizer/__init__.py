import torch


class ColossalaiOptimizer(torch.optim.Optimizer):
    """Thin wrapper that forwards to the wrapped optimizer (the shape ElixirOptimizer subclasses)."""

    def __init__(self, optim):
        self.optim = optim

    @property
    def param_groups(self):
        return self.optim.param_groups

    @property
    def defaults(self):
        return self.optim.defaults

    @property
    def state(self):
        return self.optim.state

    def zero_grad(self, *args, **kwargs):
        self.optim.zero_grad(*args, **kwargs)

    def step(self, *args, **kwargs):
        return self.optim.step(*args, **kwargs)


class _TorchBackedAdam(torch.optim.Optimizer):
    """HybridAdam-shaped front: step(div_scale) divides the gradients and delegates the arithmetic to
    torch.optim.AdamW (adamw_mode) or torch.optim.Adam with L2 decay, single-tensor code path."""

    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, weight_decay=0,
                 adamw_mode=True, **kwargs):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.adamw_mode = adamw_mode
        self._inner = None

    def _inner_optim(self):
        cls = torch.optim.AdamW if self.adamw_mode else torch.optim.Adam
        groups = [dict(params=g['params'], lr=g['lr'], betas=g['betas'], eps=g['eps'], weight_decay=g['weight_decay'])
                  for g in self.param_groups]
        inner = cls(groups, foreach=False)
        inner.state = self.state
        return inner

    @torch.no_grad()
    def step(self, closure=None, div_scale: float = -1):
        for group in self.param_groups:
            for p in group['params']:
                if p.grad is None:
                    continue
                g = p.grad.float()
                if div_scale != -1:
                    g = g / div_scale
                p.grad = g
        self._inner_optim().step()


class FusedAdam(_TorchBackedAdam):
    pass


class CPUAdam(_TorchBackedAdam):
    pass


class HybridAdam(_TorchBackedAdam):
    pass
