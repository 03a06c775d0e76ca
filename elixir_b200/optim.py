"""The optimizer plug behind ElixirOptimizer.

``HybridAdam`` / ``FusedAdam`` take the place of the ColossalAI optimizers that the reference accepts
(``_AVAIL_OPTIM_LIST``, ``elixir/wrapper/optimizer.py:19, 54-56``): same constructor, same
``step(closure=None, div_scale=-1)`` seam, same per-parameter state keys (``step``, ``exp_avg``,
``exp_avg_sq``).  The difference is what ``step`` does: instead of looping over per-tensor views it
asks the ``ChunkStepEngine`` it is bound to for ONE fused launch over all chunk shards.  The
hyper-parameters are re-read from ``param_groups`` on every step, so lr schedulers keep working.
"""
from typing import Optional

import torch

from . import kernels


class ChunkAdam(torch.optim.Optimizer):

    def __init__(self,
                 model_params,
                 lr: float = 1e-3,
                 bias_correction: bool = True,
                 betas=(0.9, 0.999),
                 eps: float = 1e-8,
                 weight_decay: float = 0,
                 adamw_mode: bool = True,
                 **unused):
        defaults = dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(model_params, defaults)
        self.adamw_mode = adamw_mode
        self._engine = None

    def bind_engine(self, engine):
        self._engine = engine

    def hyper_table(self):
        return [
            kernels.hyper(lr=g['lr'], betas=g['betas'], eps=g['eps'], weight_decay=g['weight_decay'],
                          adamw_mode=self.adamw_mode, bias_correction=g.get('bias_correction', True))
            for g in self.param_groups
        ]

    @torch.no_grad()
    def step(self, closure=None, div_scale: Optional[float] = -1):
        """Launch the fused update.  The divisor of the gradients is NOT the ``div_scale`` argument: it is
        the value the device-side decision (``elx_step_begin``) left in the control block, i.e. the loss
        scale as it was during backward times the clip factor.  The argument is kept for signature
        compatibility and must be left at -1/None."""
        if self._engine is None:
            raise RuntimeError(f'{type(self).__name__} steps through chunk kernels: wrap it in ElixirOptimizer first')
        if div_scale is not None and div_scale != -1:
            raise ValueError('div_scale lives in the device control block; do not pass it')
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._engine.set_hyper(self.hyper_table())
        self._engine.update()
        return loss


class HybridAdam(ChunkAdam):
    pass


class FusedAdam(ChunkAdam):
    pass


class CPUAdam:

    def __init__(self, *args, **kwargs):
        raise RuntimeError('elixir_b200 keeps optimizer state in HBM and has no CPU Adam; use HybridAdam or FusedAdam')
