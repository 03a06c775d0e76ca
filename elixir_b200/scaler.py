"""Loss scalers whose state lives in the optimizer's device control block.

They stand where ElixirOptimizer builds ColossalAI's ``DynamicGradScaler`` / ``ConstantGradScaler``
(``elixir/wrapper/optimizer.py:76-86``).  The update itself runs inside ``elx_step_begin`` on the
device, in the order the reference applies it (scale read for the divisor first, then ``update``:
``optimizer.py:196-209``); these classes hold the configuration and give read access to the state.
"""
from typing import Optional

import torch

from . import kernels


class BaseGradScaler:

    def __init__(self, initial_scale: float, dynamic: bool, **cfg):
        self.initial_scale = float(initial_scale)
        self.cfg = kernels.scaler_cfg(dynamic=dynamic, **cfg)
        self.ctl: Optional[kernels.ControlBlock] = None

    def attach(self, ctl: kernels.ControlBlock):
        self.ctl = ctl
        return self

    def set_max_norm(self, max_norm: float):
        self.cfg.max_norm = float(max_norm)

    @property
    def scale(self) -> torch.Tensor:
        """0-dim float32 device tensor holding the current loss scale (no host read)."""
        return self.ctl.scale

    @property
    def inv_scale(self) -> torch.Tensor:
        return self.ctl.scale.reciprocal()

    def state_dict(self):
        c = self.ctl.read()
        return dict(scale=c.scale, growth_step=c.growth_step, hysteresis_step=c.hysteresis_step, step=c.step,
                    skipped_steps=c.skipped_steps)

    def load_state_dict(self, state):
        c = self.ctl.read()
        c.scale = float(state['scale'])
        c.growth_step = int(state.get('growth_step', 0))
        c.hysteresis_step = int(state.get('hysteresis_step', 0))
        c.step = int(state.get('step', c.step))
        c.skipped_steps = int(state.get('skipped_steps', 0))
        self.ctl.write(c)


class DynamicGradScaler(BaseGradScaler):

    def __init__(self,
                 initial_scale: float = 2**16,
                 growth_factor: float = 2,
                 backoff_factor: float = 0.5,
                 growth_interval: int = 1000,
                 min_scale: Optional[float] = None,
                 max_scale: Optional[float] = None,
                 hysteresis: int = 2,
                 verbose: bool = False):
        if not growth_factor > 1:
            raise ValueError('growth_factor must be larger than 1')
        if not 0 < backoff_factor < 1:
            raise ValueError('backoff_factor must be between 0 and 1')
        if hysteresis < 0:
            raise ValueError('hysteresis cannot be negative')
        if min_scale and max_scale and min_scale > max_scale:
            raise ValueError('min_scale exceeds max_scale')
        super().__init__(initial_scale, True, growth_factor=growth_factor, backoff_factor=backoff_factor,
                         growth_interval=growth_interval, min_scale=min_scale or 0.0, max_scale=max_scale or 0.0,
                         hysteresis=hysteresis)


class ConstantGradScaler(BaseGradScaler):

    def __init__(self, initial_scale: float = 1.0, verbose: bool = False):
        super().__init__(initial_scale, False)
