import torch


class BaseGradScaler:

    def __init__(self, initial_scale: float, verbose: bool = False):
        self._scale = torch.tensor([initial_scale], dtype=torch.float32)

    @property
    def scale(self):
        return self._scale

    def update(self, overflow: bool):
        raise NotImplementedError


class ConstantGradScaler(BaseGradScaler):

    def update(self, overflow: bool):
        pass


class DynamicGradScaler(BaseGradScaler):

    def __init__(self, initial_scale=2**16, growth_factor=2, backoff_factor=0.5, growth_interval=1000, min_scale=None,
                 max_scale=None, hysteresis=2, verbose=False):
        super().__init__(initial_scale, verbose)
        self._min_scale = torch.tensor([min_scale], dtype=torch.float32) if min_scale else None
        self._max_scale = torch.tensor([max_scale], dtype=torch.float32) if max_scale else None
        self._growth_factor = growth_factor
        self._backoff_factor = backoff_factor
        self._growth_interval = growth_interval
        self._growth_step = 0
        self._hysteresis = hysteresis
        self._hysteresis_step = 0

    def update(self, overflow: bool):
        if overflow:
            self._hysteresis_step += 1
            self._growth_step = 0
            if self._hysteresis_step >= self._hysteresis:
                self._scale = self._scale * self._backoff_factor
                if self._min_scale is not None:
                    self._scale = torch.max(self._scale, self._min_scale)
        else:
            self._growth_step += 1
            if self._growth_step == self._growth_interval:
                self._growth_step = 0
                self._hysteresis_step = 0
                self._scale = self._scale * self._growth_factor
                if self._max_scale is not None:
                    self._scale = torch.min(self._scale, self._max_scale)
