"""ElixirOptimizer: the mixed-precision optimizer step over a module's chunks.

Same constructor, methods and attributes as ``elixir/wrapper/optimizer.py`` (``ElixirOptimizer``,
``:27-265``).  What changed is where the step runs: the per-rank shards are registered once with a
``ChunkStepEngine`` and ``step()`` issues — without reading anything back from the device —

    1. (W > 1) a 4-byte MAX all-reduce of the overflow word, so every rank takes the same decision
       (the reference decides per rank, ``:137-142``);
    2. ``elx_step_begin``: skip decision, combined divisor (loss scale as it was during backward, times
       the clip factor), loss-scaler update, step count (``:192-209``, ``:166-183``);
    3. ``elx_adam_multi``: unscale + Adam/AdamW + low-precision copy-back, or the copy-back alone when
       the step is skipped (``:216-219``, ``_update_fp16_params`` ``:126-135``).

Any other ``torch.optim.Optimizer`` is accepted as in the reference (``:52-56, 211-214``), for the case it allows:
no division of the gradients (loss scale 1, no clipping).  Such an optimizer steps on views of the fp32 shards
with the gradient views bound as ``.grad``; the decision still runs on the device and is read back once per step,
because a foreign optimizer cannot branch on a device word.
"""
from enum import Enum
from typing import Dict, List, Set, Tuple

import torch
from torch.nn import Parameter

from ..chunk import Chunk
from ..engine import ChunkStepEngine
from ..optim import FusedAdam, HybridAdam
from ..scaler import BaseGradScaler, ConstantGradScaler, DynamicGradScaler
from .module import ElixirModule

_AVAIL_OPTIM_LIST = {FusedAdam, HybridAdam}


class OptimState(Enum):
    SCALED = 0
    UNSCALED = 1


class ElixirOptimizer:

    def __init__(self,
                 module: ElixirModule,
                 optimizer: torch.optim.Optimizer,
                 initial_scale: float = 32768,
                 min_scale: float = 1,
                 growth_factor: float = 2,
                 backoff_factor: float = 0.5,
                 growth_interval: int = 1000,
                 hysteresis: int = 2,
                 max_scale: float = 2**24,
                 max_norm: float = 0.0,
                 norm_type: float = 2.0,
                 init_step: bool = False,
                 sync_overflow: bool = True):
        assert isinstance(module, ElixirModule)
        if not isinstance(optimizer, torch.optim.Optimizer):
            raise TypeError(f'ElixirOptimizer wraps a torch.optim.Optimizer, got {type(optimizer).__name__}')
        self.optim = optimizer
        # an optimizer of the available list takes the divisor from the device control block; any other one is
        # stepped as it is and therefore only when the gradients need no division (``:211-214``)
        self.scaled_optimizer = type(optimizer) in _AVAIL_OPTIM_LIST
        self.module = module
        self.param_chunk_group = module.param_chunk_group
        self.optim_chunk_group = module.optim_chunk_group
        self.optim_state = OptimState.UNSCALED
        self.param_to_range: Dict[Parameter, Tuple[int, int]] = dict()
        self.param_to_optim_chunk: Dict[Parameter, Chunk] = dict()
        self.param_chunk_set: Set[Chunk] = self.param_chunk_group.fused_chunks.union(
            self.param_chunk_group.float_chunks)

        self.clipping_flag = max_norm > 0.0
        self.max_norm = max_norm
        if self.clipping_flag:
            assert norm_type == 2.0, 'ElixirOptimizer only supports L2 norm now'

        if module.use_amp:
            self.grad_scaler: BaseGradScaler = DynamicGradScaler(initial_scale=initial_scale, min_scale=min_scale,
                                                                 growth_factor=growth_factor,
                                                                 backoff_factor=backoff_factor,
                                                                 growth_interval=growth_interval,
                                                                 hysteresis=hysteresis, max_scale=max_scale)
        else:
            self.grad_scaler = ConstantGradScaler(1.0, verbose=False)

        segments = self._init_optimizer()
        self._init_engine(segments, sync_overflow)
        if init_step:
            self._zero_step()

    # ------------------------------------------------------------------ construction

    def _init_optimizer(self) -> Dict[Chunk, List[Tuple[int, int, int]]]:
        """Replace every real parameter of the wrapped optimizer by an empty stand-in and remember its range
        inside this rank's shard (``__init__optimizer``, ``:238-265``)."""
        segments: Dict[Chunk, List[Tuple[int, int, int]]] = {c: [] for c in self.param_chunk_set}
        for group_index, group in enumerate(self.optim.param_groups):
            fake_params = []
            for param in group['params']:
                if not param.requires_grad:
                    continue
                param_chunk = self.module.fetcher.get_one_chunk(param)
                if param_chunk is None:
                    raise ValueError('the optimizer holds a parameter that the wrapped module does not manage')
                info = param_chunk.tensors_info[param]
                begin = max(0, info.offset - param_chunk.shard_begin)
                end = min(param_chunk.shard_size, info.end - param_chunk.shard_begin)
                if begin >= end:
                    continue
                fake = Parameter(torch.empty([0], device=param_chunk.shard.device))
                self.param_to_optim_chunk[fake] = param_chunk.paired_chunk
                self.param_to_range[fake] = (begin, end)
                segments[param_chunk].append((begin, end, group_index))
                fake_params.append(fake)
            group['params'] = fake_params
        for segs in segments.values():
            segs.sort()
        return segments

    def _init_engine(self, segments, sync_overflow: bool):
        chunks = sorted(self.param_chunk_set, key=lambda c: c.chunk_id)
        self._chunks = chunks
        device = chunks[0].compute_device if chunks else torch.device('cuda', torch.cuda.current_device())
        dtype = self.module.dtype
        group = self.module.process_group
        self.engine = ChunkStepEngine(device, dtype, self.grad_scaler, process_group=group,
                                      sync_overflow=sync_overflow, max_norm=self.max_norm)
        for chunk in chunks:
            master = chunk.paired_chunk.shard
            # a foreign optimizer keeps its own state: no flat moments are allocated for it (the master stands in
            # for them in the descriptor, which the update kernel never sees in that case)
            moments = {} if self.scaled_optimizer else dict(exp_avg=master, exp_avg_sq=master)
            self.engine.add_shard(master, chunk.shard, chunk.valid_end, segments[chunk], **moments)
        self.engine.finalize()
        if self.engine.table.host_resident:
            # shards in host memory: the update moves them through device staging sets with the copy engines
            # (measured faster than letting the kernel reach them over PCIe)
            self.engine.enable_streaming()
        for index, chunk in enumerate(chunks):
            chunk.bind_control(self.engine.ctl, self.engine.chunk_flags[index:index + 1])
        self._index_of = {chunk.paired_chunk: i for i, chunk in enumerate(chunks)}
        if not self.scaled_optimizer:
            if self.engine.table.host_resident or self.module.nvlink_step:
                raise RuntimeError(f'{type(self.optim).__name__} is stepped by torch on device-resident shards over '
                                   f'NCCL; use an optimizer of {_AVAIL_OPTIM_LIST} for other placements')
            return
        self.optim.bind_engine(self.engine)
        self.engine.set_hyper(self.optim.hyper_table())
        # per-parameter views of the flat moments, under the keys the reference's optimizers use
        for fake, (begin, end) in self.param_to_range.items():
            _, exp_avg, exp_avg_sq, _, _ = self.engine.shards[self._index_of[self.param_to_optim_chunk[fake]]]
            self.optim.state[fake] = dict(step=0, exp_avg=exp_avg[begin:end], exp_avg_sq=exp_avg_sq[begin:end])

    def _zero_step(self):
        """One step with zero gradients before training (``__zero_step``, ``:94-113``).  The reference uses
        it to allocate optimizer state early; its side effects — the step count becomes 1 and decoupled
        weight decay is applied once — are reproduced."""
        for _, _, _, lowp, _ in self.engine.shards:
            lowp.zero_()
        if not self.scaled_optimizer:
            self._step_foreign(decided=False)
            return
        ctl = self.engine.read_control()
        ctl.skip, ctl.div_scale, ctl.inv_div = 0, -1.0, 0.0
        ctl.step += 1
        self.engine.ctl.write(ctl)
        self.optim.step()
        self.zero_grad()

    # ------------------------------------------------------------------ optimizer protocol

    @property
    def param_groups(self):
        return self.optim.param_groups

    @property
    def state(self):
        """Per-parameter optimizer state.  ``step`` is the number of applied updates, kept in the device control
        block; it is copied into the per-parameter entries when the state is looked at (this property and
        ``state_dict``), which waits for the device, and never during ``step()``."""
        self._refresh_step_counts()
        return self.optim.state

    def _refresh_step_counts(self):
        if not self.scaled_optimizer:
            return
        applied = int(self.engine.read_control().step)
        for fake in self.param_to_range:
            entry = self.optim.state.get(fake)
            if entry is not None:
                entry['step'] = applied

    @property
    def defaults(self):
        return self.optim.defaults

    def zero_grad(self, *args, **kwargs):
        return self.optim.zero_grad(set_to_none=True)

    @property
    def loss_scale(self) -> float:
        """Current loss scale as a Python float.  Synchronises (the reference does too, ``:185-187``);
        ``backward`` does not use it."""
        self.engine.check_status()    # the host waits for the device here anyway: report what the kernels flagged
        return float(self.grad_scaler.scale.item())

    def _check_overflow(self) -> bool:
        """Whether any chunk of this rank flagged inf/nan.  Synchronises; the step itself does not call it."""
        return bool(self.engine.chunk_flags.any().item())

    def _attach_nvlink(self):
        """First NVLink step: every chunk sits in a block of the peer-mapped replica cache by now; remember
        where, and from here on the chunks keep their blocks (the step leaves them gathered)."""
        offsets = []
        for chunk in self._chunks:
            assert chunk.is_replica and chunk.rcb is not None and chunk.rcb.slab_offset is not None, \
                'NVLink step: run forward/backward (or inject_gradients) before the first step'
            offsets.append(chunk.rcb.slab_offset)
        self.engine.attach_p2p(self.param_chunk_group.rcache.slab, offsets)
        self._nvlink_offsets = offsets

    def step(self, *args, **kwargs):
        self.optim_state = OptimState.UNSCALED
        if self.module.nvlink_step:
            if getattr(self, '_nvlink_offsets', None) is None:
                self._attach_nvlink()
            assert [c.rcb.slab_offset for c in self._chunks] == self._nvlink_offsets
            self.engine.set_hyper(self.optim.hyper_table())
            self.engine.step_sharded_p2p()
            for chunk in self._chunks:
                chunk._l2_valid = False
            self.zero_grad()
            return None
        self.engine.begin_step()
        if self.scaled_optimizer:
            ret = self.optim.step(*args, **kwargs)
        else:
            ret = self._step_foreign(True, *args, **kwargs)
        self.engine.end_step()
        for chunk in self._chunks:
            chunk._l2_valid = False
        self.zero_grad()
        return ret

    def _step_foreign(self, decided: bool, *args, **kwargs):
        """Step an optimizer that is not in the available list (``:211-214``): bind, for every parameter range of
        this rank, ``.data`` to the fp32 shard view and ``.grad`` to the gradient view (``_set_grad_ptr``,
        ``:115-124``), let torch step, unbind, refresh the working copies (``_update_fp16_params``, ``:126-135``).
        ``decided``: ``elx_step_begin`` has run; its decision is read back here (one synchronisation per step)."""
        ret, skip = None, False
        if decided:
            ctl = self.engine.read_control()
            skip = bool(ctl.skip)
            if not skip and ctl.div_scale != -1.0:
                raise AssertionError(f'You should use an optimizer in the available list:\n{_AVAIL_OPTIM_LIST}')
        if not skip:
            for fake, (begin, end) in self.param_to_range.items():
                master, _, _, lowp, _ = self.engine.shards[self._index_of[self.param_to_optim_chunk[fake]]]
                grad = lowp[begin:end]
                fake.data = master[begin:end]
                fake.grad = grad if grad.dtype == master.dtype else grad.to(master.dtype)
            ret = self.optim.step(*args, **kwargs)
        none_tensor = torch.empty([0], device=self.engine.device)
        for fake in self.param_to_range:
            fake.grad = None
            fake.data = none_tensor
        for chunk in self._chunks:
            chunk.optim_update()
        return ret

    def clip_grad_norm(self, model: torch.nn.Module, max_norm: float, norm_type: float = 2.0):
        raise NotImplementedError

    def backward(self, loss: torch.Tensor):
        # fp32 product with the device-resident scale: no host read, and 2^16 does not overflow a half loss
        loss = loss.float() * self.grad_scaler.scale
        self.optim_state = OptimState.SCALED
        self.module.backward(loss)

    def backward_by_grad(self, tensor: torch.Tensor, grad: torch.Tensor):
        self.optim_state = OptimState.SCALED
        self.module.backward_by_grad(tensor, grad)

    # ------------------------------------------------------------------ checkpoint

    def state_dict(self):
        """This rank's flat optimizer state: one (exp_avg, exp_avg_sq) pair per chunk shard plus the control
        block fields.  The reference saves none of this (its scaler state is lost on restart)."""
        self._quiesce_host_shards()
        self.engine.check_status()
        if not self.scaled_optimizer:
            return dict(scaler=self.grad_scaler.state_dict(), optim=self.optim.state_dict())
        self._refresh_step_counts()
        return dict(scaler=self.grad_scaler.state_dict(),
                    shards=[dict(exp_avg=s[1].detach().to('cpu', copy=True), exp_avg_sq=s[2].detach().to('cpu', copy=True))
                            for s in self.engine.shards],
                    param_groups=[{k: v for k, v in g.items() if k != 'params'} for g in self.optim.param_groups])

    def _quiesce_host_shards(self):
        """Shards in host memory are written by kernels and read here by plain host copies, which no stream
        orders: wait for the device first."""
        if self.engine.table.host_resident:
            torch.cuda.synchronize(self.engine.device)

    def load_state_dict(self, state):
        self._quiesce_host_shards()
        self.grad_scaler.load_state_dict(state['scaler'])
        if not self.scaled_optimizer:
            self.optim.load_state_dict(state['optim'])
            return
        for shard, saved in zip(self.engine.shards, state['shards']):
            shard[1].copy_(saved['exp_avg'])
            shard[2].copy_(saved['exp_avg_sq'])
        for group, saved in zip(self.optim.param_groups, state['param_groups']):
            group.update(saved)
