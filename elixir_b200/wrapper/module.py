"""ElixirModule: packs a model's parameters into paired chunks and lands gradients in them.

Mirror of ``elixir/wrapper/module.py`` for the parts the optimizer step relies on:

* ``__init_chunk_group`` (``module.py:77-138``): for every plan a low-precision *param chunk* and an
  fp32 *optim chunk* with identical size and tensor offsets, closed (each rank keeps its shard) and
  paired (``Chunk.init_pair``);
* ``_gradient_handler`` (``module.py:177-190``): an autograd hook per parameter that copies the gradient
  into the chunk's replicated block and, once every tensor of the chunk has its gradient, reduces the
  chunk (rank average -> shard, fused with the inf/nan probe).

Residency during forward / backward comes in two forms, chosen by the replica cache of the plan:

* a block for every public chunk (what ``simple_plan`` allocates by default): all chunks are gathered
  before forward and stay gathered until their reduce;
* fewer blocks than public chunks (``simple_plan(..., public_block_number=k)`` or ``allocate_factor < 1``):
  *scheduled* residency.  The reference intercepts every torch function that touches a parameter
  (``elixir/hook/parameter.py``); here the unit is the sub-module that owns parameters: a forward
  pre-hook fetches the chunks of its parameters, a forward hook marks them held again (so the scheduler may
  release them), a hook on the gradients of its outputs fetches them again before its backward runs, and
  the post-accumulate hook of each parameter lands the gradient and reduces the chunk when complete.
  Which resident chunk makes room is the scheduler's choice (``FIFOScheduler``; with ``prefetch=True``
  ``PrefetchScheduler``, which also gathers ahead on a side stream).  Tensors that autograd saves for
  backward and that alias a block (a parameter, or a view of one such as ``weight.t()``) are saved as
  (chunk, offset, shape, strides) and rebuilt on the block the chunk occupies when backward needs them,
  because a chunk may come back into a different block.
  Limits: a parameter must be used through the module that owns it (or be shared, which gives it a
  private, always resident chunk); every parameter must receive a gradient in every backward pass.
"""
import weakref
from bisect import bisect_right
from collections import OrderedDict
from copy import copy
from functools import partial
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import comm
from ..chunk import ChunkFetcher, ChunkGroup, FIFOScheduler, MemoryPool, PrefetchScheduler, TensorState
from .plan import SearchResult


def get_param_optim_data(param_data: torch.Tensor, param_dtype: torch.dtype, device):
    """Low-precision working copy and fp32 master of one parameter (``module.py:21-25``)."""
    param_data = param_data.to(device)
    optim_data = param_data.clone() if param_data.dtype == torch.float else param_data.float()
    return param_data.to(param_dtype), optim_data


class _MovedAlias:
    """A tensor saved for backward that aliased a replica-cache block: where in which chunk it lives."""
    __slots__ = ('chunk', 'offset', 'shape', 'stride')

    def __init__(self, chunk, offset, shape, stride):
        self.chunk, self.offset, self.shape, self.stride = chunk, offset, shape, stride


def _tensors_of(obj):
    if isinstance(obj, torch.Tensor):
        yield obj
    elif isinstance(obj, (list, tuple)):
        for o in obj:
            yield from _tensors_of(o)
    elif isinstance(obj, dict):
        for o in obj.values():
            yield from _tensors_of(o)
    elif hasattr(obj, '__dataclass_fields__'):
        for name in obj.__dataclass_fields__:
            yield from _tensors_of(getattr(obj, name, None))


class ElixirModule(nn.Module):

    def __init__(self,
                 module: nn.Module,
                 search_result: SearchResult,
                 process_group,
                 prefetch: bool = False,
                 dtype: torch.dtype = torch.float,
                 reduce_always_fp32: bool = False,
                 output_fp32: bool = False,
                 use_fused_kernels: bool = False,
                 residency: Optional[str] = None) -> None:
        """Arguments as ``elixir.wrapper.ElixirModule`` (``module.py:40-48``).  ``residency`` (not in the
        reference): ``'all'``, ``'scheduled'`` or None = scheduled exactly when the replica cache has fewer
        public blocks than there are public chunks."""
        super().__init__()
        # the reference accepts float and float16 (module.py:51); bfloat16 is an extension that runs with
        # a constant loss scale of 1
        assert dtype in {torch.float, torch.float16, torch.bfloat16}
        self.module = module
        self.dtype = dtype
        self.use_amp = dtype == torch.float16
        self.process_group = process_group
        self.prefetch_flag = prefetch
        self.reduce_always_fp32 = reduce_always_fp32
        self.output_fp32 = output_fp32
        self.use_fused_kernels = use_fused_kernels

        self.no_grad_state_dict: Dict[str, torch.Tensor] = dict()
        self.grad_state_dict: Dict[str, torch.Tensor] = dict()
        self._init_chunk_group(search_result)
        pool = search_result.chunk_group.rcache
        # replica cache in peer-mapped memory and more than one rank: the optimizer step does the collectives
        self.nvlink_step = getattr(pool, 'slab', None) is not None and dist.get_world_size(process_group) > 1
        if self.nvlink_step and reduce_always_fp32:
            raise ValueError('the NVLink step always accumulates in fp32; drop reduce_always_fp32')
        n_public = len(self.param_chunk_group.float_chunks)
        assert residency in (None, 'all', 'scheduled')
        if residency is None:
            residency = 'scheduled' if pool.public_free_cnt < n_public else 'all'
        if residency == 'all' and pool.public_free_cnt < n_public:
            raise ValueError(f'{n_public} public chunks do not fit {pool.public_free_cnt} blocks without scheduling')
        self.scheduled = residency == 'scheduled'
        self._reduced: set = set()    # chunks reduced in the running backward pass
        if self.scheduled and self.nvlink_step:
            raise ValueError('the NVLink step keeps every chunk in its block; give the plan a block per chunk')
        self._init_chunk_fetcher(search_result, prefetch)

        # The hook fires once per backward, after autograd has summed every use of the parameter.  It reaches this
        # object through a weak reference: the tensor keeps its hooks on the C++ side, where the garbage collector
        # cannot follow a parameter -> hook -> wrapper -> parameter cycle, and the whole model would never be freed.
        me = weakref.ref(self)

        def landed(param):
            wrapper = me()
            if wrapper is not None:
                wrapper._post_accumulate(param)

        for name, param in module.named_parameters():
            if not param.requires_grad:
                continue
            param.register_post_accumulate_grad_hook(landed)
        if self.scheduled:
            self._install_residency_hooks()

    # ------------------------------------------------------------------ construction

    def _device(self, sr: SearchResult):
        dev = sr.chunk_group.rcache.device_type
        if str(dev) == 'cuda':
            return torch.device('cuda', torch.cuda.current_device())
        return torch.device(dev)

    def _init_chunk_group(self, sr: SearchResult):
        device = self._device(sr)
        for name, tensor in self.module.state_dict(keep_vars=True).items():
            if isinstance(tensor, nn.Parameter):
                assert tensor.is_floating_point(), 'the dtypes of parameters should be float dtypes'
                if tensor.requires_grad:
                    self.grad_state_dict[name] = tensor
                else:
                    self.no_grad_state_dict[name] = tensor
                    tensor.data = tensor.data.to(dtype=self.dtype, device=device)
            else:
                to_dtype = self.dtype if tensor.is_floating_point() else tensor.dtype
                tensor.data = tensor.data.to(dtype=to_dtype, device=device)

        empty_pool = MemoryPool(sr.chunk_group.rcache.device_type)
        empty_pool.allocate()
        self.param_chunk_group: ChunkGroup = sr.chunk_group
        self.optim_chunk_group = ChunkGroup(empty_pool)
        self.param_to_optim = dict()
        seen = set()
        for plan in sr.param_chunk_plans:
            assert plan.chunk_dtype == self.dtype
            optim_kwargs = copy(plan.kwargs)
            optim_kwargs.pop('rcache_fused', None)
            p_chunk = self.param_chunk_group.open_chunk(plan.chunk_size, plan.chunk_dtype, self.process_group,
                                                        plan.kwargs)
            o_chunk = self.optim_chunk_group.open_chunk(plan.chunk_size, torch.float, self.process_group,
                                                        optim_kwargs)
            for name in plan.name_list:
                param = self.grad_state_dict[name]
                param_data, optim_data = get_param_optim_data(param.data, self.dtype, device)
                param.data = param_data
                p_chunk.append_tensor(param)
                o_chunk.append_tensor(optim_data)
                self.param_to_optim[param] = optim_data
                seen.add(param)
            self.param_chunk_group.close_chunk(p_chunk)
            self.optim_chunk_group.close_chunk(o_chunk)
            p_chunk.init_pair(o_chunk)
        for param in self.module.parameters():
            if param.requires_grad:
                assert param in seen, 'a parameter that requires grad is missing from the chunk plans'

    def _init_chunk_fetcher(self, sr: SearchResult, prefetch: bool):
        """``module.py:140-163``: Belady scheduling on the plan's access trace with ``prefetch``, FIFO
        otherwise.  A plan without a trace makes the scheduler learn it from the first iteration."""
        scheduler = None
        if self.scheduled:
            if prefetch:
                trace = None
                if sr.param_called_per_step is not None:
                    trace = []
                    for names in sr.param_called_per_step:
                        params = [self.grad_state_dict[n] for n in names if n in self.grad_state_dict]
                        trace.append({self.param_chunk_group.ten_to_chunk[p] for p in params})
                scheduler = PrefetchScheduler(trace)
            else:
                scheduler = FIFOScheduler()
        self.fetcher = ChunkFetcher(scheduler, self.param_chunk_group, overlap=prefetch,
                                    reduce_always_fp32=self.reduce_always_fp32)
        # public blocks by position in the pool's slab: lets a saved tensor be traced back to its chunk
        pool = sr.chunk_group.rcache
        slab = getattr(pool, '_public_slab', None)
        self._slab_ptr = slab.untyped_storage().data_ptr() if (self.scheduled and slab is not None) else None
        self._slab_device = slab.device if slab is not None else None
        self._slab_blocks = sorted(pool.public_free_blocks or [], key=lambda b: b.slab_offset) if self.scheduled else []
        self._slab_starts = [b.slab_offset for b in self._slab_blocks]

    @property
    def param_chunks(self):
        group = self.param_chunk_group
        return sorted(group.fused_chunks | group.float_chunks, key=lambda c: c.chunk_id)

    # ------------------------------------------------------------------ gradients

    def _post_accumulate(self, param: nn.Parameter):
        grad, param.grad = param.grad, None    # the gradient moves into the chunk; nothing stays on the parameter
        self._gradient_handler(grad, param)

    def _gradient_handler(self, grad: torch.Tensor, param: nn.Parameter):
        chunk = self.fetcher.get_one_chunk(param)
        if self.scheduled:
            state = chunk.tensors_info[param].state
            if state == TensorState.HOLD:    # nothing announced this parameter's backward: fetch its chunk now
                self._fetch([param])
                state = TensorState.COMPUTE
            if state == TensorState.COMPUTE:
                self.param_chunk_group.tensor_trans_state(param, TensorState.HOLD_AFTER_BWD)
        assert self.param_chunk_group.is_accessed(chunk)
        if chunk.tensors_info[param].state != TensorState.HOLD_AFTER_BWD:
            raise RuntimeError('a gradient arrived for a parameter that is not waiting for one')
        self.param_chunk_group.tensor_trans_state(param, TensorState.READY_FOR_REDUCE)
        chunk.copy_tensor_to_chunk_slice(param, grad)
        if self.nvlink_step:
            if chunk.reduce_check:
                chunk.defer_reduce()
        elif self.fetcher.reduce_chunk(chunk):
            self._reduced.add(chunk)

    def inject_gradients(self, grads: Dict[str, torch.Tensor]):
        """Drive the backward tail without running a model: gather the chunks, hand every parameter its
        gradient (by name) exactly as the autograd hook would, which reduces each chunk when complete."""
        self._reduced = set()
        if self.scheduled:
            with torch.no_grad():    # not a pass a learning scheduler should take for the model's access trace
                self.fetcher.reset()
                for param, grad in self._unique_grads(grads):
                    self._gradient_handler(grad, param)
                self._end_backward()
            return
        self._gather_all()
        self._set_states(TensorState.COMPUTE)
        self._set_states(TensorState.HOLD_AFTER_BWD)
        for param, grad in self._unique_grads(grads):
            self._gradient_handler(grad, param)
        self._end_backward()

    def _unique_grads(self, grads: Dict[str, torch.Tensor]):
        """(parameter, gradient) once per parameter; a shared parameter is listed under each of its names in the
        state dict and takes the gradient given under any of them."""
        names: Dict[nn.Parameter, List[str]] = dict()
        for name, param in self.grad_state_dict.items():
            names.setdefault(param, []).append(name)
        for param, aliases in names.items():
            given = [n for n in aliases if n in grads]
            if not given:
                raise KeyError(f'no gradient for {aliases[0]}')
            yield param, grads[given[0]].to(self.dtype)

    # ------------------------------------------------------------------ forward / backward

    def _gather_all(self):
        for chunk in self.param_chunks:
            self.param_chunk_group.access_chunk(chunk)

    def _set_states(self, state: TensorState):
        for chunk in self.param_chunks:
            for tensor in chunk.get_tensors():
                chunk.tensor_trans_state(tensor, state)

    def _cast_inputs(self, obj: Any):
        if isinstance(obj, torch.Tensor) and obj.is_floating_point():
            return obj.to(self.dtype)
        if isinstance(obj, (list, tuple)):
            return type(obj)(self._cast_inputs(o) for o in obj)
        if isinstance(obj, dict):
            return {k: self._cast_inputs(v) for k, v in obj.items()}
        return obj

    def forward(self, *args, **kwargs):
        args, kwargs = self._cast_inputs(args), self._cast_inputs(kwargs)
        self._reduced = set()
        if self.scheduled:
            self.fetcher.reset()
            with self._saved_tensor_hooks():
                outputs = self.module(*args, **kwargs)
            if not torch.is_grad_enabled():
                self.fetcher.release_all()
                self.fetcher.clear()
        else:
            self._gather_all()
            self._set_states(TensorState.COMPUTE)
            outputs = self.module(*args, **kwargs)
            if not torch.is_grad_enabled():
                self._set_states(TensorState.HOLD)
        if self.output_fp32:
            outputs = outputs.float() if isinstance(outputs, torch.Tensor) else outputs
        return outputs

    def backward(self, loss: torch.Tensor):
        self.backward_by_grad(loss, None)

    def backward_by_grad(self, tensor: torch.Tensor, grad: torch.Tensor):
        if self.scheduled:
            with self._saved_tensor_hooks():    # a recomputed (checkpointed) forward saves tensors too
                torch.autograd.backward(tensor, grad)
        else:
            self._set_states(TensorState.HOLD_AFTER_BWD)
            torch.autograd.backward(tensor, grad)
        self._end_backward()

    def _end_backward(self):
        if self.scheduled:
            missing = [n for n, p in self.grad_state_dict.items() if self.fetcher.get_one_chunk(p) not in self._reduced]
            if missing:
                raise RuntimeError('no gradient arrived for: ' + ', '.join(missing[:8]) +
                                   (' ...' if len(missing) > 8 else ''))
        self.fetcher.clear()

    # ------------------------------------------------------------------ scheduled residency

    def _install_residency_hooks(self):
        for sub in self.module.modules():
            params = [p for p in sub.parameters(recurse=False) if p.requires_grad]
            if not params:
                continue
            sub.register_forward_pre_hook(partial(self._pre_forward, params))
            sub.register_forward_hook(partial(self._post_forward, params))

    def _fetch(self, params: List[nn.Parameter]):
        chunks = self.fetcher.trans_to_compute(params)
        self.fetcher.fetch_chunks(chunks)

    def _pre_forward(self, params, module, args):
        self._fetch(params)

    def _post_forward(self, params, module, args, output):
        self.fetcher.trans_to_hold(params, phase='f')
        if torch.is_grad_enabled():
            announce = partial(self._pre_backward, params)
            for t in _tensors_of(output):
                if t.requires_grad:
                    t.register_hook(announce)

    def _pre_backward(self, params, grad):
        """The gradient of one of the sub-module's outputs is known: its backward is about to run."""
        info = lambda p: self.fetcher.get_one_chunk(p).tensors_info[p]    # noqa: E731
        waiting = [p for p in params
                   if info(p).state in (TensorState.HOLD, TensorState.HOLD_AFTER_BWD)
                   and self.fetcher.get_one_chunk(p) not in self._reduced]
        if waiting:
            self._fetch(waiting)
        return None

    def _saved_tensor_hooks(self):
        return torch.autograd.graph.saved_tensors_hooks(self._pack_saved, self._unpack_saved)

    def _pack_saved(self, t: torch.Tensor):
        if (self._slab_ptr is not None and t.layout == torch.strided and t.device == self._slab_device
                and t.untyped_storage().data_ptr() == self._slab_ptr):
            offset = t.storage_offset()
            i = bisect_right(self._slab_starts, offset) - 1
            if i >= 0:
                block = self._slab_blocks[i]
                if block.owner is not None and offset < block.slab_offset + block.numel:
                    return _MovedAlias(block.owner, offset - block.slab_offset, tuple(t.shape), tuple(t.stride()))
        return t

    def _unpack_saved(self, packed):
        if isinstance(packed, _MovedAlias):
            chunk = packed.chunk
            assert chunk.is_replica, 'backward needs a parameter whose chunk is not resident'
            payload = chunk.rcb.payload
            return payload.as_strided(packed.shape, packed.stride, payload.storage_offset() + packed.offset)
        return packed

    # ------------------------------------------------------------------ checkpoint

    def state_dict(self, destination=None, prefix='', keep_vars=False, only_rank_0: bool = False, from_param: bool = False):
        """Full tensors on the CPU, from the fp32 masters unless ``from_param`` (``module.py:258-292``)."""
        assert not keep_vars
        out = destination if destination is not None else OrderedDict()
        collected = dict()
        for p_chunk in self.param_chunks:
            source = p_chunk if from_param else p_chunk.paired_chunk
            for tensor, copy_ in zip(p_chunk.get_tensors(), source.get_cpu_copy(only_rank_0)):
                collected[tensor] = copy_
        for name, tensor in self.module.state_dict(keep_vars=True).items():
            if name in self.grad_state_dict:
                out[prefix + name] = collected[self.grad_state_dict[name]]
            else:
                out[prefix + name] = tensor.detach().cpu()
        return out

    def load_state_dict(self, state_dict, only_rank_0: bool = False):
        """Load full tensors into the fp32 masters and refresh the low-precision shards
        (``module.py:294-344``)."""
        for p_chunk in self.param_chunks:
            o_chunk = p_chunk.paired_chunk
            loads = []
            for tensor in p_chunk.get_tensors():
                # a shared parameter appears under several names; any of them that the state dict holds will do
                aliases = [n for n, q in self.grad_state_dict.items() if q is tensor]
                held = [n for n in aliases if state_dict is not None and n in state_dict]
                loads.append(state_dict[held[0]].float() if held else None)
            o_chunk.load_tensors(loads, only_rank_0)
            p_chunk.optim_update()
            if p_chunk.is_replica:    # the chunk is gathered (e.g. left so by the NVLink step): refresh the replica too
                comm.all_gather(p_chunk.rcb.payload, p_chunk.shard, p_chunk.torch_pg)
        for name, tensor in self.no_grad_state_dict.items():
            if state_dict is not None and name in state_dict:
                tensor.data.copy_(state_dict[name])
