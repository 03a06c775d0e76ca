"""ElixirModule: packs a model's parameters into paired chunks and lands gradients in them.

Mirror of ``elixir/wrapper/module.py`` for the parts the optimizer step relies on:

* ``__init_chunk_group`` (``module.py:77-138``): for every plan a low-precision *param chunk* and an
  fp32 *optim chunk* with identical size and tensor offsets, closed (each rank keeps its shard) and
  paired (``Chunk.init_pair``);
* ``_gradient_handler`` (``module.py:177-190``): an autograd hook per parameter that copies the gradient
  into the chunk's replicated block and, once every tensor of the chunk has its gradient, reduces the
  chunk (rank average -> shard, fused with the inf/nan probe).

Forward / backward residency is deliberately simple here: all chunks are gathered before forward and
stay gathered until their reduce, so no per-operator fetching (the reference's HookParam machinery) is
needed; that machinery is outside the optimizer-step path.
"""
from collections import OrderedDict
from copy import copy
from typing import Any, Dict

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import comm
from ..chunk import ChunkFetcher, ChunkGroup, MemoryPool, TensorState
from .plan import SearchResult


def get_param_optim_data(param_data: torch.Tensor, param_dtype: torch.dtype, device):
    """Low-precision working copy and fp32 master of one parameter (``module.py:21-25``)."""
    param_data = param_data.to(device)
    optim_data = param_data.clone() if param_data.dtype == torch.float else param_data.float()
    return param_data.to(param_dtype), optim_data


class ElixirModule(nn.Module):

    def __init__(self,
                 module: nn.Module,
                 search_result: SearchResult,
                 process_group,
                 prefetch: bool = False,
                 dtype: torch.dtype = torch.float,
                 reduce_always_fp32: bool = False,
                 output_fp32: bool = False,
                 use_fused_kernels: bool = False) -> None:
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
        self.fetcher = ChunkFetcher(self.param_chunk_group, overlap=prefetch, reduce_always_fp32=reduce_always_fp32)

        for name, param in module.named_parameters():
            if not param.requires_grad:
                continue
            # fires once per backward, after autograd has summed every use of the parameter
            param.register_post_accumulate_grad_hook(self._post_accumulate)

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
        assert self.param_chunk_group.is_accessed(chunk)
        if chunk.tensors_info[param].state != TensorState.HOLD_AFTER_BWD:
            raise RuntimeError('a gradient arrived for a parameter that is not waiting for one')
        self.param_chunk_group.tensor_trans_state(param, TensorState.READY_FOR_REDUCE)
        chunk.copy_tensor_to_chunk_slice(param, grad)
        if self.nvlink_step:
            if chunk.reduce_check:
                chunk.defer_reduce()
        else:
            self.fetcher.reduce_chunk(chunk)

    def inject_gradients(self, grads: Dict[str, torch.Tensor]):
        """Drive the backward tail without running a model: gather the chunks, hand every parameter its
        gradient (by name) exactly as the autograd hook would, which reduces each chunk when complete."""
        self._gather_all()
        self._set_states(TensorState.COMPUTE)
        self._set_states(TensorState.HOLD_AFTER_BWD)
        for name, param in self.grad_state_dict.items():
            self._gradient_handler(grads[name].to(self.dtype), param)
        self.fetcher.clear()

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
        self._gather_all()
        self._set_states(TensorState.COMPUTE)
        args, kwargs = self._cast_inputs(args), self._cast_inputs(kwargs)
        outputs = self.module(*args, **kwargs)
        if self.output_fp32:
            outputs = outputs.float() if isinstance(outputs, torch.Tensor) else outputs
        if not torch.is_grad_enabled():
            self._set_states(TensorState.HOLD)
        return outputs

    def backward(self, loss: torch.Tensor):
        self._set_states(TensorState.HOLD_AFTER_BWD)
        loss.backward()
        self.fetcher.clear()

    def backward_by_grad(self, tensor: torch.Tensor, grad: torch.Tensor):
        self._set_states(TensorState.HOLD_AFTER_BWD)
        torch.autograd.backward(tensor, grad)
        self.fetcher.clear()

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
            names = [n for t in p_chunk.get_tensors() for n, q in self.grad_state_dict.items() if q is t]
            loads = [state_dict[n].float() if state_dict is not None and n in state_dict else None for n in names]
            o_chunk.load_tensors(loads, only_rank_0)
            p_chunk.optim_update()
            if p_chunk.is_replica:    # the chunk is gathered (e.g. left so by the NVLink step): refresh the replica too
                comm.all_gather(p_chunk.rcb.payload, p_chunk.shard, p_chunk.torch_pg)
        for name, tensor in self.no_grad_state_dict.items():
            if state_dict is not None and name in state_dict:
                tensor.data.copy_(state_dict[name])
