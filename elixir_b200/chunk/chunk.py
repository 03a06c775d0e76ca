"""A chunk: a flat buffer that packs tensors back to back and is sharded over a process group.

Host-side mirror of ``elixir/chunk/core/chunk.py`` (same constructor, attributes and methods for the
optimizer path), with the device work routed through the sm_100a kernels:

* ``reduce``: rank-average reduce-scatter, then ONE pass that copies the reduced slice into the
  persistent shard and probes it for inf/nan (``elx_reduce_epilogue``) — the reference runs a divide
  pass, the collective, a copy and two isinf/isnan passes with two host syncs (``chunk.py:282-315,
  214-216``);
* ``overflow`` / ``l2_norm`` live in device words and are read by the step on the device; reading
  them from Python synchronises and is meant for tests and logging;
* ``optim_update``: fp32 -> low-precision copy-back kernel (``chunk.py:403-415``).

Geometry is the reference's: ``shard = chunk[rank * S:(rank + 1) * S]`` with ``S = chunk_size / W``
(``chunk.py:72-77``); ``valid_end`` = used elements inside this rank's shard (``chunk.py:253-257``).
"""
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import comm, kernels
from .memory_pool import MemoryPool, TensorBlock
from .states import TensorState, ts_update_sanity_check


class ChunkFullError(Exception):
    pass


@dataclass
class TensorInfo:
    state: TensorState
    fake_data: torch.Tensor
    offset: int
    end: int


def _placeholder(t: torch.Tensor) -> torch.Tensor:
    """Storage-free stand-in with the tensor's shape, dtype and device (one element, expanded)."""
    return torch.zeros(1, dtype=t.dtype, device=t.device).expand(t.shape)


class Chunk:
    total_count = 0

    def __init__(self,
                 rcache: MemoryPool,
                 chunk_size: int,
                 chunk_dtype: torch.dtype,
                 process_group,
                 temp_device: Optional[torch.device] = None,
                 shard_device: Optional[torch.device] = None,
                 rcache_fused: bool = False,
                 cpu_pin_memory: bool = False) -> None:
        self.chunk_id = Chunk.total_count
        Chunk.total_count += 1
        self.rcache = rcache
        self.chunk_size = chunk_size
        self.chunk_dtype = chunk_dtype
        self.utilized_size = 0

        self.torch_pg = process_group
        self.pg_size = dist.get_world_size(process_group)
        self.pg_rank = dist.get_rank(process_group)
        if chunk_size % self.pg_size != 0:
            raise ValueError(f'chunk_size {chunk_size} is not divisible by the group size {self.pg_size}')
        self.shard_size = chunk_size // self.pg_size
        self.shard_begin = self.shard_size * self.pg_rank
        self.shard_end = self.shard_begin + self.shard_size
        self.valid_end = self.shard_size + 1    # illegal until close_chunk()

        self.rcb: Optional[TensorBlock] = None
        self.rcache_fused = rcache_fused
        self._my_block = rcache.get_private_block(chunk_size, chunk_dtype) if rcache_fused else None
        self.is_replica = True

        default_device = torch.device(rcache.device_type)
        if default_device.type == 'cuda' and default_device.index is None:
            default_device = torch.device('cuda', torch.cuda.current_device())
        temp_device = torch.device(temp_device) if temp_device is not None else default_device
        shard_device = torch.device(shard_device) if shard_device is not None else default_device
        if rcache_fused:
            self.chunk_temp = self._my_block.payload
            self.chunk_temp.zero_()
        else:
            self.chunk_temp = torch.zeros(chunk_size, dtype=chunk_dtype, device=temp_device)
        # where the kernels that touch this chunk run: the shard's device, or -- for a shard kept in host
        # memory beside a replica cache on a GPU (the reference's shard_device=cpu placement) -- that GPU;
        # such a shard is always page-locked, because the kernels reach it through its mapped address
        host_resident = shard_device.type == 'cpu' and default_device.type == 'cuda'
        self.compute_device = default_device if host_resident else shard_device
        pin = (cpu_pin_memory or host_resident) and shard_device.type == 'cpu'
        self.shard = torch.empty(self.shard_size, dtype=chunk_dtype, device=shard_device, pin_memory=pin)
        self.host_resident = host_resident

        self.chunk_memo = chunk_size * self.chunk_temp.element_size()
        self.shard_memo = self.chunk_memo // self.pg_size

        self.tensors_info: Dict[torch.Tensor, TensorInfo] = {}
        self.num_tensors = 0
        self.tensor_state_cnter: Dict[TensorState, int] = {state: 0 for state in TensorState}

        self.paired_chunk: Optional['Chunk'] = None
        self.optim_sync_flag = True
        self.l2_norm_flag = False

        # probe results on the device: [0] overflow word; l2: sum of squares of the reduced gradients
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.compute_device)
        self._l2sq = torch.zeros(1, dtype=torch.float32, device=self.compute_device)
        self._l2_valid = False
        self._l2_scratch = None
        self._ctl = None    # ControlBlock of the optimizer that steps this chunk (set by bind_control)
        self._probed = False
        self.ready_event = None    # set by a gather issued ahead of time on a side stream; its consumer waits on it

    # ------------------------------------------------------------------ properties

    @property
    def prepared_block(self):
        return self._my_block

    @property
    def is_init(self) -> bool:
        return self.chunk_temp is not None

    @property
    def in_rcache(self) -> bool:
        return self.rcb is not None

    @property
    def shard_device(self) -> torch.device:
        return self.shard.device

    @property
    def memory_usage(self) -> Dict[str, int]:
        usage = dict(cuda=0, cpu=0)
        if self.is_init:
            usage[self.chunk_temp.device.type] += self.chunk_memo
        if self.in_rcache:
            usage['cuda' if self.rcb.payload.is_cuda else 'cpu'] += self.rcb.memo_occ
        usage[self.shard_device.type] += self.shard_memo
        return usage

    @property
    def payload(self) -> torch.Tensor:
        if self.is_init:
            return self.chunk_temp
        return self.rcb.payload if self.in_rcache else self.shard

    @property
    def shard_move_check(self) -> bool:
        return not self.in_rcache

    @property
    def scatter_check(self) -> bool:
        if self.rcache_fused:
            return False
        idle = sum(self.tensor_state_cnter[s]
                   for s in (TensorState.HOLD, TensorState.HOLD_AFTER_BWD, TensorState.READY_FOR_REDUCE))
        return idle == self.num_tensors

    @property
    def evict_check(self) -> bool:
        """Whether the replica may be dropped for another chunk: every tensor merely held.  Stricter than
        ``scatter_check``: a chunk that already holds gradients of this backward pass in its block (tensors
        in HOLD_AFTER_BWD or READY_FOR_REDUCE) keeps the block until it is reduced, since a scatter would
        lose them."""
        if self.rcache_fused:
            return False
        return self.tensor_state_cnter[TensorState.HOLD] == self.num_tensors

    @property
    def reduce_check(self) -> bool:
        return self.tensor_state_cnter[TensorState.READY_FOR_REDUCE] == self.num_tensors

    @property
    def overflow(self) -> bool:
        """Whether the last reduce found inf/nan in this rank's valid shard.  Reads the device word."""
        return bool(self._flag.item())

    @overflow.setter
    def overflow(self, value: bool):
        self._flag.fill_(1 if value else 0)

    @property
    def l2_norm(self) -> Optional[float]:
        """Sum of squares of this rank's reduced (still scaled) gradients, or None if not computed."""
        return float(self._l2sq.item()) if self._l2_valid else None

    @l2_norm.setter
    def l2_norm(self, value):
        self._l2_valid = value is not None
        if value is not None:
            self._l2sq.fill_(float(value))

    def bind_control(self, ctl, flag_view: torch.Tensor = None, l2_view: torch.Tensor = None):
        """Attach the optimizer's control block (its ``found_inf`` word is raised by every probe of this
        chunk) and, optionally, slots of the optimizer's flag / norm arrays to write the results to."""
        self._ctl = ctl
        if flag_view is not None:
            flag_view.copy_(self._flag)
            self._flag = flag_view
        if l2_view is not None:
            l2_view.copy_(self._l2sq)
            self._l2sq = l2_view

    # ------------------------------------------------------------------ probes

    def _norm_args(self):
        if not self.l2_norm_flag:
            return dict()
        if self._l2_scratch is None:
            self._l2_scratch = torch.empty(kernels.n_tiles(self.shard_size), dtype=torch.float32,
                                           device=self.compute_device)
        self._l2_valid = True
        return dict(l2sq=self._l2sq, scratch=self._l2_scratch)

    def set_overflow_flag(self, valid_tensor: torch.Tensor) -> None:
        kernels.grad_check(valid_tensor, flag=self._flag, ctl=self._ctl)

    def set_l2_norm(self, valid_tensor: torch.Tensor) -> None:
        assert not self._l2_valid, 'you are calculating the l2 norm twice'
        self.l2_norm_flag, keep = True, self.l2_norm_flag
        try:
            kernels.grad_check(valid_tensor, **self._norm_args())
        finally:
            self.l2_norm_flag = keep

    def update_extra_reduce_info(self, block: Optional[TensorBlock]):
        """Probe the reduced gradients ``shard[:valid_end]`` (``chunk.py:345-356``).  A no-op when the
        reduce already fused the probe into its copy."""
        if self.rcache_fused:
            assert block is None
        else:
            assert block is not None
        if self._probed:
            return
        kernels.grad_check(self.shard, n_valid=self.valid_end, flag=self._flag, ctl=self._ctl, **self._norm_args())
        self._probed = True

    # ------------------------------------------------------------------ building

    def append_tensor(self, tensor: torch.Tensor):
        assert self.is_init
        assert tensor.dtype == self.chunk_dtype
        new_size = self.utilized_size + tensor.numel()
        if new_size > self.chunk_size:
            raise ChunkFullError
        slot = self.chunk_temp[self.utilized_size:new_size]
        slot.copy_(tensor.data.flatten())
        tensor.data = slot.view(tensor.shape)
        self.tensors_info[tensor] = TensorInfo(TensorState.HOLD, _placeholder(tensor.data), self.utilized_size,
                                               new_size)
        self.num_tensors += 1
        self.tensor_state_cnter[TensorState.HOLD] += 1
        self.utilized_size = new_size

    def close_chunk(self):
        assert self.is_init
        if self.utilized_size <= self.shard_begin:
            self.valid_end = 0
        elif self.utilized_size < self.shard_end:
            self.valid_end = self.utilized_size - self.shard_begin
        else:
            self.valid_end = self.shard_size
        self._remove_tensors_ptr()
        self._update_shard(self.chunk_temp, self.shard)
        self.is_replica = False
        self.chunk_temp = None

    def init_pair(self, friend_chunk: 'Chunk') -> None:
        if self.paired_chunk is None and friend_chunk.paired_chunk is None:
            self.paired_chunk = friend_chunk
            friend_chunk.paired_chunk = self
        else:
            assert self.paired_chunk is friend_chunk and friend_chunk.paired_chunk is self

    # ------------------------------------------------------------------ gather / scatter

    def replicate(self):
        assert not self.is_replica
        self.is_replica = True
        source = self.shard if self.optim_sync_flag else self._paired_shard()
        self._update_replica(self.rcb.payload, source)
        self._update_tensors_ptr()

    def scatter(self):
        assert not self.rcache_fused
        assert self.is_replica
        self._remove_tensors_ptr()
        if not self.optim_sync_flag:
            self._update_shard(self.rcb.payload, self.shard)
            self.optim_sync_flag = True
        self.is_replica = False

    def access_chunk(self, block: Optional[TensorBlock] = None):
        assert not self.is_init
        assert not self.is_replica
        if self.rcache_fused:
            assert block is None
            self.rcb = self._my_block
        else:
            assert block in self.rcache.public_used_blocks
            assert self.rcb is None
            self.rcb = block
        self.rcb.owner = self
        self.replicate()

    def release_chunk(self) -> TensorBlock:
        assert not self.is_init
        assert self.is_replica
        if self.rcache_fused:
            raise RuntimeError('a fused chunk keeps its private block')
        self.scatter()
        block, self.rcb = self.rcb, None
        return block

    # ------------------------------------------------------------------ reduce

    def reduce(self, always_fp32: bool = False):
        """Average the replicated gradients over the group into this rank's shard and probe them."""
        assert self.is_replica
        self._remove_tensors_ptr()
        payload = self.rcb.payload
        my_slice = payload[self.shard_begin:self.shard_end]
        self._probed = False
        widen = always_fp32 and self.chunk_dtype != torch.float
        if self.pg_size > 1 and not widen and not self.host_resident:
            # the collective writes this rank's average straight into the persistent shard; one read-only
            # pass then probes it
            comm.reduce_scatter_avg(self.shard, payload, self.torch_pg)
            kernels.grad_check(self.shard, n_valid=self.valid_end, flag=self._flag, ctl=self._ctl,
                               **self._norm_args())
        elif self.pg_size > 1 and widen:
            # fp32 accumulation (reduce_always_fp32, ``chunk.py:288-308``): widen the block, average in fp32 inside
            # the collective, then round this rank's slice of the average into the persistent shard and probe the
            # rounded values, in one pass
            wide = torch.empty(self.chunk_size, dtype=torch.float, device=payload.device)
            kernels.widen(payload, wide)
            wide_slice = wide[self.shard_begin:self.shard_end]
            comm.reduce_scatter_avg(wide_slice, wide, self.torch_pg)
            kernels.narrow_epilogue(wide_slice, self.shard, n_valid=self.valid_end, flag=self._flag, ctl=self._ctl)
            norm = self._norm_args()
            if norm:
                kernels.grad_check(self.shard, n_valid=self.valid_end, **norm)
        else:
            if self.pg_size > 1:
                # shard in host memory: the collective cannot write there; it leaves the average in this rank's
                # slice of the block (output aliased inside the input, as the reference does, chunk.py:299-303)
                comm.reduce_scatter_avg(my_slice, payload, self.torch_pg)
            # copy into the persistent shard fused with the inf/nan probe (and the norm when asked for)
            kernels.reduce_epilogue(my_slice, self.shard, n_valid=self.valid_end, flag=self._flag, ctl=self._ctl,
                                    **self._norm_args())
        self._probed = True
        self.is_replica = False

    def defer_reduce(self):
        """NVLink step: all gradients of the chunk are in its replicated block; leave them there (the
        optimizer pulls every rank's slice at step time) and keep the block."""
        assert not self.is_init and self.is_replica and self.reduce_check
        self._update_tensors_state(TensorState.HOLD)
        self._probed = True

    def reduce_chunk(self, always_fp32: bool = False, sync: bool = True) -> Optional[TensorBlock]:
        assert not self.is_init
        assert self.is_replica
        self.reduce(always_fp32=always_fp32)
        self._update_tensors_state(TensorState.HOLD)
        block, self.rcb = self.rcb, None
        if self.rcache_fused:
            block = None
        if sync:
            self.update_extra_reduce_info(block)
        return block

    # ------------------------------------------------------------------ tensor bookkeeping

    def tensor_trans_state(self, tensor: torch.Tensor, tensor_state: TensorState) -> None:
        info = self.tensors_info[tensor]
        if info.state == tensor_state:
            return
        if ts_update_sanity_check(info.state, tensor_state):
            self._set_state(info, tensor_state)

    def copy_tensor_to_chunk_slice(self, tensor: torch.Tensor, data_slice: torch.Tensor) -> None:
        assert self.is_replica
        info = self.tensors_info[tensor]
        slot = self.rcb.payload[info.offset:info.end]
        slot.copy_(data_slice.data.flatten())
        tensor.data = slot.view(tensor.shape)

    def optim_update(self) -> None:
        """Refresh this (low-precision) chunk's shard from its paired fp32 chunk."""
        friend = self.paired_chunk
        assert friend is not None and not friend.is_replica
        assert self.shard_device.type == friend.shard_device.type
        kernels.cast_copyback(friend.shard, self.shard)
        self.optim_sync_flag = True

    def get_tensors(self) -> List[torch.Tensor]:
        return list(self.tensors_info.keys())

    # ------------------------------------------------------------------ checkpoint helpers

    def _gathered_copy(self) -> torch.Tensor:
        if self.is_replica:
            return self.rcb.payload
        buffer = torch.empty(self.chunk_size, dtype=self.chunk_dtype, device=self.compute_device)
        self._gather_into(buffer, self.shard)
        return buffer

    def get_cpu_copy(self, only_rank_0: bool = False) -> List[Optional[torch.Tensor]]:
        assert not self.is_init
        buffer = self._gathered_copy()
        copies: List[Optional[torch.Tensor]] = [None] * self.num_tensors
        if not only_rank_0 or self.pg_rank == 0:
            for i, (t, info) in enumerate(self.tensors_info.items()):
                copies[i] = buffer[info.offset:info.end].view(t.shape).cpu()
        if self.pg_size > 1:
            dist.barrier(group=self.torch_pg)
        return copies

    def load_tensors(self, tensor_list: List[Optional[torch.Tensor]], only_rank_0: bool = False) -> None:
        assert not self.is_replica and not self.is_init
        buffer = self._gathered_copy()
        if not only_rank_0 or self.pg_rank == 0:
            for info, src in zip(self.tensors_info.values(), tensor_list):
                if src is not None:
                    buffer[info.offset:info.end].copy_(src.data.flatten())
        if self.pg_size > 1:
            dist.barrier(group=self.torch_pg)
            if only_rank_0:
                dist.broadcast(buffer, src=dist.get_global_rank(self.torch_pg, 0) if self.torch_pg is not None else 0,
                               group=self.torch_pg)
        self.shard.copy_(buffer[self.shard_begin:self.shard_end])

    # ------------------------------------------------------------------ internals

    def _update_replica(self, replica: torch.Tensor, shard: torch.Tensor):
        assert self.is_replica
        assert replica.numel() == self.chunk_size and shard.numel() == self.shard_size
        self._gather_into(replica, shard)

    def _gather_into(self, replica: torch.Tensor, shard: torch.Tensor):
        if shard.device != replica.device:
            # shard in host memory: into its own slot of the replica first, then gather in place
            slot = replica[self.shard_begin:self.shard_end]
            slot.copy_(shard, non_blocking=True)
            shard = slot
        comm.all_gather(replica, shard, self.torch_pg)

    def _update_shard(self, replica: torch.Tensor, shard: torch.Tensor):
        assert self.is_replica
        assert replica.numel() == self.chunk_size and shard.numel() == self.shard_size
        shard.copy_(replica[self.shard_begin:self.shard_end])

    def _paired_shard(self) -> torch.Tensor:
        friend = self.paired_chunk
        assert friend is not None, 'chunks should be paired before training'
        assert self.chunk_size == friend.chunk_size
        out = torch.empty(self.shard_size, dtype=self.chunk_dtype, device=self.rcb.payload.device)
        source = friend.shard
        if source.device != out.device and not kernels.is_mapped_host(source):
            source = source.to(out.device)
        kernels.cast_copyback(source, out)
        return out

    def _remove_tensors_ptr(self) -> None:
        assert self.is_replica
        for tensor, info in self.tensors_info.items():
            tensor.data = info.fake_data

    def _update_tensors_ptr(self) -> None:
        assert self.is_replica
        payload = self.rcb.payload
        for tensor, info in self.tensors_info.items():
            tensor.data = payload[info.offset:info.end].view(tensor.shape)

    def _set_state(self, info: TensorInfo, next_state: TensorState):
        self.tensor_state_cnter[info.state] -= 1
        info.state = next_state
        self.tensor_state_cnter[next_state] += 1

    def _update_tensors_state(self, next_state: TensorState, prev_state: Optional[TensorState] = None):
        for info in self.tensors_info.values():
            if prev_state is None or info.state == prev_state:
                self._set_state(info, next_state)

    def __hash__(self) -> int:
        return self.chunk_id

    def __lt__(self, other: 'Chunk') -> bool:
        return self.chunk_id < other.chunk_id

    def __eq__(self, other: object) -> bool:
        return isinstance(other, Chunk) and self.chunk_id == other.chunk_id

    def __repr__(self) -> str:
        state = 'initialization' if self.is_init else ('replicated' if self.in_rcache else 'scattered')
        used = 100 * self.utilized_size / max(1, self.chunk_size)
        return (f'Chunk {self.chunk_id}: {state}, length {self.chunk_size}, dtype {self.chunk_dtype}, '
                f'group size {self.pg_size}, tensors {self.num_tensors}, used {self.utilized_size} ({used:.0f}%), '
                f'shard [{self.shard_begin}, {self.shard_end}) valid_end {self.valid_end}, '
                f'memory {self.memory_usage}')
