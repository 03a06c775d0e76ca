"""Replica cache ("rcache"): the blocks a scattered chunk is gathered into.

Counterpart of ``elixir/chunk/core/memory_pool.py`` (TensorBlock / PublicBlock / PrivateBlock /
MemoryPool, same methods and counters).  Public blocks are equal-sized and recycled between chunks;
a private block belongs to one chunk for good.  Here all public blocks are carved out of ONE
allocation, so the collectives always see the same few address ranges.
"""
from collections import defaultdict
from typing import Iterable, NamedTuple

import torch


class BlockRequire(NamedTuple):
    numel: int
    dtype: torch.dtype


class TensorBlock:
    total_count: int = 0
    block_type = 'block'

    def __init__(self, numel: int, dtype: torch.dtype, device_type, payload: torch.Tensor = None,
                 slab_offset: int = None) -> None:
        self.block_id = TensorBlock.total_count
        TensorBlock.total_count += 1
        self.device_type = device_type
        self.slab_offset = slab_offset    # element offset inside the pool's slab, when the pool has one
        self.payload = payload if payload is not None else torch.empty((numel,), dtype=dtype, device=device_type)
        assert self.payload.numel() == numel and self.payload.dtype == dtype
        self.memo_occ = numel * self.payload.element_size()
        self.owner = None         # the chunk whose replica lives here at the moment
        self.free_event = None    # CUDA event after which a new owner may overwrite the payload

    @property
    def numel(self):
        return self.payload.numel()

    @property
    def dtype(self):
        return self.payload.dtype

    @property
    def device(self):
        return self.payload.device

    def __hash__(self) -> int:
        return self.block_id

    def __eq__(self, other: object) -> bool:
        return isinstance(other, TensorBlock) and self.block_id == other.block_id

    def __repr__(self) -> str:
        return (f'{type(self).__name__}(id={self.block_id}, numel={self.numel}, device={self.device_type}, '
                f'dtype={self.dtype}, memo={self.memo_occ})')


class PublicBlock(TensorBlock):
    block_type = 'public'


class PrivateBlock(TensorBlock):
    block_type = 'private'


class MemoryPool:

    def __init__(self, device_type, slab_factory=None) -> None:
        """``slab_factory(numel, dtype)``, when given, returns an object with a ``local`` tensor out of which
        EVERY block (public and private) is carved — used to place the replica cache in peer-mapped memory
        (``elixir_b200.peer.PeerBuffer``) for the NVLink step."""
        self.device_type = device_type
        self.slab_factory = slab_factory
        self.slab = None
        self.public_space = 0
        self.public_block_size = 0
        self.public_dtype = None
        self.public_free_blocks = None
        self.public_used_blocks = None
        self.public_free_cnt = 0
        self.public_used_cnt = 0
        self.private_space = 0
        self.private_blocks = None
        self.private_lookup_dict = None
        self._allocated = False
        self._public_slab = None

    def allocate(self,
                 public_dtype: torch.dtype = torch.float,
                 public_block_size: int = 1024,
                 public_block_number: int = 0,
                 private_block_list: Iterable[BlockRequire] = ()):
        assert not self._allocated, 'the pool is allocated once'
        assert public_block_number >= 0
        self.public_dtype = public_dtype
        self.public_block_size = public_block_size
        self.public_free_blocks = []
        self.public_used_blocks = set()
        private_block_list = list(private_block_list)
        pad = lambda n: (n + 15) // 16 * 16
        cursor = 0
        if self.slab_factory is not None:
            assert all(r.dtype == public_dtype for r in private_block_list), 'one dtype per slab'
            total = public_block_number * pad(public_block_size) + sum(pad(r.numel) for r in private_block_list)
            self.slab = self.slab_factory(max(total, 16), public_dtype)
        if public_block_number > 0:
            if self.slab is not None:
                self._public_slab = self.slab.local
                stride = pad(public_block_size)
            else:
                self._public_slab = torch.empty(public_block_number * public_block_size, dtype=public_dtype,
                                                device=self.device_type)
                stride = public_block_size
            for i in range(public_block_number):
                view = self._public_slab[i * stride:i * stride + public_block_size]
                self.public_free_blocks.append(
                    PublicBlock(public_block_size, public_dtype, self.device_type, view, slab_offset=i * stride))
            cursor = public_block_number * stride
            self.public_space = public_block_number * public_block_size * self._public_slab.element_size()
        self.public_free_cnt = public_block_number
        self.public_used_cnt = 0

        self.private_blocks = []
        self.private_lookup_dict = defaultdict(list)
        self.private_space = 0
        for require in private_block_list:
            if self.slab is not None:
                view = self.slab.local[cursor:cursor + require.numel]
                block = PrivateBlock(require.numel, require.dtype, self.device_type, view, slab_offset=cursor)
                cursor += pad(require.numel)
            else:
                block = PrivateBlock(require.numel, require.dtype, self.device_type)
            self.private_space += block.memo_occ
            self.private_blocks.append(block)
            self.private_lookup_dict[require].append(block)
        self._allocated = True

    def __repr__(self) -> str:
        return f'MP(public_space={self.public_space} B, private_space={self.private_space} B)'

    def get_private_block(self, numel: int, dtype: torch.dtype) -> PrivateBlock:
        return self.private_lookup_dict[BlockRequire(numel=numel, dtype=dtype)].pop()

    def get_public_block(self) -> PublicBlock:
        """A free block.  If its last user gave it back from another CUDA stream, the current stream is made
        to wait for that user's queued work before the caller may overwrite the payload."""
        block = self.public_free_blocks.pop()
        if block.free_event is not None:
            torch.cuda.current_stream(block.payload.device).wait_event(block.free_event)
            block.free_event = None
        self.public_used_blocks.add(block)
        self.public_free_cnt -= 1
        self.public_used_cnt += 1
        return block

    def free_public_block(self, block: TensorBlock) -> TensorBlock:
        assert isinstance(block, PublicBlock) and block in self.public_used_blocks
        block.owner = None
        if block.payload.is_cuda:
            # whatever the current stream still has queued on this payload finishes before the next owner writes
            block.free_event = torch.cuda.current_stream(block.payload.device).record_event()
        self.public_used_blocks.remove(block)
        self.public_free_blocks.append(block)
        self.public_free_cnt += 1
        self.public_used_cnt -= 1
        return block
