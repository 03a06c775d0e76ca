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

    def __init__(self, numel: int, dtype: torch.dtype, device_type, payload: torch.Tensor = None) -> None:
        self.block_id = TensorBlock.total_count
        TensorBlock.total_count += 1
        self.device_type = device_type
        self.payload = payload if payload is not None else torch.empty((numel,), dtype=dtype, device=device_type)
        assert self.payload.numel() == numel and self.payload.dtype == dtype
        self.memo_occ = numel * self.payload.element_size()

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

    def __init__(self, device_type) -> None:
        self.device_type = device_type
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
        if public_block_number > 0:
            self._public_slab = torch.empty(public_block_number * public_block_size,
                                            dtype=public_dtype,
                                            device=self.device_type)
            for i in range(public_block_number):
                view = self._public_slab[i * public_block_size:(i + 1) * public_block_size]
                self.public_free_blocks.append(PublicBlock(public_block_size, public_dtype, self.device_type, view))
            self.public_space = self._public_slab.numel() * self._public_slab.element_size()
        self.public_free_cnt = public_block_number
        self.public_used_cnt = 0

        self.private_blocks = []
        self.private_lookup_dict = defaultdict(list)
        self.private_space = 0
        for require in private_block_list:
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
        block = self.public_free_blocks.pop()
        self.public_used_blocks.add(block)
        self.public_free_cnt -= 1
        self.public_used_cnt += 1
        return block

    def free_public_block(self, block: TensorBlock) -> TensorBlock:
        assert isinstance(block, PublicBlock) and block in self.public_used_blocks
        self.public_used_blocks.remove(block)
        self.public_free_blocks.append(block)
        self.public_free_cnt += 1
        self.public_used_cnt -= 1
        return block
