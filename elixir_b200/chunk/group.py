"""The set of chunks of one dtype that share a replica cache (mirror of
``elixir/chunk/core/group.py``: same methods; "fused" chunks own a private block, "float" chunks
borrow public blocks)."""
from typing import Dict, List, Optional

import torch

from .chunk import Chunk
from .memory_pool import MemoryPool, TensorBlock
from .states import TensorState


class ChunkGroup:

    def __init__(self, rcache: MemoryPool) -> None:
        self.rcache = rcache
        self.fused_chunks: set = set()
        self.float_chunks: set = set()
        self.ten_to_chunk: Dict[torch.Tensor, Chunk] = dict()
        self.accessed_fused_chunks: set = set()
        self.accessed_float_chunks: set = set()

    def _home(self, chunk: Chunk) -> set:
        return self.fused_chunks if chunk.rcache_fused else self.float_chunks

    def _accessed(self, chunk: Chunk) -> set:
        return self.accessed_fused_chunks if chunk.rcache_fused else self.accessed_float_chunks

    def inside_check(self, chunk: Chunk) -> None:
        assert chunk in self._home(chunk), 'the chunk does not belong to this group'

    def is_accessed(self, chunk: Chunk) -> bool:
        self.inside_check(chunk)
        return chunk in self._accessed(chunk)

    def open_chunk(self, chunk_size: int, chunk_dtype: torch.dtype, process_group,
                   chunk_config: Optional[Dict] = None) -> Chunk:
        chunk = Chunk(rcache=self.rcache,
                      chunk_size=chunk_size,
                      chunk_dtype=chunk_dtype,
                      process_group=process_group,
                      **(chunk_config or {}))
        if not chunk.rcache_fused and self.rcache.public_space != 0:
            assert chunk_size == self.rcache.public_block_size
            assert chunk_dtype == self.rcache.public_dtype
        return chunk

    def close_chunk(self, chunk: Chunk) -> bool:
        chunk.close_chunk()
        self._home(chunk).add(chunk)
        for t in chunk.get_tensors():
            assert t not in self.ten_to_chunk
            self.ten_to_chunk[t] = chunk
        return True

    def allocate_chunk(self, tensor_list: List[torch.Tensor], chunk_size: int, chunk_dtype: torch.dtype, process_group,
                       chunk_config: Optional[Dict] = None) -> Chunk:
        chunk = self.open_chunk(chunk_size, chunk_dtype, process_group, chunk_config)
        for t in tensor_list:
            chunk.append_tensor(t)
        self.close_chunk(chunk)
        return chunk

    def tensors_to_chunks(self, tensor_list: List[torch.Tensor]) -> List[Chunk]:
        found = {self.ten_to_chunk.get(t) for t in tensor_list}
        return sorted(found, key=lambda c: c.chunk_id)

    def rcache_enough_check(self, chunk: Chunk) -> bool:
        return chunk.rcache_fused or self.rcache.public_free_cnt > 0

    def access_chunk(self, chunk: Chunk) -> bool:
        if self.is_accessed(chunk):
            return False
        chunk.access_chunk(None if chunk.rcache_fused else self.rcache.get_public_block())
        self._accessed(chunk).add(chunk)
        return True

    def release_chunk(self, chunk: Chunk) -> bool:
        assert self.is_accessed(chunk)
        assert chunk.scatter_check
        block = chunk.release_chunk()
        if block:
            self.rcache.free_public_block(block)
        self._accessed(chunk).remove(chunk)
        return True

    def reduce_chunk(self, chunk: Chunk, always_fp32: bool = False, sync: bool = True) -> Optional[TensorBlock]:
        assert self.is_accessed(chunk)
        assert chunk.reduce_check
        block = chunk.reduce_chunk(always_fp32=always_fp32, sync=sync)
        if block and sync:
            self.rcache.free_public_block(block)
            block = None
        self._accessed(chunk).remove(chunk)
        return block

    def tensor_trans_state(self, tensor: torch.Tensor, state: TensorState):
        self.ten_to_chunk[tensor].tensor_trans_state(tensor, state)
