"""The chunks of one dtype that share a replica cache.

Same public face as ``elixir/chunk/core/group.py`` (method names, the four chunk sets, ``ten_to_chunk``), kept
differently: one registry maps every closed chunk to whether it currently holds a replica block, and the sets the
reference stores — ``fused_chunks`` (own a private block), ``float_chunks`` (borrow public blocks) and their
``accessed_*`` subsets — are views computed from it.
"""
from typing import Dict, List, Optional, Set

import torch

from .chunk import Chunk
from .memory_pool import MemoryPool, TensorBlock
from .states import TensorState


class ChunkGroup:

    def __init__(self, rcache: MemoryPool) -> None:
        self.rcache = rcache
        self.ten_to_chunk: Dict[torch.Tensor, Chunk] = {}
        self._holds_block: Dict[Chunk, bool] = {}    # closed chunk -> is replicated in a block right now

    # ------------------------------------------------------------------ the reference's four sets, as views

    def _select(self, fused: bool, only_accessed: bool) -> Set[Chunk]:
        return {c for c, held in self._holds_block.items() if c.rcache_fused == fused and (held or not only_accessed)}

    @property
    def fused_chunks(self) -> Set[Chunk]:
        return self._select(True, False)

    @property
    def float_chunks(self) -> Set[Chunk]:
        return self._select(False, False)

    @property
    def accessed_fused_chunks(self) -> Set[Chunk]:
        return self._select(True, True)

    @property
    def accessed_float_chunks(self) -> Set[Chunk]:
        return self._select(False, True)

    # ------------------------------------------------------------------ membership

    def inside_check(self, chunk: Chunk) -> None:
        assert chunk in self._holds_block, 'the chunk does not belong to this group'

    def is_accessed(self, chunk: Chunk) -> bool:
        self.inside_check(chunk)
        return self._holds_block[chunk]

    def tensors_to_chunks(self, tensor_list: List[torch.Tensor]) -> List[Chunk]:
        by_id = {}
        for t in tensor_list:
            chunk = self.ten_to_chunk[t]
            by_id[chunk.chunk_id] = chunk
        return [by_id[i] for i in sorted(by_id)]

    def tensor_trans_state(self, tensor: torch.Tensor, state: TensorState):
        self.ten_to_chunk[tensor].tensor_trans_state(tensor, state)

    # ------------------------------------------------------------------ building

    def open_chunk(self, chunk_size: int, chunk_dtype: torch.dtype, process_group,
                   chunk_config: Optional[Dict] = None) -> Chunk:
        chunk = Chunk(self.rcache, chunk_size, chunk_dtype, process_group, **(chunk_config or {}))
        shares_public_blocks = not chunk.rcache_fused and self.rcache.public_space != 0
        if shares_public_blocks:
            assert (chunk_size, chunk_dtype) == (self.rcache.public_block_size, self.rcache.public_dtype)
        return chunk

    def close_chunk(self, chunk: Chunk) -> bool:
        chunk.close_chunk()
        tensors = chunk.get_tensors()
        assert not any(t in self.ten_to_chunk for t in tensors)
        self.ten_to_chunk.update((t, chunk) for t in tensors)
        self._holds_block[chunk] = False
        return True

    def allocate_chunk(self, tensor_list: List[torch.Tensor], chunk_size: int, chunk_dtype: torch.dtype, process_group,
                       chunk_config: Optional[Dict] = None) -> Chunk:
        chunk = self.open_chunk(chunk_size, chunk_dtype, process_group, chunk_config)
        for t in tensor_list:
            chunk.append_tensor(t)
        self.close_chunk(chunk)
        return chunk

    # ------------------------------------------------------------------ replica blocks

    def rcache_enough_check(self, chunk: Chunk) -> bool:
        return chunk.rcache_fused or self.rcache.public_free_cnt > 0

    def _give_back(self, block: Optional[TensorBlock]) -> None:
        if block:
            self.rcache.free_public_block(block)

    def access_chunk(self, chunk: Chunk) -> bool:
        if self.is_accessed(chunk):
            return False
        chunk.access_chunk(None if chunk.rcache_fused else self.rcache.get_public_block())
        self._holds_block[chunk] = True
        return True

    def release_chunk(self, chunk: Chunk) -> bool:
        assert self.is_accessed(chunk) and chunk.scatter_check
        self._give_back(chunk.release_chunk())
        self._holds_block[chunk] = False
        return True

    def reduce_chunk(self, chunk: Chunk, always_fp32: bool = False, sync: bool = True) -> Optional[TensorBlock]:
        """With ``sync`` the block goes back to the pool here; without, the caller frees it once the reduce that
        still reads it has been ordered behind (``ChunkFetcher.reduce_chunk``)."""
        assert self.is_accessed(chunk) and chunk.reduce_check
        block = chunk.reduce_chunk(always_fp32=always_fp32, sync=sync)
        self._holds_block[chunk] = False
        if sync:
            self._give_back(block)
            return None
        return block
