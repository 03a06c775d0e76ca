from .chunk import Chunk, ChunkFullError, TensorInfo
from .fetcher import ChunkFetcher
from .group import ChunkGroup
from .scheduler import ChunkScheduler, FIFOScheduler, PrefetchScheduler
from .memory_pool import BlockRequire, MemoryPool, PrivateBlock, PublicBlock, TensorBlock
from .states import TensorState, ts_update_sanity_check

__all__ = [
    'BlockRequire', 'Chunk', 'ChunkFetcher', 'ChunkFullError', 'ChunkGroup', 'ChunkScheduler', 'FIFOScheduler',
    'MemoryPool', 'PrefetchScheduler', 'PrivateBlock', 'PublicBlock',
    'TensorBlock', 'TensorInfo', 'TensorState', 'ts_update_sanity_check'
]
