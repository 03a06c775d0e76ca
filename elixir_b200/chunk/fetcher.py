"""What the optimizer path needs of ``elixir/chunk/fetcher.py``: the tensor -> chunk lookup and the
trigger that reduces a chunk once all of its gradients have arrived, optionally on a side stream
(``fetcher.py:128-153``).  Residency scheduling of the forward/backward pass is not part of it: every
chunk owns a block of the replica cache while a step is in flight."""
from typing import Optional

import torch

from .chunk import Chunk
from .group import ChunkGroup


class ChunkFetcher:

    def __init__(self, group: ChunkGroup, overlap: bool = False, reduce_always_fp32: bool = False) -> None:
        self.group = group
        self.overlap_flag = overlap
        self.reduce_always_fp32 = reduce_always_fp32
        self.reduce_stream: Optional[torch.cuda.Stream] = None

    def get_one_chunk(self, tensor: torch.Tensor) -> Chunk:
        return self.group.ten_to_chunk.get(tensor)

    def get_chunks(self, tensors) -> list:
        return self.group.tensors_to_chunks(tensors)

    def is_in_fused(self, tensor: torch.Tensor) -> bool:
        return self.get_one_chunk(tensor).rcache_fused

    def reduce_chunk(self, chunk: Chunk) -> bool:
        """Reduce ``chunk`` if every tensor in it is READY_FOR_REDUCE.  With ``overlap`` the collective,
        the copy into the shard and the probe run on a side stream behind the work already queued on the
        main stream; nothing is read back, so no callback is needed."""
        if not chunk.reduce_check:
            return False
        payload = chunk.rcb.payload
        if self.overlap_flag and payload.is_cuda:
            if self.reduce_stream is None:
                self.reduce_stream = torch.cuda.Stream(payload.device)
            main = torch.cuda.current_stream(payload.device)
            self.reduce_stream.wait_stream(main)
            with torch.cuda.stream(self.reduce_stream):
                self.group.reduce_chunk(chunk, always_fp32=self.reduce_always_fp32, sync=True)
        else:
            self.group.reduce_chunk(chunk, always_fp32=self.reduce_always_fp32, sync=True)
        return True

    def clear(self):
        """End of backward: later work on the main stream sees every reduce."""
        if self.reduce_stream is not None:
            torch.cuda.current_stream(self.reduce_stream.device).wait_stream(self.reduce_stream)
