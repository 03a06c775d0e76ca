"""Brings chunks into the replica cache when their tensors are about to be used, sends them back when a
block is needed, and reduces a chunk once all of its gradients have arrived.

Counterpart of ``elixir/chunk/fetcher.py`` (same methods: ``reset``, ``clear``, ``trans_to_compute``,
``trans_to_hold``, ``fetch_chunks``, ``prefetch``, ``reduce_chunk``, ``step``), with these differences:

* stream ordering is carried by CUDA events on the objects that move (``TensorBlock.free_event``: the
  block may be overwritten after it; ``Chunk.ready_event``: the gathered replica may be read after it)
  instead of stream-wide waits at fixed points, so a reduce, a gather ahead of time and the computation
  overlap without the bookkeeping of one "reduced chunk in flight";
* nothing is read back from the device after a reduce (the overflow word and the norm stay there), so the
  reduce needs no call-back;
* a chunk that already holds gradients of the running backward pass is never chosen for release
  (``Chunk.evict_check``);
* with a ``PrefetchScheduler`` up to ``prefetch_depth`` chunks are gathered ahead on a side stream, and a
  resident chunk is released for one only if its own next use comes later than the use of the chunk
  gathered ahead.
"""
from typing import List, Optional, Sequence

import torch

from .chunk import Chunk
from .group import ChunkGroup
from .scheduler import ChunkScheduler, FIFOScheduler
from .states import TensorState


class ChunkFetcher:

    def __init__(self,
                 scheduler: Optional[ChunkScheduler],
                 group: ChunkGroup,
                 overlap: bool = False,
                 reduce_always_fp32: bool = False,
                 prefetch_depth: int = 2) -> None:
        self.scheduler: ChunkScheduler = scheduler if scheduler is not None else FIFOScheduler()
        self.group = group
        self.overlap_flag = overlap
        self.reduce_always_fp32 = reduce_always_fp32
        self.prefetch_depth = prefetch_depth
        self.current_step = -1
        self.reduce_stream: Optional[torch.cuda.Stream] = None
        self.prefetch_stream: Optional[torch.cuda.Stream] = None
        self.predict_next_chunk: Optional[Chunk] = None
        self._ahead: set = set()    # gathered ahead of time, not asked for yet
        # counters of the running pass (tests and tuning read them)
        self.stats = dict(fetched=0, released=0, ahead=0, ahead_hit=0)

    # ------------------------------------------------------------------ lookups

    def get_one_chunk(self, tensor: torch.Tensor) -> Chunk:
        return self.group.ten_to_chunk.get(tensor)

    def get_chunks(self, tensors) -> List[Chunk]:
        return self.group.tensors_to_chunks(tensors)

    def is_in_fused(self, tensor: torch.Tensor) -> bool:
        return self.get_one_chunk(tensor).rcache_fused

    def filter_chunks(self, chunks: Sequence[Chunk]) -> List[Chunk]:
        return [c for c in chunks if not self.group.is_accessed(c)]

    # ------------------------------------------------------------------ one pass

    def reset(self) -> None:
        """Start of a pass.  Replicas left behind by a pass that was abandoned (a forward with gradients
        enabled that no backward followed) go back first, so that their blocks are not lost."""
        for stream in (self.reduce_stream, self.prefetch_stream):
            if stream is not None:
                torch.cuda.current_stream(stream.device).wait_stream(stream)
        for chunk in sorted(self.group.accessed_float_chunks):
            chunk.ready_event = None
            if chunk.evict_check:
                self.group.release_chunk(chunk)
        self.scheduler.reset()
        self.current_step = -1
        self.predict_next_chunk = None
        self._ahead = set()
        self.stats = dict(fetched=0, released=0, ahead=0, ahead_hit=0)

    def step(self, chunks: Sequence[Chunk] = ()) -> None:
        self.scheduler.step(chunks)
        self.current_step += 1

    def clear(self) -> None:
        """End of the pass: later work on the main stream sees every reduce and every gather; chunks gathered
        ahead and never asked for give their blocks back."""
        for stream in (self.reduce_stream, self.prefetch_stream):
            if stream is not None:
                torch.cuda.current_stream(stream.device).wait_stream(stream)
        for chunk in sorted(self._ahead):
            chunk.ready_event = None
            if self.group.is_accessed(chunk) and chunk.evict_check:
                self.group.release_chunk(chunk)
        self._ahead = set()
        self.predict_next_chunk = None
        if self.scheduler.releasable_set is not None:
            self.scheduler.clear()

    def release_all(self) -> None:
        """Send every releasable chunk back (end of a pass without gradients)."""
        while True:
            chunk = self.scheduler.top()
            if chunk is None:
                break
            self.scheduler.remove(chunk)
            self.group.release_chunk(chunk)
            self.stats['released'] += 1

    # ------------------------------------------------------------------ tensor states

    def trans_to_compute(self, tensors: Sequence[torch.Tensor]) -> List[Chunk]:
        for t in tensors:
            self.group.tensor_trans_state(t, TensorState.COMPUTE)
        chunks = self.group.tensors_to_chunks(tensors)
        for chunk in chunks:
            self.scheduler.remove(chunk)
        return chunks

    def trans_to_hold(self, tensors: Sequence[torch.Tensor], phase: str) -> None:
        assert phase in ('f', 'b')
        next_state = TensorState.HOLD if phase == 'f' else TensorState.HOLD_AFTER_BWD
        for t in tensors:
            self.group.tensor_trans_state(t, next_state)
        for chunk in self.group.tensors_to_chunks(tensors):
            if chunk.evict_check and self.group.is_accessed(chunk):
                self.scheduler.add(chunk)

    # ------------------------------------------------------------------ gather

    def _main_stream(self, chunk: Chunk):
        device = chunk.shard.device if chunk.rcb is None else chunk.rcb.payload.device
        return torch.cuda.current_stream(device) if device.type == 'cuda' else None

    def _make_room(self, chunk: Chunk) -> None:
        if self.group.rcache_enough_check(chunk):
            return
        victim = self.scheduler.top()
        if victim is None:
            raise RuntimeError('R cache is not enough. Try to allocate more.')
        self.scheduler.remove(victim)
        self.group.release_chunk(victim)
        self.stats['released'] += 1

    def fetch_chunks(self, chunks: Sequence[Chunk]) -> None:
        """Make ``chunks`` resident for the computation about to be queued on the current stream."""
        self.step(chunks)
        for chunk in chunks:
            if self.group.is_accessed(chunk):
                if chunk.ready_event is not None:    # gathered ahead on the side stream
                    self._main_stream(chunk).wait_event(chunk.ready_event)
                    chunk.ready_event = None
                if chunk in self._ahead:
                    self._ahead.remove(chunk)
                    self.stats['ahead_hit'] += 1
                continue
            self._make_room(chunk)
            self.group.access_chunk(chunk)
            self.stats['fetched'] += 1
        if self.overlap_flag:
            self.prefetch(chunks)

    def prefetch(self, chunks: Sequence[Chunk]) -> None:
        """Gather chunks of later fetches ahead of time, on a side stream behind the work already queued."""
        self.predict_next_chunk = self.scheduler.get_next_chunk(chunks)
        room = self.prefetch_depth - len(self._ahead)
        if room <= 0:
            return
        for step, chunk in self.scheduler.upcoming(exclude=chunks):
            if room <= 0:
                break
            if self.group.is_accessed(chunk):
                continue
            victim = None
            if not self.group.rcache_enough_check(chunk):
                victim = self.scheduler.top()
                if victim is None or self.scheduler.next_use(victim) <= step:
                    break    # everything resident is needed sooner than this chunk
                self.scheduler.remove(victim)
            main = self._main_stream(chunk)
            if main is None:    # host memory: no streams, the gather simply happens now
                if victim is not None:
                    self.group.release_chunk(victim)
                self.group.access_chunk(chunk)
            else:
                if self.prefetch_stream is None:
                    self.prefetch_stream = torch.cuda.Stream(main.device)
                self.prefetch_stream.wait_stream(main)
                with torch.cuda.stream(self.prefetch_stream):
                    if victim is not None:
                        self.group.release_chunk(victim)
                    self.group.access_chunk(chunk)
                    chunk.ready_event = self.prefetch_stream.record_event()
            if victim is not None:
                self.stats['released'] += 1
            self._ahead.add(chunk)
            self.stats['ahead'] += 1
            room -= 1

    # ------------------------------------------------------------------ reduce

    def reduce_chunk(self, chunk: Chunk) -> bool:
        """Reduce ``chunk`` if every tensor in it is READY_FOR_REDUCE.  With ``overlap`` the collective,
        the copy into the shard and the probe run on a side stream behind the work already queued on the
        main stream; the block goes back to the pool at once and carries the event its next owner waits on."""
        if not chunk.reduce_check:
            return False
        if self.scheduler.releasable_set is not None:
            self.scheduler.remove(chunk)
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
