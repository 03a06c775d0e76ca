"""Which resident chunk gives up its replica-cache block when another chunk needs one.

Counterpart of ``elixir/chunk/scheduler/{base,fifo,prefetch}.py`` with the same methods (``reset``,
``clear``, ``top``, ``add``, ``remove``, ``step``, ``get_next_chunk``):

* ``FIFOScheduler``: the chunk that became releasable first goes first.
* ``PrefetchScheduler``: Belady's rule on a known access trace (one set of chunks per fetch): the
  releasable chunk whose next use lies furthest ahead goes first, ties to the larger chunk id, and the
  trace also tells the fetcher what to gather ahead of time.  The reference takes the trace from a
  tracing pre-run of the model; here it may also be left out, in which case the first training
  iteration runs in FIFO order while its fetches are written down, and the trace is in force from the
  second iteration on.
"""
import heapq
from abc import ABC, abstractmethod
from bisect import bisect_right
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch

from .chunk import Chunk


class ChunkScheduler(ABC):

    def __init__(self) -> None:
        self.releasable_set: Optional[set] = None
        self.current_step = -1

    def reset(self) -> None:
        self.releasable_set = set()
        self.current_step = -1

    def clear(self) -> None:
        assert not self.releasable_set, 'chunks are still waiting for release at the end of the pass'

    @abstractmethod
    def top(self) -> Optional[Chunk]:
        """The chunk to release next, or None when nothing is releasable.  Does not remove it."""

    def add(self, chunk: Chunk) -> bool:
        if chunk in self.releasable_set:
            return False
        self.releasable_set.add(chunk)
        return True

    def remove(self, chunk: Chunk) -> bool:
        if chunk not in self.releasable_set:
            return False
        self.releasable_set.remove(chunk)
        return True

    def step(self, chunks: Iterable[Chunk] = ()) -> None:
        """One fetch; ``chunks`` are the chunks it asks for."""
        self.current_step += 1

    def get_next_chunk(self, chunks: Sequence[Chunk]) -> Optional[Chunk]:
        """The first chunk a later fetch will ask for that is not among ``chunks`` (None: unknown)."""
        return None

    def upcoming(self, exclude: Sequence[Chunk] = (), horizon: int = 32) -> Iterator[Tuple[int, Chunk]]:
        """(step, chunk) of the next ``horizon`` fetches in order, each chunk once.  Nothing when the future is
        unknown."""
        return iter(())

    def next_use(self, chunk: Chunk) -> int:
        """Step of the next fetch that asks for ``chunk``; a large number when unknown or never."""
        return 1 << 62


class FIFOScheduler(ChunkScheduler):

    def __init__(self) -> None:
        super().__init__()
        self._queue: Optional[Dict[Chunk, None]] = None    # insertion-ordered

    def reset(self) -> None:
        super().reset()
        self._queue = dict()

    def clear(self) -> None:
        super().clear()
        self._queue = None

    def top(self) -> Optional[Chunk]:
        if not self.releasable_set:
            return None
        return next(iter(self._queue))

    def add(self, chunk: Chunk) -> bool:
        if not super().add(chunk):
            return False
        self._queue[chunk] = None
        return True

    def remove(self, chunk: Chunk) -> bool:
        if not super().remove(chunk):
            return False
        del self._queue[chunk]
        return True


class PrefetchScheduler(ChunkScheduler):

    def __init__(self, chunk_called_per_step: Optional[List[Iterable[Chunk]]] = None) -> None:
        super().__init__()
        self.chunks_per_step: Optional[List[List[Chunk]]] = None
        self.total_steps = 0
        self._uses: Dict[Chunk, List[int]] = dict()
        self._heap: Optional[list] = None    # (-next use, -chunk id, chunk); entries go stale, `_key` tells
        self._key: Optional[Dict[Chunk, Tuple[int, int]]] = None
        self._fifo: Optional[Dict[Chunk, None]] = None    # order of release while the trace is being learnt
        self._recorded: Optional[List[List[Chunk]]] = None
        self.search_step = -1
        if chunk_called_per_step is not None:
            self._install_trace(chunk_called_per_step)

    # ------------------------------------------------------------------ the trace

    @property
    def learning(self) -> bool:
        return self.chunks_per_step is None

    def _install_trace(self, chunk_called_per_step: List[Iterable[Chunk]]) -> None:
        self.chunks_per_step = [sorted(set(step)) for step in chunk_called_per_step]
        self.total_steps = len(self.chunks_per_step)
        self._uses = dict()
        for i, step in enumerate(self.chunks_per_step):
            for chunk in step:
                self._uses.setdefault(chunk, []).append(i)

    def relearn(self) -> None:
        """Forget the trace; the next training iteration writes a new one."""
        self.chunks_per_step = None
        self.total_steps = 0
        self._uses = dict()

    def next_use(self, chunk: Chunk) -> int:
        if self.learning:
            return 1 << 62
        steps = self._uses.get(chunk, ())
        i = bisect_right(steps, self.current_step)
        return steps[i] if i < len(steps) else self.total_steps

    # kept under the reference's name
    _get_next_step = next_use

    # ------------------------------------------------------------------ one pass

    def reset(self) -> None:
        super().reset()
        self._heap, self._key, self._fifo = [], dict(), dict()
        self.search_step = -1
        self._recorded = [] if (self.learning and torch.is_grad_enabled()) else None

    def clear(self) -> None:
        super().clear()
        if self._recorded is not None:
            if torch.is_grad_enabled() and self._recorded:
                self._install_trace(self._recorded)
        elif not self.learning and torch.is_grad_enabled():
            assert self.current_step == self.total_steps - 1, (
                f'the pass made {self.current_step + 1} fetches, the trace has {self.total_steps}')
        self._heap = self._key = self._fifo = self._recorded = None
        self.search_step = -1

    def step(self, chunks: Iterable[Chunk] = ()) -> None:
        super().step(chunks)
        if self._recorded is not None:
            self._recorded.append(list(chunks))
        elif not self.learning and self.current_step >= self.total_steps:
            raise RuntimeError('more fetches than the access trace holds: the model does not repeat the traced '
                               'pass; call relearn() on the scheduler or use the FIFO scheduler')

    def top(self) -> Optional[Chunk]:
        if not self.releasable_set:
            return None
        if self.learning:
            return next(iter(self._fifo))
        while True:
            neg_step, neg_id, chunk = self._heap[0]
            if self._key.get(chunk) == (neg_step, neg_id):
                return chunk
            heapq.heappop(self._heap)    # the chunk was removed or re-added since

    def add(self, chunk: Chunk) -> bool:
        if not super().add(chunk):
            return False
        self._fifo[chunk] = None
        key = (-self.next_use(chunk), -chunk.chunk_id)
        self._key[chunk] = key
        heapq.heappush(self._heap, (*key, chunk))
        return True

    def remove(self, chunk: Chunk) -> bool:
        if not super().remove(chunk):
            return False
        del self._fifo[chunk]
        del self._key[chunk]
        return True

    # ------------------------------------------------------------------ looking ahead

    def get_next_chunk(self, chunks: Sequence[Chunk]) -> Optional[Chunk]:
        if self.learning:
            return None
        self.search_step = max(self.search_step, self.current_step + 1)
        while self.search_step < self.total_steps:
            for chunk in self.chunks_per_step[self.search_step]:
                if chunk not in chunks:
                    return chunk
            self.search_step += 1
        return None

    def upcoming(self, exclude: Sequence[Chunk] = (), horizon: int = 32) -> Iterator[Tuple[int, Chunk]]:
        if self.learning:
            return
        seen = set(exclude)
        for step in range(self.current_step + 1, min(self.total_steps, self.current_step + 1 + horizon)):
            for chunk in self.chunks_per_step[step]:
                if chunk not in seen:
                    seen.add(chunk)
                    yield step, chunk
