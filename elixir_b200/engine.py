"""ChunkStepEngine: one rank's optimizer step over its chunk shards, launched as whole-chunk-set kernels.

It replaces the per-tensor loop of the reference (``ElixirOptimizer._set_grad_ptr`` /
``optim.step`` / ``_update_fp16_params``, ``elixir/wrapper/optimizer.py:115-135, 192-220``): the
shards are registered once in device tables, and a step is

    [gradients arrive]   land() / probe()   copy into the shard + inf/nan probe, per chunk
    begin_step()         overflow agreement across ranks (4-byte MAX all-reduce), the optional global
                         norm, then ``elx_step_begin``: skip decision, divisor, scaler update, per-chunk
                         overflow words cleared — on the device, no host read
    update()             ``elx_adam_multi``: unscale + Adam/AdamW + low-precision copy-back (or the
                         copy-back alone on a skipped step)

For sharded runs ``step_sharded`` pipelines reduce-scatter -> probe per chunk on a reduce stream and
update -> all-gather per chunk on a gather stream; ``step_from_host`` does the same with host buffers
on the two ends (pinned gradients in, updated low-precision parameters out).  Shards may also live in
pinned host memory: ``step`` then reaches them over PCIe with the same kernels, and after
``enable_streaming`` the copy engines move them through device staging sets around the update.
"""
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import comm, kernels
from .scaler import BaseGradScaler, ConstantGradScaler


class ChunkStepEngine:

    def __init__(self,
                 device,
                 dtype: torch.dtype,
                 scaler: Optional[BaseGradScaler] = None,
                 process_group=None,
                 sync_overflow: bool = True,
                 max_norm: float = 0.0):
        self.device = torch.device(device)
        self.dtype = dtype
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.sync_overflow = sync_overflow
        self.scaler = scaler if scaler is not None else ConstantGradScaler(1.0)
        self.scaler.set_max_norm(max_norm)
        self.clipping = max_norm > 0.0
        self.ctl = kernels.ControlBlock(self.device, self.scaler.initial_scale)
        self.scaler.attach(self.ctl)
        self.table = kernels.ChunkTable(self.device, dtype)
        self.shards: List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, int]] = []
        self.grad_srcs: List[Optional[torch.Tensor]] = []    # per shard: separate gradient source, or None
        self.chunk_flags: Optional[torch.Tensor] = None
        self.chunk_l2sq: Optional[torch.Tensor] = None
        self.total_l2sq: Optional[torch.Tensor] = None
        self._scratch: Optional[torch.Tensor] = None
        self._streams = None
        self._slots = None    # device staging sets of the streamed update (enable_streaming)
        self._sets = None     # the two sets of master/moment arrays of the single-pass step (enable_single_pass)

    # ------------------------------------------------------------------ registration

    def add_shard(self,
                  master: torch.Tensor,
                  lowp: torch.Tensor,
                  n_valid: int,
                  segments: Sequence[Tuple[int, int, int]],
                  exp_avg: Optional[torch.Tensor] = None,
                  exp_avg_sq: Optional[torch.Tensor] = None,
                  grad_src: Optional[torch.Tensor] = None) -> int:
        """Register a shard: fp32 master, the paired low-precision shard (gradient in / parameter out),
        ``valid_end`` and the (begin, end, param-group) ranges the optimizer updates.  The two moments
        are allocated here, flat and congruent with the master, unless given.  With ``grad_src`` the probe
        and the update read the gradient from that tensor (the block the backward pass filled) instead of
        from ``lowp``, so that nothing has to be copied into the shard before the step (``probe`` instead of
        ``land``); ``lowp`` still receives the refreshed working copy.  The four arrays may also be
        pinned host tensors (a shard kept off the GPU): ``land``/``probe``/``step`` then reach them over PCIe
        with the same kernels; the collective pipelines (``step_sharded*``) need device-resident shards."""
        def zeros():    # where the master lives, page-locked if it is
            return torch.zeros(master.shape, dtype=master.dtype, device=master.device,
                               pin_memory=kernels.is_mapped_host(master))

        exp_avg = zeros() if exp_avg is None else exp_avg
        exp_avg_sq = zeros() if exp_avg_sq is None else exp_avg_sq
        index = self.table.add_chunk(master, exp_avg, exp_avg_sq, lowp, n_valid, segments, grad_src=grad_src)
        self.shards.append((master, exp_avg, exp_avg_sq, lowp, n_valid))
        self.grad_srcs.append(grad_src)
        return index

    def finalize(self):
        self.table.finalize()
        n = max(1, self.table.n_chunks)
        self.chunk_flags = torch.zeros(n, dtype=torch.int32, device=self.device)
        self.chunk_l2sq = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.total_l2sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        if self.clipping:
            self._scratch = torch.empty(max(1, self.table.tiles()), dtype=torch.float32, device=self.device)
        return self

    @property
    def n_chunks(self) -> int:
        return self.table.n_chunks

    def n_elements(self) -> int:
        return sum(s[0].numel() for s in self.shards)

    def set_hyper(self, groups):
        self.table.set_hyper(groups)

    # ------------------------------------------------------------------ gradient arrival

    def land(self, index: int, src: torch.Tensor):
        """Copy reduced gradients ``src`` into shard ``index`` and probe them in the same pass."""
        lowp, n_valid = self.shards[index][3], self.shards[index][4]
        if self.grad_srcs[index] is not None:
            raise RuntimeError(f'shard {index} reads its gradient from a separate source: fill that tensor and call '
                               'probe() instead of land()')
        kernels.reduce_epilogue(src, lowp, n_valid=n_valid, flag=self.chunk_flags[index:index + 1], ctl=self.ctl)

    def land_all(self, srcs: Sequence[torch.Tensor], streams: int = 2):
        """``land`` for every shard, issued round-robin on ``streams`` side streams so that the tail of one
        launch overlaps the ramp-up of the next (the launches are independent: different shards, and the flag
        words are only ever raised).  The current stream waits for all of them."""
        assert len(srcs) == self.n_chunks
        main = torch.cuda.current_stream(self.device)
        if streams <= 1 or self.device.type != 'cuda':
            for k, src in enumerate(srcs):
                self.land(k, src)
            return
        if getattr(self, '_land_streams', None) is None or len(self._land_streams) != streams:
            self._land_streams = [torch.cuda.Stream(self.device) for _ in range(streams)]
        for st in self._land_streams:
            st.wait_stream(main)
        for k, src in enumerate(srcs):
            with torch.cuda.stream(self._land_streams[k % streams]):
                self.land(k, src)
        for st in self._land_streams:
            main.wait_stream(st)

    def _grad_home(self, index: int) -> torch.Tensor:
        """Where the kernels read shard ``index``'s gradient: its separate source, or the shard itself."""
        src = self.grad_srcs[index]
        return src if src is not None else self.shards[index][3]

    def probe(self, first: int = 0, count: Optional[int] = None):
        """Probe, in one launch, gradients that sit where the update will read them: in the shards, or in the
        separate sources given to ``add_shard``."""
        kernels.grad_check_multi(self.table, self.ctl, chunk_flags=self.chunk_flags, first=first, count=count)

    def probe_one(self, index: int):
        kernels.grad_check(self._grad_home(index), n_valid=self.shards[index][4],
                           flag=self.chunk_flags[index:index + 1], ctl=self.ctl)

    # ------------------------------------------------------------------ the step

    def begin_step(self):
        if self.world > 1 and self.sync_overflow:
            comm.agree_on_overflow(self.ctl.found_inf, self.group)
        norm_sq = None
        if self.clipping:
            kernels.grad_check_multi(self.table, None, chunk_l2sq=self.chunk_l2sq, total_l2sq=self.total_l2sq,
                                     scratch=self._scratch)
            if self.world > 1:
                dist.all_reduce(self.total_l2sq, group=self.group)
            norm_sq = self.total_l2sq
        kernels.step_begin(self.ctl, self.scaler.cfg, norm_sq, self.chunk_flags)

    def update(self, first: int = 0, count: Optional[int] = None):
        """The fused update of shards [first, first + count).  After ``enable_streaming`` the update of the whole
        set goes through the staging sets (shards in host memory travel with the copy engines)."""
        if self._slots is not None and first == 0 and count is None:
            self._update_streamed()
        else:
            kernels.adam_multi(self.table, self.ctl, first=first, count=count)

    def end_step(self):
        """Nothing left to do: ``elx_step_begin`` clears the per-chunk overflow words together with
        ``found_inf``, where the reference clears ``Chunk.overflow`` (``optimizer.py:144-147``).  Kept so that
        call sites written against the begin / update / end sequence stay valid."""

    def step(self):
        """Decision + fused update of every shard.  Gradients must already sit (probed) in the shards."""
        self.begin_step()
        self.update()
        self.end_step()

    def capture_step(self, srcs: Sequence[torch.Tensor]) -> 'torch.cuda.CUDAGraph':
        """Record ``land_all(srcs)`` + ``step()`` as one CUDA graph and return it; ``graph.replay()`` then runs
        a whole step (landing copies with their probes, decision, update, flag reset) with a single launch
        from the host.  Possible because nothing in the step reads the device: the skip decision, the loss
        scale and the step count live in the control block and the kernels branch on them.  It frees the host
        thread (one call per step); it does not shorten the step itself: eager launches already run ahead of
        the device (measured on 4 chunks of 4 Mi elements: 150 us eager, 167 us replayed).  The gradient sources are the
        tensors given here: refill them in place between replays.  Hyper-parameter changes (``set_hyper``) take
        effect without a new capture as long as the number of groups stays the same; one rank only."""
        assert self.world == 1 and self._slots is None and not self.table.host_resident
        assert len(srcs) == self.n_chunks
        current = torch.cuda.current_stream(self.device)
        warm = torch.cuda.Stream(self.device)
        warm.wait_stream(current)
        with torch.cuda.stream(warm):    # first launches outside the capture: per-device set-up of the kernels
            backup = self.ctl.tensor.clone()
            saved = [[t.clone() for t in shard[:4]] for shard in self.shards]
            self.land_all(srcs, streams=1)
            self.step()
            self.ctl.tensor.copy_(backup)    # the warm-up step must leave no trace
            for shard, kept in zip(self.shards, saved):
                for t, old in zip(shard[:4], kept):
                    t.copy_(old)
        current.wait_stream(warm)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.land_all(srcs, streams=1)
            self.step()
        return graph

    # ------------------------------------------------------------------ pipelines

    def _phase_marks(self, stream):
        """When ``self.profile`` is set, timestamp the phases of a pipelined step with CUDA events on the
        main stream; ``phase_ms()`` reads them back (after a synchronize)."""
        if not getattr(self, 'profile', False):
            return lambda name: None
        events = [('start', torch.cuda.Event(enable_timing=True))]
        events[0][1].record(stream)
        self._last_marks = events

        def mark(name):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            events.append((name, ev))

        return mark

    def phase_ms(self):
        marks = getattr(self, '_last_marks', None)
        if not marks:
            return {}
        return {b[0]: a[1].elapsed_time(b[1]) for a, b in zip(marks, marks[1:])}

    def _side_streams(self):
        if self._streams is None:
            self._streams = (torch.cuda.Stream(self.device), torch.cuda.Stream(self.device))
        return self._streams

    def step_sharded(self,
                     grad_blocks: Sequence[torch.Tensor],
                     gather_blocks: Sequence[Optional[torch.Tensor]],
                     host_grads: Optional[Sequence[torch.Tensor]] = None,
                     host_params: Optional[Sequence[torch.Tensor]] = None):
        """Sharded step: for chunk k, ``grad_blocks[k]`` is the replicated gradient block (chunk_size
        elements) and ``gather_blocks[k]`` the block the updated parameters are gathered into (or None).

        reduce stream:  RS(0) RS(1) ...            (rank average, output straight into the shard)
        main stream:       probe(0) probe(1) ... | decision | Adam(0) Adam(1) ...
        gather stream:                                           AG(0)   AG(1) ...
        The update of any chunk starts only after every chunk was reduced and probed, because one
        overflow anywhere skips the whole step (``elixir/wrapper/optimizer.py:194-203``).
        Shards must be device-resident (the collective writes into them).

        With ``host_grads`` (pinned, chunk_size each) block k is first filled from the host on the reduce
        stream; with ``host_params`` (pinned, shard_size each) the updated shard k is copied out on the
        gather stream.  Blocks may be reused between chunks: stream order keeps each reuse behind the
        collective that last read or wrote the block.
        """
        assert len(grad_blocks) == self.n_chunks and len(gather_blocks) == self.n_chunks
        if self.table.host_resident:
            raise RuntimeError('step_sharded needs device-resident shards: the collectives write into them')
        main = torch.cuda.current_stream(self.device)
        reduce_stream, gather_stream = self._side_streams()
        reduce_stream.wait_stream(main)
        gather_stream.wait_stream(main)
        marks = self._phase_marks(main)
        for k, block in enumerate(grad_blocks):
            lowp = self.shards[k][3]
            with torch.cuda.stream(reduce_stream):
                if host_grads is not None:
                    block.copy_(host_grads[k], non_blocking=True)
                comm.reduce_scatter_avg(lowp, block, self.group)
                done = torch.cuda.Event()
                done.record(reduce_stream)
            main.wait_event(done)
            self.probe_one(k)
        marks('reduced')
        self.begin_step()
        marks('decided')
        for k, block in enumerate(gather_blocks):
            self.update(first=k, count=1)
            if block is None and host_params is None:
                continue
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(gather_stream):
                gather_stream.wait_event(done)
                if block is not None:
                    comm.all_gather(block, self.shards[k][3], self.group)
                if host_params is not None:
                    host_params[k].copy_(self.shards[k][3], non_blocking=True)
        self.end_step()
        marks('updated')
        main.wait_stream(gather_stream)
        marks('gathered')

    # ------------------------------------------------------------------ NVLink path

    def enable_p2p(self, chunk_sizes: Sequence[int], timeout_ms: int = 20000, pool: Optional[int] = None):
        """Allocate the peer-mapped slabs of the NVLink path: one gradient slab and one gather slab per rank, plus
        the barrier flags.  By default each slab holds a block of ``chunk_sizes[k]`` elements for every
        registered chunk k.  With ``pool`` = P the slabs hold only P blocks (of the largest chunk size) and chunk
        k uses block ``k % P`` — the regime of models whose replicated blocks cannot all be resident; the step
        then runs chunk by chunk (``step_sharded_p2p``).  ``grad_block(k)`` / ``gather_block(k)`` are this rank's
        blocks."""
        from .peer import PeerBarrier, PeerBuffer
        assert len(chunk_sizes) == self.n_chunks
        for k, size in enumerate(chunk_sizes):
            if size != self.shards[k][0].numel() * self.world:
                raise ValueError(f'chunk {k}: chunk size {size} is not world x shard size')
        pad = lambda n: (n + 15) // 16 * 16
        if pool:
            stride = pad(max(chunk_sizes))
            offsets = [(k % pool) * stride for k in range(self.n_chunks)]
            total = min(pool, self.n_chunks) * stride
        else:
            offsets, total = [], 0
            for size in chunk_sizes:
                offsets.append(total)
                total += pad(size)
        self._p2p_pool = pool or 0
        self._p2p_sizes = list(chunk_sizes)
        self._p2p_offsets = offsets
        self.block_off = torch.tensor(offsets, dtype=torch.int64, device=self.device)
        self.grad_slab = PeerBuffer(total, self.dtype, self.device, self.group, zero=True)    # finite padding
        self.gather_slab = PeerBuffer(total, self.dtype, self.device, self.group)
        self.peer_barrier = PeerBarrier(self.device, self.group, timeout_ms)
        return self

    def attach_p2p(self, slab, block_offsets: Sequence[int], timeout_ms: int = 20000):
        """NVLink path over ONE existing peer-mapped slab (a replica cache): block k of every rank, at element
        offset ``block_offsets[k]``, holds that rank's gradients of chunk k before the step and receives the
        gathered parameters after it.  Rank r only ever reads and writes slice r of the other ranks' blocks, so
        sharing the slab between the two directions needs no extra ordering."""
        from .peer import PeerBarrier
        assert len(block_offsets) == self.n_chunks
        self._p2p_pool = 0
        self._p2p_sizes = [self.shards[k][0].numel() * self.world for k in range(self.n_chunks)]
        self._p2p_offsets = list(block_offsets)
        self.block_off = torch.tensor(self._p2p_offsets, dtype=torch.int64, device=self.device)
        self.grad_slab = self.gather_slab = slab
        self.peer_barrier = PeerBarrier(self.device, self.group, timeout_ms)
        return self

    def grad_block(self, k: int) -> torch.Tensor:
        return self.grad_slab.local[self._p2p_offsets[k]:self._p2p_offsets[k] + self._p2p_sizes[k]]

    def gather_block(self, k: int) -> torch.Tensor:
        return self.gather_slab.local[self._p2p_offsets[k]:self._p2p_offsets[k] + self._p2p_sizes[k]]

    def step_sharded_p2p(self, host_grads: Optional[Sequence[torch.Tensor]] = None,
                         host_params: Optional[Sequence[torch.Tensor]] = None):
        """Sharded step with both collectives fused into the kernels, over peer-mapped memory:

            barrier            every rank's gradient blocks are written
            pull reduce        one launch: rank average of this rank's slices, read from all ranks, + probe
            barrier + agree    every rank is done reading (blocks may be rewritten); overflow word OR-ed
            decision           elx_step_begin
            update + push      one launch: fused Adam, refreshed parameters stored into every rank's gather block
            barrier            every rank's pushes have landed: the gather blocks are complete

        Six launches per step, no NCCL call, no host synchronisation.

        With pooled blocks (``enable_p2p(pool=P)``) the two fused kernels are launched chunk by chunk, with a
        barrier before each pull (chunk k's gradients are in block ``k % P`` on every rank) — the order in which
        a backward pass produces them; the decision still waits for the last chunk.

        With ``host_grads`` (pinned, chunk_size elements each: this rank's gradients of chunk k) the step also runs
        chunk by chunk: block k is filled from the host on a copy stream while earlier chunks are being pulled.
        With ``host_params`` (pinned, shard_size each) the refreshed shard k leaves for the host on a second copy
        stream behind its update, while later chunks are updated and pushed."""
        pooled = getattr(self, '_p2p_pool', 0)
        main = torch.cuda.current_stream(self.device)
        if host_grads is not None or host_params is not None:
            h2d, d2h = self._side_streams()
            h2d.wait_stream(main)
            d2h.wait_stream(main)
        if host_grads is not None:
            assert len(host_grads) == self.n_chunks
            # Block k % P is refilled for chunk k while OTHER ranks may still be reading its previous tenant, chunk
            # k - P.  A rank launches the barrier that precedes pull(k - P + 1) only behind its own pull(k - P), so
            # once that barrier has completed here every rank is done with chunk k - P: the refill waits for it.
            passed = [None] * (self.n_chunks + 1)    # passed[k]: the barrier before pull(k) has completed on this rank
            for k in range(self.n_chunks):
                refill = pooled and k >= pooled
                if refill and passed[k - pooled + 1] is None:    # pool of one block: no later barrier exists yet
                    self.peer_barrier(self.ctl)
                    passed[k - pooled + 1] = main.record_event()
                with torch.cuda.stream(h2d):
                    if refill:
                        h2d.wait_event(passed[k - pooled + 1])
                    self.grad_block(k).copy_(host_grads[k], non_blocking=True)
                    arrived = h2d.record_event()
                main.wait_event(arrived)
                self.peer_barrier(self.ctl)
                passed[k] = passed[k] or main.record_event()
                kernels.pull_reduce_multi(self.table, self.grad_slab.table, self.block_off, self.ctl,
                                          chunk_flags=self.chunk_flags, first=k, count=1)
        elif pooled:
            for k in range(self.n_chunks):
                self.peer_barrier(self.ctl)
                kernels.pull_reduce_multi(self.table, self.grad_slab.table, self.block_off, self.ctl,
                                          chunk_flags=self.chunk_flags, first=k, count=1)
        else:
            self.peer_barrier(self.ctl)
            kernels.pull_reduce_multi(self.table, self.grad_slab.table, self.block_off, self.ctl,
                                      chunk_flags=self.chunk_flags)
        self.peer_barrier(self.ctl, exchange_overflow=self.sync_overflow)
        norm_sq = None
        if self.clipping:
            kernels.grad_check_multi(self.table, None, chunk_l2sq=self.chunk_l2sq, total_l2sq=self.total_l2sq,
                                     scratch=self._scratch)
            dist.all_reduce(self.total_l2sq, group=self.group)
            norm_sq = self.total_l2sq
        kernels.step_begin(self.ctl, self.scaler.cfg, norm_sq, self.chunk_flags)
        if pooled or host_params is not None:
            for k in range(self.n_chunks):
                kernels.adam_multi_push(self.table, self.ctl, self.gather_slab.table, self.block_off, first=k, count=1)
                if host_params is not None:
                    updated = main.record_event()
                    with torch.cuda.stream(d2h):
                        d2h.wait_event(updated)
                        host_params[k].copy_(self.shards[k][3], non_blocking=True)
        else:
            kernels.adam_multi_push(self.table, self.ctl, self.gather_slab.table, self.block_off)
        if host_params is not None:
            main.wait_stream(d2h)
        self.peer_barrier(self.ctl)

    def step_sharded_pull_push(self):
        """The peer-mapped sharded step with BOTH collectives inside the update kernel (two ranks): per tile the
        kernel fetches the slice of every rank's gradient block with bulk loads, averages it as the pull kernel
        does, updates in place and bulk-stores the refreshed tile to every rank's gather block, so the link-bound
        fetch of the next tiles runs under the HBM-bound update of the current one and the reduced gradient never
        touches memory.  The decision is taken first, from a probe of every rank's OWN gradient slab (see
        ``step_sharded_probe_first`` for why that is the same decision):

            barrier, probe of the own slab, barrier + agree, elx_step_begin
            elx_adam_multi_pull_push     one launch over all chunks
            barrier

        Same results as ``step_sharded_p2p``, bit for bit (tested); the per-chunk overflow words are not filled in."""
        if getattr(self, '_p2p_pool', 0) or self.clipping:
            raise RuntimeError('step_sharded_pull_push needs a block per chunk and no gradient clipping')
        self.peer_barrier(self.ctl)
        kernels.grad_check(self.grad_slab.local, ctl=self.ctl)
        self.peer_barrier(self.ctl, exchange_overflow=True)
        kernels.step_begin(self.ctl, self.scaler.cfg, None, self.chunk_flags)
        kernels.adam_multi_pull_push(self.table, self.ctl, self.grad_slab.table, self.gather_slab.table, self.block_off)
        self.peer_barrier(self.ctl)

    def step_sharded_probe_first(self, pull_ctas: int = 36):
        """The peer-mapped sharded step with the decision taken BEFORE the reduction, so that the in-place update of
        chunk k can run while chunk k + 1 is still being reduced on a second stream (the SMs split between the two
        kernels).  It rests on one property of the pull reduce-scatter — the rank average, accumulated in fp32 and
        rounded once, is non-finite exactly when one of its inputs is — so the overflow word can be formed from
        the INPUTS: every rank probes its own gradient slab (one launch, HBM speed), and the barrier ORs the words.

            barrier                  every rank's gradient blocks are written
            probe of the own slab    elx_grad_check over all blocks of this rank
            barrier + agree          found_inf OR-ed over the ranks
            decision                 elx_step_begin
            side stream:  pull(0) pull(1) pull(2) ...                     (``pull_ctas`` CTAs)
            main stream:       update+push(0) update+push(1) ...          (the remaining SMs)
            barrier                  every rank's pushes have landed

        Same results as ``step_sharded_p2p`` (tested bit for bit); the per-chunk overflow words are not filled in
        (only the global decision exists).  Pays where the two phases are bound by different things — two ranks:
        the pull by the links, the update by HBM.  Needs slabs whose padding is finite (``enable_p2p`` zeroes
        them) and one block per chunk."""
        if getattr(self, '_p2p_pool', 0) or self.clipping:
            raise RuntimeError('step_sharded_probe_first needs a block per chunk and no gradient clipping')
        main = torch.cuda.current_stream(self.device)
        side = self._side_streams()[0]
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.peer_barrier(self.ctl)
        kernels.grad_check(self.grad_slab.local, ctl=self.ctl)
        self.peer_barrier(self.ctl, exchange_overflow=True)
        kernels.step_begin(self.ctl, self.scaler.cfg, None, self.chunk_flags)
        side.wait_stream(main)
        kernels.set_tuning(pull_tma_ctas=pull_ctas, adam_tma_ctas=max(1, sms - pull_ctas))
        try:
            pulled = []
            with torch.cuda.stream(side):
                for k in range(self.n_chunks):
                    # no control block: the decision of this step is taken, and what this probe would raise
                    # must not leak into the next one
                    kernels.pull_reduce_multi(self.table, self.grad_slab.table, self.block_off, None, first=k, count=1)
                    pulled.append(side.record_event())
            for k in range(self.n_chunks):
                main.wait_event(pulled[k])
                kernels.adam_multi_push(self.table, self.ctl, self.gather_slab.table, self.block_off, first=k, count=1)
        finally:
            kernels.set_tuning(pull_tma_ctas=-1, adam_tma_ctas=-1)
        self.peer_barrier(self.ctl)

    def enable_staging(self, pool: int = 4):
        """Local staging buffers for ``step_sharded_staged``: ``pool`` slots, each with room for the W - 1
        slices of the largest shard that the other ranks hold for this rank."""
        assert hasattr(self, 'grad_slab'), 'call enable_p2p() first'
        from ._abi import ElxPeerTable
        shard_max = (max(s[0].numel() for s in self.shards) + 15) // 16 * 16
        self._stage_pool = pool
        self._stage = torch.empty(pool * self.world * shard_max, dtype=self.dtype, device=self.device)
        self._stage_tables = []
        itemsize = self._stage.element_size()
        for slot in range(pool):
            table = ElxPeerTable()
            for j in range(self.world):
                table.base[j] = (self.grad_slab.table.base[j] if j == self.grad_slab.rank else
                                 self._stage.data_ptr() + (slot * self.world + j) * shard_max * itemsize)
            table.rank, table.world = self.grad_slab.rank, self.world
            self._stage_tables.append(table)
        self._stage_zero_off = torch.zeros(self.n_chunks, dtype=torch.int64, device=self.device)
        self._copy_streams = [torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)]
        return self

    def step_sharded_staged(self):
        """Sharded step over peer-mapped memory with the copy engines moving the slices over NVLink:

            barrier                  every rank's gradient blocks are written
            per chunk k              W - 1 copies (one per other rank, rotated so that at any moment every rank
                                     reads from a different one) of this rank's slice of block k into a local
                                     staging slot, on two copy streams; then the reduce + probe kernel on local
                                     memory only (``elx_pull_reduce_multi`` with staged sources)
            barrier + agree          overflow word OR-ed over the ranks
            decision                 ``elx_step_begin``
            per chunk k              fused update on the main stream; then W copies of the refreshed shard into
                                     every rank's gather block k, on the copy streams
            barrier                  every rank's copies have landed

        Same results as ``step_sharded_p2p`` bit for bit (same reduction order and arithmetic); the difference
        is who moves the bytes."""
        rank, world = self.grad_slab.rank, self.world
        main = torch.cuda.current_stream(self.device)
        c0, c1 = self._copy_streams
        itemsize = self._stage.element_size()
        pool = self._stage_pool
        marks = self._phase_marks(main)
        self.peer_barrier(self.ctl)
        for st in self._copy_streams:
            st.wait_stream(main)
        reduce_done = [None] * self.n_chunks
        for k in range(self.n_chunks):
            slot = k % pool
            shard_elems = self.shards[k][0].numel()
            nbytes = shard_elems * itemsize
            src_off = (self._p2p_offsets[k] + rank * shard_elems) * itemsize
            table = self._stage_tables[slot]
            if k >= pool:
                for st in self._copy_streams:
                    st.wait_event(reduce_done[k - pool])    # the slot's previous user has been reduced
            for t in range(1, world):
                j = (rank + t) % world
                kernels.copy_async(table.base[j], self.grad_slab.table.base[j] + src_off, nbytes, c0 if t % 2 else c1)
            for st in self._copy_streams:
                arrived = torch.cuda.Event()
                arrived.record(st)
                main.wait_event(arrived)
            kernels.pull_reduce_multi(self.table, table, self.block_off, self.ctl, chunk_flags=self.chunk_flags,
                                      first=k, count=1, stage_off=self._stage_zero_off)
            reduce_done[k] = torch.cuda.Event()
            reduce_done[k].record(main)
        marks('reduced')
        self.peer_barrier(self.ctl, exchange_overflow=self.sync_overflow)
        norm_sq = None
        if self.clipping:
            kernels.grad_check_multi(self.table, None, chunk_l2sq=self.chunk_l2sq, total_l2sq=self.total_l2sq,
                                     scratch=self._scratch)
            dist.all_reduce(self.total_l2sq, group=self.group)
            norm_sq = self.total_l2sq
        kernels.step_begin(self.ctl, self.scaler.cfg, norm_sq, self.chunk_flags)
        for k in range(self.n_chunks):
            self.update(first=k, count=1)
            updated = torch.cuda.Event()
            updated.record(main)
            shard = self.shards[k][3]
            nbytes = shard.numel() * itemsize
            dst_off = (self._p2p_offsets[k] + rank * shard.numel()) * itemsize
            for t in range(world):
                j = (rank + t) % world
                st = c0 if t % 2 else c1
                if t < 2:
                    st.wait_event(updated)
                kernels.copy_async(self.gather_slab.table.base[j] + dst_off, shard.data_ptr(), nbytes, st)
        marks('updated')
        for st in self._copy_streams:
            main.wait_stream(st)
        marks('gathered')
        self.end_step()
        self.peer_barrier(self.ctl)

    def step_from_host(self, host_grads: Sequence[torch.Tensor], host_params: Sequence[torch.Tensor],
                       speculative: bool = False):
        """A whole step with host buffers on both ends: ``host_grads[k]`` (pinned, shard_size elements of
        the chunk dtype) holds the reduced gradients of shard k; ``host_params[k]`` (pinned) receives the
        updated low-precision parameters.  Copies in, probes, updates and copies out are pipelined per
        chunk on three streams; fp32 master and moments never leave the device.  No parameter is updated
        before the last gradient has been probed, so the two directions of the link cannot overlap;
        ``speculative`` (after ``enable_speculation``) lifts that, see ``_step_from_host_speculative``."""
        assert len(host_grads) == self.n_chunks and len(host_params) == self.n_chunks
        if speculative:
            assert self._sets is not None, 'enable_speculation() first'
            return self._step_from_host_speculative(host_grads, host_params)
        main = torch.cuda.current_stream(self.device)
        h2d, d2h = self._side_streams()
        h2d.wait_stream(main)
        for k, src in enumerate(host_grads):
            with torch.cuda.stream(h2d):
                self._grad_home(k).copy_(src, non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(h2d)
            main.wait_event(arrived)
            self.probe_one(k)
        self.begin_step()
        for k, dst in enumerate(host_params):
            self.update(first=k, count=1)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(d2h):
                d2h.wait_event(done)
                dst.copy_(self.shards[k][3], non_blocking=True)
        self.end_step()
        main.wait_stream(d2h)

    # ------------------------------------------------------------------ single-pass step over two state sets

    def enable_single_pass(self):
        """Prepare the single-pass step: a second set of master and moment arrays per shard (12 bytes per element
        more) and its descriptor table.  ``step_single_pass`` / ``step_sharded_single_pass`` then read the current
        set and write the other one; which one is current is a word of the device control block, so the host never
        has to know (``current_shards`` reads it back for checkpoints and tests)."""
        assert self.table.descs_dev is not None, 'finalize() first'
        if self._sets is not None:
            return self
        if self.clipping or self.table.host_resident:
            raise RuntimeError('the single-pass step is for device-resident shards and no gradient clipping '
                               '(the clip factor needs every gradient before the first update)')
        other = kernels.ChunkTable(self.device, self.dtype)
        other_shards = []
        for k, (master, exp_avg, exp_avg_sq, lowp, n_valid) in enumerate(self.shards):
            twin = (master.clone(), exp_avg.clone(), exp_avg_sq.clone())
            other.add_chunk(twin[0], twin[1], twin[2], lowp, n_valid, self.table._segs_of(k), grad_src=self.grad_srcs[k])
            other_shards.append((twin[0], twin[1], twin[2], lowp, n_valid))
        other.finalize()
        self._sets = ((self.table, self.shards), (other, other_shards))
        return self

    def current_shards(self):
        """The shard tuples of the state set that is current (synchronises: reads the control block)."""
        if self._sets is None:
            return self.shards
        return self._sets[int(self.ctl.read().cur_set)][1]

    def normalize_sets(self):
        """Make the current state set "set 0" again (``self.table`` / ``self.shards``), so that the in-place paths
        (``step``, ``step_from_host``, checkpoints) see the live state after single-pass steps.  Synchronises."""
        if self._sets is None:
            return
        c = self.ctl.read()
        if c.cur_set:
            self._sets = (self._sets[1], self._sets[0])
            self._sets[0][0].set_hyper_from(self._sets[1][0])
            self.table, self.shards = self._sets[0]
            c.cur_set = 0
            self.ctl.write(c)

    def step_single_pass(self):
        """One rank's step as ONE pass over memory (28 bytes per element with 16-bit gradients, no separate probe):

            elx_step_begin_optimistic    decision on the assumption of no overflow
            elx_adam_multi_single_pass   unscale + inf/nan detection + Adam/AdamW + working copy, out of place
            elx_step_commit              clean: the sets change roles; overflow: the decision is taken back -> skip
            elx_adam_multi_repair        only after an overflow: working copies rebuilt from the untouched set

        Four launches, nothing read back.  Gradients sit, unprobed, where the update reads them (the shards or the
        sources given to ``add_shard``)."""
        (t0, _), (t1, _) = self._sets
        t1.set_hyper_from(t0)
        kernels.step_begin_optimistic(self.ctl, self.scaler.cfg, self.chunk_flags)
        kernels.adam_multi_single_pass(t0, t1, self.ctl, self.chunk_flags)
        kernels.step_commit(self.ctl, self.scaler.cfg, self.chunk_flags)
        kernels.adam_multi_repair(t0, t1, self.ctl)

    def enable_multicast(self, chunk_sizes: Sequence[int], timeout_ms: int = 20000):
        """Slabs for ``step_sharded_single_pass``: like ``enable_p2p`` (a gradient block and a gather block of
        ``chunk_sizes[k]`` elements per chunk on every rank), but in symmetric memory bound to an NVLink multicast
        object, so that the switch can add up the ranks' gradient blocks and deliver one store to all gather blocks."""
        from .peer import PeerBarrier, SymmBuffer
        assert len(chunk_sizes) == self.n_chunks
        for k, size in enumerate(chunk_sizes):
            if size != self.shards[k][0].numel() * self.world:
                raise ValueError(f'chunk {k}: chunk size {size} is not world x shard size')
        offsets, total = [], 0
        for size in chunk_sizes:
            offsets.append(total)
            total += (size + 15) // 16 * 16
        self._p2p_pool = 0
        self._p2p_sizes = list(chunk_sizes)
        self._p2p_offsets = offsets
        self.block_off = torch.tensor(offsets, dtype=torch.int64, device=self.device)
        self.grad_slab = SymmBuffer(total, self.dtype, self.device, self.group)
        self.gather_slab = SymmBuffer(total, self.dtype, self.device, self.group)
        self.peer_barrier = PeerBarrier(self.device, self.group, timeout_ms)
        return self

    def switch_reduced_gradients(self) -> List[torch.Tensor]:
        """What ``step_sharded_single_pass`` will consume, made visible: for every chunk the SUM over the ranks of
        this rank's slice of the gradient blocks as the NVLink switch forms it (the kernel multiplies it by 1/W).
        For checks and tests; the step itself never stores these values.  Every rank's blocks must be written and
        the shard sizes multiples of 8."""
        out = []
        itemsize = self.grad_slab.local.element_size()
        for k, shard in enumerate(self.shards):
            n = shard[0].numel()
            dst = torch.empty(n, dtype=self.dtype, device=self.device)
            kernels.multimem_reduce(dst, self.grad_slab.mc_ptr + (self._p2p_offsets[k] + self.grad_slab.rank * n) * itemsize)
            out.append(dst)
        return out

    def step_sharded_single_pass(self, host_grads: Optional[Sequence[torch.Tensor]] = None,
                                 host_params: Optional[Sequence[torch.Tensor]] = None):
        """The sharded step with reduce-scatter, update and all-gather in ONE kernel, tile by tile, through the
        NVLink switch (after ``enable_single_pass`` and ``enable_multicast``):

            barrier                      every rank's gradient blocks are written
            elx_step_begin_optimistic
            elx_adam_multi_single_pass   per tile: sum of all ranks' gradient tiles fetched from the switch
                                         (multimem.ld_reduce) -> 1/W -> unscale, inf/nan detection, Adam/AdamW ->
                                         working-copy tile stored once to all ranks' gather blocks (multimem.st)
            barrier + agree              overflow words OR-ed over the ranks; all stores have landed
            elx_step_commit              every rank adopts the update, or none does
            elx_adam_multi_repair        only after an overflow: old parameters re-sent
            barrier                      (the gather blocks are final)

        Seven launches, no NCCL call, nothing read back by the host.  Each direction of a rank's links carries
        about (W + 1) / W of the chunk bytes instead of 2 (W - 1) / W; the reduced gradients never touch HBM.

        With ``host_grads`` / ``host_params`` (pinned; chunk_size and shard_size elements per chunk) the kernel is
        launched chunk by chunk behind a barrier each: block k is filled from the host while earlier chunks are in
        flight, and shard k leaves for the host right behind its update — before the step is known to be clean, so
        after an overflow the rebuilt shards are sent again (the host reads the result once, at the end)."""
        (t0, _), (t1, _) = self._sets
        t1.set_hyper_from(t0)
        fused = dict(grads_table=self.grad_slab.table, gather_table=self.gather_slab.table, block_off=self.block_off,
                     grads_mc=self.grad_slab.mc_ptr, gather_mc=self.gather_slab.mc_ptr)
        if host_grads is None and host_params is None:
            self.peer_barrier(self.ctl)
            kernels.step_begin_optimistic(self.ctl, self.scaler.cfg, self.chunk_flags)
            kernels.adam_multi_single_pass(t0, t1, self.ctl, self.chunk_flags, **fused)
        else:
            main = torch.cuda.current_stream(self.device)
            h2d, d2h = self._side_streams()
            h2d.wait_stream(main)
            d2h.wait_stream(main)
            kernels.step_begin_optimistic(self.ctl, self.scaler.cfg, self.chunk_flags)
            for k in range(self.n_chunks):
                if host_grads is not None:
                    with torch.cuda.stream(h2d):
                        self.grad_block(k).copy_(host_grads[k], non_blocking=True)
                        arrived = h2d.record_event()
                    main.wait_event(arrived)
                self.peer_barrier(self.ctl)    # chunk k's gradients are in place on every rank
                kernels.adam_multi_single_pass(t0, t1, self.ctl, self.chunk_flags, first=k, count=1, **fused)
                if host_params is not None:
                    updated = main.record_event()
                    with torch.cuda.stream(d2h):
                        d2h.wait_event(updated)
                        host_params[k].copy_(self.shards[k][3], non_blocking=True)
        self.peer_barrier(self.ctl, exchange_overflow=True)
        kernels.step_commit(self.ctl, self.scaler.cfg, self.chunk_flags)
        kernels.adam_multi_repair(t0, t1, self.ctl, gather_table=self.gather_slab.table, block_off=self.block_off)
        self.peer_barrier(self.ctl)
        if host_params is not None:
            main.wait_stream(d2h)
            if self.ctl.read().repair:    # the step's result, read by the host (synchronises)
                for k, dst in enumerate(host_params):
                    dst.copy_(self.shards[k][3], non_blocking=True)
                main.synchronize()

    def step_sharded_overlapped(self, pull_ctas: int = 36):
        """The peer-mapped sharded step (``enable_p2p`` slabs) with the reduction of later chunks running WHILE
        earlier chunks are updated — possible because the update goes out of place (``enable_single_pass``) and is
        adopted only after every chunk turned out clean:

            barrier                      every rank's gradient blocks are written
            elx_step_begin_optimistic
            side stream:  pull(0) pull(1) pull(2) ...          (reduce-scatter + probe, ``pull_ctas`` CTAs)
            main stream:       update+push(0) update+push(1) ...   (single-pass kernel on the remaining SMs)
            barrier + agree, elx_step_commit, elx_adam_multi_repair, barrier

        Worth it where the two phases are bound by different things (two ranks: the pull by the links, the update by
        HBM); where both are link-bound the links are already busy in both directions in either phase."""
        (t0, _), (t1, _) = self._sets
        t1.set_hyper_from(t0)
        main = torch.cuda.current_stream(self.device)
        side = self._side_streams()[0]
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.peer_barrier(self.ctl)
        kernels.step_begin_optimistic(self.ctl, self.scaler.cfg, self.chunk_flags)
        side.wait_stream(main)
        kernels.set_tuning(pull_tma_ctas=pull_ctas, adam_tma_ctas=max(1, sms - pull_ctas))
        try:
            pulled = []
            with torch.cuda.stream(side):
                for k in range(self.n_chunks):
                    kernels.pull_reduce_multi(self.table, self.grad_slab.table, self.block_off, self.ctl,
                                              chunk_flags=self.chunk_flags, first=k, count=1)
                    pulled.append(side.record_event())
            for k in range(self.n_chunks):
                main.wait_event(pulled[k])
                kernels.adam_multi_single_pass(t0, t1, self.ctl, self.chunk_flags, first=k, count=1,
                                               grads_table=self.grad_slab.table, gather_table=self.gather_slab.table,
                                               block_off=self.block_off)
        finally:
            kernels.set_tuning(pull_tma_ctas=-1, adam_tma_ctas=-1)
        self.peer_barrier(self.ctl, exchange_overflow=True)
        kernels.step_commit(self.ctl, self.scaler.cfg, self.chunk_flags)
        kernels.adam_multi_repair(t0, t1, self.ctl, gather_table=self.gather_slab.table, block_off=self.block_off)
        self.peer_barrier(self.ctl)

    # ------------------------------------------------------------------ single-pass step with host buffers

    def enable_speculation(self):
        """Prepare ``step_from_host(..., speculative=True)``: the two state sets of the single-pass step."""
        if self.world > 1:
            raise RuntimeError('the host-buffer form of the single-pass step is for one rank')
        return self.enable_single_pass()

    def _step_from_host_speculative(self, host_grads, host_params):
        """The single-pass step fed from host buffers: every chunk is updated (out of place, with the inf/nan
        test inside the update kernel) as soon as its gradients have arrived, and its parameters leave for the
        host while later gradients still come in — PCIe busy in both directions at once.  If an overflow turns
        up the update is not adopted (``elx_step_commit``), the working copies are rebuilt from the untouched set
        (``elx_adam_multi_repair``) and sent out again.  The host reads the step's result once, at the end.
        Returns True if the step was applied."""
        (t0, _), (t1, _) = self._sets
        t1.set_hyper_from(t0)
        main = torch.cuda.current_stream(self.device)
        h2d, d2h = self._side_streams()
        kernels.step_begin_optimistic(self.ctl, self.scaler.cfg, self.chunk_flags)
        h2d.wait_stream(main)
        d2h.wait_stream(main)
        for k, src in enumerate(host_grads):
            lowp = self.shards[k][3]
            with torch.cuda.stream(h2d):
                self._grad_home(k).copy_(src, non_blocking=True)
                arrived = h2d.record_event()
            main.wait_event(arrived)
            kernels.adam_multi_single_pass(t0, t1, self.ctl, self.chunk_flags, first=k, count=1)
            done = main.record_event()
            with torch.cuda.stream(d2h):
                d2h.wait_event(done)
                host_params[k].copy_(lowp, non_blocking=True)
        kernels.step_commit(self.ctl, self.scaler.cfg, self.chunk_flags)
        kernels.adam_multi_repair(t0, t1, self.ctl)
        main.wait_stream(d2h)
        result = self.ctl.read()    # the step's result, read by the host (synchronises)
        if result.repair:
            # late overflow: the parameters that left were those of the dropped update; send the rebuilt ones
            for k, dst in enumerate(host_params):
                dst.copy_(self.shards[k][3], non_blocking=True)
            main.synchronize()
        return not result.skip

    # ------------------------------------------------------------------ shards in host memory, streamed

    def enable_streaming(self, slots: int = 3):
        """Prepare ``step_streamed``: ``slots`` device staging sets (master, two moments, working copy) of the
        largest shard's size, and a second descriptor table whose entry k points into set ``k % slots``."""
        assert self.table.descs_dev is not None, 'finalize() first'
        assert self.table.host_resident, 'streaming is for shards kept in pinned host memory'
        size = max(s[0].numel() for s in self.shards)
        f32 = lambda: torch.empty(size, dtype=torch.float32, device=self.device)    # noqa: E731
        self._slots = [(f32(), f32(), f32(), torch.empty(size, dtype=self.dtype, device=self.device))
                       for _ in range(slots)]
        self._stage_table = kernels.ChunkTable(self.device, self.dtype)
        self._streamed = []    # per shard: its arrays are in host memory and travel through a staging set
        for k, (master, exp_avg, exp_avg_sq, lowp, n_valid) in enumerate(self.shards):
            n = master.numel()
            on_host = kernels.is_mapped_host(master)
            assert all(kernels.is_mapped_host(t) == on_host for t in (exp_avg, exp_avg_sq, lowp)), \
                'the four arrays of a shard live in the same kind of memory'
            self._streamed.append(on_host)
            if on_host:
                slot = self._slots[k % slots]
                self._stage_table.add_chunk(slot[0][:n], slot[1][:n], slot[2][:n], slot[3][:n], n_valid,
                                            self.table._segs_of(k))
            else:    # a device-resident shard is updated where it is
                self._stage_table.add_chunk(master, exp_avg, exp_avg_sq, lowp, n_valid, self.table._segs_of(k),
                                            grad_src=self.grad_srcs[k])
        self._stage_table.finalize()
        self._slot_free = [None] * slots

    def step_streamed(self):
        """``step`` after ``enable_streaming`` (kept as a name of its own for call sites that want to say so)."""
        assert self._slots is not None, 'enable_streaming() first'
        self.step()

    def _update_streamed(self):
        """The update for shards in pinned host memory, with the copy engines instead of kernel accesses over
        PCIe: chunk by chunk, the four arrays are copied into a device staging set (h2d stream), updated there
        by the same fused kernel (main stream) and copied back (d2h stream); with three staging sets the three
        stages overlap, so the update takes what the slower PCIe direction takes (14 bytes per element each way
        with 16-bit gradients).  Gradients must already sit, probed, in the host shards."""
        slots = len(self._slots)
        main = torch.cuda.current_stream(self.device)
        h2d, d2h = self._side_streams()
        self._stage_table.set_hyper_from(self.table)
        h2d.wait_stream(main)
        for k, host in enumerate(self.shards):
            if not self._streamed[k]:
                kernels.adam_multi(self._stage_table, self.ctl, first=k, count=1)
                continue
            n = host[0].numel()
            stage = [t[:n] for t in self._slots[k % slots]]
            with torch.cuda.stream(h2d):
                if self._slot_free[k % slots] is not None:
                    h2d.wait_event(self._slot_free[k % slots])    # the set's previous tenant has been copied out
                for dst, src in zip(stage, host[:4]):
                    dst.copy_(src, non_blocking=True)
                arrived = h2d.record_event()
            main.wait_event(arrived)
            kernels.adam_multi(self._stage_table, self.ctl, first=k, count=1)
            updated = main.record_event()
            with torch.cuda.stream(d2h):
                d2h.wait_event(updated)
                for dst, src in zip(host[:4], stage):
                    dst.copy_(src, non_blocking=True)
                self._slot_free[k % slots] = d2h.record_event()
        main.wait_stream(d2h)

    # ------------------------------------------------------------------ introspection (synchronising)

    def read_control(self):
        return self.ctl.read()

    def check_status(self):
        """Raise if a kernel reported an anomaly (sticky status word).  Synchronises, so it is called where the
        host waits for the device anyway (``loss_scale``, ``state_dict``, the end of a benchmark).  While the
        time-out bit is set every step is skipped on the device (``elx_step_begin``), on all ranks."""
        c = self.ctl.read()
        if c.status:
            raise RuntimeError(f'elixir_b200 kernels reported status {c.status:#x} '
                               '(1: non-finite gradient met on an applied step, 2: descriptor table mismatch, '
                               '4: a bounded wait on a copy or on another rank expired; '
                               f'{c.forced_skips} step(s) were skipped because of it)')
