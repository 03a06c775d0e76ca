"""Tensor-level bindings of the C ABI: every function takes torch tensors, passes raw device pointers
and the current CUDA stream to ``libelixir_b200.so`` and raises on a non-zero status.

torch is plumbing here (it owns the memory and the streams); no arithmetic of the optimizer step is
done by a torch operator.
"""
import ctypes
from typing import List, Optional, Sequence, Tuple

import torch

from . import _abi, _lib
from ._abi import ElxChunkDesc, ElxCtl, ElxHyper, ElxScalerCfg, ElxSeg

_DTYPE_CODES = {torch.float16: _abi.F16, torch.bfloat16: _abi.BF16, torch.float32: _abi.F32}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODES[dtype]
    except KeyError:
        raise TypeError(f'elixir_b200 supports float16, bfloat16 and float32 chunks, not {dtype}') from None


def is_mapped_host(t: torch.Tensor) -> bool:
    """Page-locked host memory: under unified addressing a kernel reaches it through the same pointer."""
    return t.device.type == 'cpu' and t.is_pinned()


def _check_tensor(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None, mapped_host: bool = False):
    """``mapped_host``: the argument may also be a pinned host tensor (shard data of a host-resident chunk);
    the kernels then read and write it over PCIe.  Pageable host memory is never accepted."""
    if not isinstance(t, torch.Tensor):
        raise TypeError(f'{name} must be a tensor')
    if not t.is_contiguous():
        raise ValueError(f'{name} must be contiguous')
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f'{name} must be {dtype}, got {t.dtype}')
    if t.is_cuda or _lib.host_memory_backend():
        return
    if mapped_host and is_mapped_host(t):
        return
    raise RuntimeError(f'{name} lives on {t.device}: the elixir_b200 kernels run on CUDA tensors (and, for shard '
                       'data, pinned host tensors) only; there is no CPU path')


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(t: Optional[torch.Tensor]):
    if t is not None and t.is_cuda:
        return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
    return None


def _home(*tensors) -> Optional[torch.Tensor]:
    """The first CUDA tensor among the arguments: its device runs the kernel, its current stream orders it."""
    for t in tensors:
        if t is not None and t.is_cuda:
            return t
    if _lib.host_memory_backend():
        return None
    raise RuntimeError('at least one argument must live on a CUDA device (flag, control block or data)')


class _DeviceGuard:
    """Make the tensor's device current for the duration of a native call."""

    def __init__(self, t: Optional[torch.Tensor]):
        self._ctx = torch.cuda.device(t.device) if (t is not None and t.is_cuda) else None

    def __enter__(self):
        if self._ctx is not None:
            self._ctx.__enter__()

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)


def n_tiles(n_elems: int) -> int:
    return (n_elems + _abi.TILE - 1) // _abi.TILE


def set_tuning(**knobs):
    """``set_tuning(adam_threads=256, probe_unroll=8, ...)``; a negative value restores a default."""
    for name, value in knobs.items():
        _lib.check(_lib.get().elx_set_tuning(name.encode(), int(value)), f'elx_set_tuning({name})')


# ---------------------------------------------------------------------------------------------------
# control block
# ---------------------------------------------------------------------------------------------------


def scaler_cfg(dynamic=True,
               growth_factor=2.0,
               backoff_factor=0.5,
               min_scale=1.0,
               max_scale=2.0**24,
               growth_interval=1000,
               hysteresis=2,
               max_norm=0.0) -> ElxScalerCfg:
    return ElxScalerCfg(int(bool(dynamic)), float(growth_factor), float(backoff_factor),
                        float(min_scale) if min_scale else 0.0,
                        float(max_scale) if max_scale else 0.0, int(growth_interval), int(hysteresis),
                        float(max_norm))


class ControlBlock:
    """The device-resident ``ElxCtl`` of one optimizer, held in a 32-word int32 tensor."""

    WORDS = ctypes.sizeof(ElxCtl) // 4

    def __init__(self, device, initial_scale: float = 1.0):
        self.tensor = torch.zeros(self.WORDS, dtype=torch.int32, device=device)
        with _DeviceGuard(self.tensor):
            _lib.check(_lib.get().elx_ctl_init(_ptr(self.tensor), float(initial_scale), _stream(self.tensor)),
                       'elx_ctl_init')

    @property
    def ptr(self):
        return _ptr(self.tensor)

    @property
    def scale(self) -> torch.Tensor:
        """0-dim float32 view of the loss scale; multiply the loss by it without a host read."""
        return self.tensor[ElxCtl.scale.offset // 4:ElxCtl.scale.offset // 4 + 1].view(torch.float32)[0]

    @property
    def found_inf(self) -> torch.Tensor:
        """1-element int32 view of the overflow word (for the cross-rank MAX all-reduce)."""
        return self.tensor[ElxCtl.found_inf.offset // 4:ElxCtl.found_inf.offset // 4 + 1]

    def read(self) -> ElxCtl:
        """Host copy of the block.  Synchronises; meant for logging, tests and checkpoints."""
        raw = self.tensor.cpu().numpy().tobytes()
        return ElxCtl.from_buffer_copy(raw)

    def write(self, ctl: ElxCtl):
        raw = torch.frombuffer(bytearray(bytes(ctl)), dtype=torch.int32)
        self.tensor.copy_(raw)


def step_begin(ctl: ControlBlock, cfg: ElxScalerCfg, norm_sq: Optional[torch.Tensor] = None,
               chunk_flags: Optional[torch.Tensor] = None):
    """The device-side decision of a step (``elx_step_begin``).  ``chunk_flags`` (the per-chunk overflow words)
    are cleared by the same launch, as the reference clears ``Chunk.overflow`` at this point."""
    if norm_sq is not None:
        _check_tensor(norm_sq, 'norm_sq', torch.float32)
    if chunk_flags is not None:
        _check_tensor(chunk_flags, 'chunk_flags', torch.int32)
    with _DeviceGuard(ctl.tensor):
        _lib.check(_lib.get().elx_step_begin(ctl.ptr, cfg, _ptr(norm_sq), _ptr(chunk_flags),
                                             chunk_flags.numel() if chunk_flags is not None else 0,
                                             _stream(ctl.tensor)), 'elx_step_begin')


# ---------------------------------------------------------------------------------------------------
# single-shard entry points
# ---------------------------------------------------------------------------------------------------


def grad_check(g: torch.Tensor,
               n_valid: Optional[int] = None,
               flag: Optional[torch.Tensor] = None,
               ctl: Optional[ControlBlock] = None,
               l2sq: Optional[torch.Tensor] = None,
               scratch: Optional[torch.Tensor] = None):
    """Probe ``g[:n_valid]`` for inf/nan (``flag`` / ``ctl.found_inf`` are raised, never cleared) and,
    when ``l2sq`` is given, write its sum of squares there."""
    _check_tensor(g, 'g', mapped_host=True)
    n_valid = g.numel() if n_valid is None else int(n_valid)
    if n_valid > g.numel():
        raise ValueError('n_valid exceeds the tensor')
    if flag is not None:
        _check_tensor(flag, 'flag', torch.int32)
    if l2sq is not None:
        _check_tensor(l2sq, 'l2sq', torch.float32)
        if scratch is None:
            raise ValueError('l2sq needs a scratch tensor of probe_scratch_elems(n_tiles) floats')
        _check_tensor(scratch, 'scratch', torch.float32)
    home = _home(g, flag, ctl.tensor if ctl else None, l2sq)
    with _DeviceGuard(home):
        _lib.check(
            _lib.get().elx_grad_check(_ptr(g), dtype_code(g.dtype), n_valid, _ptr(flag), ctl.ptr if ctl else None,
                                      _ptr(l2sq), _ptr(scratch), scratch.numel() if scratch is not None else 0,
                                      _stream(home)), 'elx_grad_check')


def reduce_epilogue(src: torch.Tensor,
                    dst: torch.Tensor,
                    n_valid: Optional[int] = None,
                    flag: Optional[torch.Tensor] = None,
                    ctl: Optional[ControlBlock] = None,
                    l2sq: Optional[torch.Tensor] = None,
                    scratch: Optional[torch.Tensor] = None):
    """``dst.copy_(src)`` fused with the probe of ``src[:n_valid]``."""
    _check_tensor(src, 'src', mapped_host=True)
    _check_tensor(dst, 'dst', src.dtype, mapped_host=True)
    if src.numel() != dst.numel():
        raise ValueError('src and dst differ in size')
    n_valid = src.numel() if n_valid is None else int(n_valid)
    if flag is not None:
        _check_tensor(flag, 'flag', torch.int32)
    if l2sq is not None:
        _check_tensor(l2sq, 'l2sq', torch.float32)
        _check_tensor(scratch, 'scratch', torch.float32)
    home = _home(src, dst, flag, ctl.tensor if ctl else None)
    with _DeviceGuard(home):
        _lib.check(
            _lib.get().elx_reduce_epilogue(_ptr(src), _ptr(dst), dtype_code(src.dtype), src.numel(), n_valid,
                                           _ptr(flag), ctl.ptr if ctl else None, _ptr(l2sq), _ptr(scratch),
                                           scratch.numel() if scratch is not None else 0, _stream(home)),
            'elx_reduce_epilogue')


def widen(src: torch.Tensor, dst: torch.Tensor):
    """``dst = src.float()`` for a 16-bit ``src`` (``elx_widen``): the block that goes into an fp32 reduction."""
    _check_tensor(src, 'src')
    _check_tensor(dst, 'dst', torch.float32)
    if src.numel() != dst.numel():
        raise ValueError('src and dst differ in size')
    home = _home(src, dst)
    with _DeviceGuard(home):
        _lib.check(_lib.get().elx_widen(_ptr(src), dtype_code(src.dtype), _ptr(dst), src.numel(), _stream(home)),
                   'elx_widen')


def narrow_epilogue(src: torch.Tensor,
                    dst: torch.Tensor,
                    n_valid: Optional[int] = None,
                    flag: Optional[torch.Tensor] = None,
                    ctl: Optional[ControlBlock] = None):
    """``dst.copy_(src)`` from fp32 to the 16-bit ``dst`` fused with the probe of the rounded ``dst[:n_valid]``
    (``elx_narrow_epilogue``): the fp32 rank average of this rank's slice lands in its shard."""
    _check_tensor(src, 'src', torch.float32)
    _check_tensor(dst, 'dst', mapped_host=True)
    if src.numel() != dst.numel():
        raise ValueError('src and dst differ in size')
    n_valid = src.numel() if n_valid is None else int(n_valid)
    if flag is not None:
        _check_tensor(flag, 'flag', torch.int32)
    home = _home(src, dst, flag, ctl.tensor if ctl else None)
    with _DeviceGuard(home):
        _lib.check(
            _lib.get().elx_narrow_epilogue(_ptr(src), _ptr(dst), dtype_code(dst.dtype), src.numel(), n_valid, _ptr(flag),
                                           ctl.ptr if ctl else None, _stream(home)), 'elx_narrow_epilogue')


def hyper(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adamw_mode=True, bias_correction=True) -> ElxHyper:
    return ElxHyper(float(lr), float(betas[0]), float(betas[1]), float(eps), float(weight_decay), int(bool(adamw_mode)),
                    int(bool(bias_correction)), 0)


def adam_chunk(master: torch.Tensor,
               exp_avg: torch.Tensor,
               exp_avg_sq: torch.Tensor,
               grad_param: torch.Tensor,
               h: ElxHyper,
               ctl: ControlBlock,
               n_valid: Optional[int] = None):
    """Fused step on one shard with one hyper-parameter set (see ``elx_adam_chunk``)."""
    for name, t in (('master', master), ('exp_avg', exp_avg), ('exp_avg_sq', exp_avg_sq)):
        _check_tensor(t, name, torch.float32)
    _check_tensor(grad_param, 'grad_param')
    n = master.numel()
    if not (exp_avg.numel() == exp_avg_sq.numel() == grad_param.numel() == n):
        raise ValueError('master, moments and the low-precision shard differ in size')
    n_valid = n if n_valid is None else int(n_valid)
    with _DeviceGuard(master):
        _lib.check(
            _lib.get().elx_adam_chunk(_ptr(master), _ptr(exp_avg), _ptr(exp_avg_sq), _ptr(grad_param),
                                      dtype_code(grad_param.dtype), n_valid, n, h, ctl.ptr, _stream(master)),
            'elx_adam_chunk')


def cast_copyback(master: torch.Tensor, dst: torch.Tensor):
    _check_tensor(master, 'master', torch.float32, mapped_host=True)
    _check_tensor(dst, 'dst', mapped_host=True)
    if master.numel() != dst.numel():
        raise ValueError('master and dst differ in size')
    if _lib.host_memory_backend():
        home = None
    elif master.is_cuda or dst.is_cuda:
        home = master if master.is_cuda else dst
    else:
        home = torch.empty(0, device='cuda')    # both ends in mapped host memory: run on the current device
    with _DeviceGuard(home):
        _lib.check(
            _lib.get().elx_cast_copyback(_ptr(master), _ptr(dst), dtype_code(dst.dtype), master.numel(),
                                         _stream(home)), 'elx_cast_copyback')


# ---------------------------------------------------------------------------------------------------
# descriptor tables and the multi-chunk launches
# ---------------------------------------------------------------------------------------------------


def _struct_array_to_tensor(arr, device) -> torch.Tensor:
    raw = bytearray(bytes(arr))
    if not raw:
        raw = bytearray(8)
    pad = (-len(raw)) % 8
    raw.extend(b'\0' * pad)
    return torch.frombuffer(raw, dtype=torch.int64).to(device)


class ChunkTable:
    """Device tables (descriptors, segments, hyper-parameters) of one rank's chunk shards.

    ``add_chunk`` records a shard with its parameter segments; ``finalize`` uploads the descriptor
    and segment tables once; ``set_hyper`` uploads the (small) hyper-parameter table whenever a
    value changed, from a ring of pinned staging buffers so that no upload ever waits for the host.
    """

    _RING = 4

    def __init__(self, device, dtype: torch.dtype):
        self.device = torch.device(device)
        self.dtype = dtype
        self.code = dtype_code(dtype)
        self._descs: List[ElxChunkDesc] = []
        self._segs: List[ElxSeg] = []
        self._keep = []    # tensors referenced by raw pointer
        self.tile_begin: List[int] = [0]
        self.descs_dev = None
        self.segs_dev = None
        self.hyper_dev = None
        self.n_groups = 0
        self._hyper_bytes = None
        self._ring = []
        self._ring_events = []
        self._ring_pos = 0
        self.host_resident = False    # some shard data lives in pinned host memory

    @property
    def n_chunks(self) -> int:
        return len(self._descs)

    def add_chunk(self,
                  master: torch.Tensor,
                  exp_avg: torch.Tensor,
                  exp_avg_sq: torch.Tensor,
                  grad_param: torch.Tensor,
                  n_valid: int,
                  segments: Sequence[Tuple[int, int, int]] = (),
                  grad_src: Optional[torch.Tensor] = None) -> int:
        """``grad_src``: where the kernels read this shard's gradient (same size and dtype as ``grad_param``),
        when it is not copied into ``grad_param`` before the step; the working copy is written to
        ``grad_param`` either way."""
        if self.descs_dev is not None:
            raise RuntimeError('the table is already finalized')
        for name, t in (('master', master), ('exp_avg', exp_avg), ('exp_avg_sq', exp_avg_sq)):
            _check_tensor(t, name, torch.float32, mapped_host=True)
        _check_tensor(grad_param, 'grad_param', self.dtype, mapped_host=True)
        n = master.numel()
        if not (exp_avg.numel() == exp_avg_sq.numel() == grad_param.numel() == n):
            raise ValueError('master, moments and the low-precision shard differ in size')
        if not 0 <= n_valid <= n:
            raise ValueError('n_valid outside [0, n_shard]')
        if grad_src is not None:
            _check_tensor(grad_src, 'grad_src', self.dtype, mapped_host=True)
            if grad_src.numel() != n:
                raise ValueError('grad_src and the shard differ in size')
        for t in (master, exp_avg, exp_avg_sq, grad_param) + ((grad_src,) if grad_src is not None else ()):
            if is_mapped_host(t) and not _lib.host_memory_backend():
                self.host_resident = True    # at least one array is reached over PCIe: see adam_multi
            elif t.device != self.device and not _lib.host_memory_backend():
                raise ValueError(f'tensor on {t.device}, table on {self.device}')
        merged: List[List[int]] = []
        last_end = 0
        for begin, end, group in segments:
            if not (last_end <= begin < end <= n_valid):
                raise ValueError(f'segment [{begin}, {end}) is unsorted, empty, overlapping or outside [0, n_valid)')
            if merged and merged[-1][1] == begin and merged[-1][2] == group:
                merged[-1][1] = end
            else:
                merged.append([begin, end, group])
            last_end = end
        desc = ElxChunkDesc(master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), grad_param.data_ptr(), n,
                            n_valid, self.tile_begin[-1], len(self._segs), len(merged), self.code, 0,
                            grad_src.data_ptr() if grad_src is not None else None)
        self._descs.append(desc)
        self._segs.extend(ElxSeg(b, e, g, 0) for b, e, g in merged)
        self._keep.append((master, exp_avg, exp_avg_sq, grad_param, grad_src))
        self.tile_begin.append(self.tile_begin[-1] + n_tiles(n))
        return len(self._descs) - 1

    def _segs_of(self, index: int):
        """(begin, end, group) of descriptor ``index`` as registered (neighbours merged)."""
        d = self._descs[index]
        return [(s.begin, s.end, s.group) for s in self._segs[d.seg_first:d.seg_first + d.seg_count]]

    def finalize(self):
        self.descs_dev = _struct_array_to_tensor((ElxChunkDesc * len(self._descs))(*self._descs), self.device)
        self.segs_dev = _struct_array_to_tensor((ElxSeg * len(self._segs))(*self._segs), self.device)
        return self

    def tiles(self, first: int = 0, count: Optional[int] = None) -> int:
        count = self.n_chunks - first if count is None else count
        return self.tile_begin[first + count] - self.tile_begin[first]

    def set_hyper_from(self, other: 'ChunkTable'):
        """Use the hyper-parameter table of ``other`` (same device): nothing is uploaded twice."""
        self.hyper_dev, self.n_groups = other.hyper_dev, other.n_groups

    def set_hyper(self, groups: Sequence[ElxHyper]):
        if len(groups) > _abi.MAX_GROUPS:
            raise ValueError(f'at most {_abi.MAX_GROUPS} param groups are supported')
        raw = bytes((ElxHyper * len(groups))(*groups))
        if raw == self._hyper_bytes:
            return
        if self.hyper_dev is None or self.n_groups != len(groups):
            self.hyper_dev = torch.zeros(max(1, len(groups)) * 8, dtype=torch.int32, device=self.device)
            self._ring = []
        self.n_groups = len(groups)
        src = torch.frombuffer(bytearray(raw), dtype=torch.int32) if raw else None
        if src is not None:
            if self.device.type == 'cuda':
                if not self._ring:
                    self._ring = [torch.empty_like(src).pin_memory() for _ in range(self._RING)]
                    self._ring_events = [None] * self._RING
                slot = self._ring_pos % self._RING
                self._ring_pos += 1
                if self._ring_events[slot] is not None:
                    self._ring_events[slot].synchronize()
                self._ring[slot].copy_(src)
                self.hyper_dev.copy_(self._ring[slot], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream(self.device))
                self._ring_events[slot] = ev
            else:
                self.hyper_dev.copy_(src)
        self._hyper_bytes = raw


def grad_check_multi(table: ChunkTable,
                     ctl: Optional[ControlBlock],
                     chunk_flags: Optional[torch.Tensor] = None,
                     chunk_l2sq: Optional[torch.Tensor] = None,
                     total_l2sq: Optional[torch.Tensor] = None,
                     scratch: Optional[torch.Tensor] = None,
                     first: int = 0,
                     count: Optional[int] = None):
    count = table.n_chunks - first if count is None else count
    if chunk_flags is not None:
        _check_tensor(chunk_flags, 'chunk_flags', torch.int32)
        if chunk_flags.numel() < table.n_chunks:
            raise ValueError('chunk_flags is shorter than the table')
    for name, t in (('chunk_l2sq', chunk_l2sq), ('total_l2sq', total_l2sq), ('scratch', scratch)):
        if t is not None:
            _check_tensor(t, name, torch.float32)
    if chunk_l2sq is not None and chunk_l2sq.numel() < table.n_chunks:
        raise ValueError('chunk_l2sq is shorter than the table')
    with _DeviceGuard(table.descs_dev):
        _lib.check(
            _lib.get().elx_grad_check_multi(_ptr(table.descs_dev), first, count, table.tiles(first, count), table.code,
                                            _ptr(chunk_flags), ctl.ptr if ctl else None, _ptr(chunk_l2sq),
                                            _ptr(total_l2sq), _ptr(scratch),
                                            scratch.numel() if scratch is not None else 0, _stream(table.descs_dev)),
            'elx_grad_check_multi')


def adam_multi(table: ChunkTable, ctl: ControlBlock, first: int = 0, count: Optional[int] = None):
    count = table.n_chunks - first if count is None else count
    if table.descs_dev is None:
        raise RuntimeError('finalize() the table first')
    if table.n_groups and table.hyper_dev is None:
        raise RuntimeError('set_hyper() before the first step')
    # shards in pinned host memory are updated in place over PCIe by the load/store variant of the kernel
    entry, name = ((_lib.get().elx_adam_multi_hostmem, 'elx_adam_multi_hostmem') if table.host_resident else
                   (_lib.get().elx_adam_multi, 'elx_adam_multi'))
    with _DeviceGuard(table.descs_dev):
        _lib.check(
            entry(_ptr(table.descs_dev), first, count, table.tiles(first, count), table.code, _ptr(table.segs_dev),
                  _ptr(table.hyper_dev), table.n_groups, ctl.ptr, _stream(table.descs_dev)), name)


def adam_multi_shadow(table: ChunkTable, shadow: ChunkTable, ctl: ControlBlock, first: int = 0,
                      count: Optional[int] = None):
    """The fused update out of place (``elx_adam_multi_shadow``): reads the arrays of ``table``, writes the new
    master and moments into those of ``shadow`` (same shards, registered in the same order) and the refreshed
    working copy over the gradients as usual."""
    count = table.n_chunks - first if count is None else count
    if table.descs_dev is None or shadow.descs_dev is None:
        raise RuntimeError('finalize() both tables first')
    if shadow.n_chunks != table.n_chunks or shadow.tile_begin != table.tile_begin:
        raise ValueError('the shadow table does not describe the same shards')
    if table.host_resident or shadow.host_resident:
        raise RuntimeError('the out-of-place update runs on device-resident shards only')
    with _DeviceGuard(table.descs_dev):
        _lib.check(
            _lib.get().elx_adam_multi_shadow(_ptr(table.descs_dev), _ptr(shadow.descs_dev), first, count,
                                             table.tiles(first, count), table.code, _ptr(table.segs_dev),
                                             _ptr(table.hyper_dev), table.n_groups, ctl.ptr,
                                             _stream(table.descs_dev)), 'elx_adam_multi_shadow')


def _no_peers():
    table = _abi.ElxPeerTable()
    table.rank, table.world = 0, 0
    return table


def step_begin_optimistic(ctl: ControlBlock, cfg: ElxScalerCfg, chunk_flags: Optional[torch.Tensor] = None):
    """Decision of a single-pass step, taken before the gradients have been looked at (``elx_step_begin_optimistic``)."""
    with _DeviceGuard(ctl.tensor):
        _lib.check(_lib.get().elx_step_begin_optimistic(ctl.ptr, cfg, _ptr(chunk_flags),
                                                        chunk_flags.numel() if chunk_flags is not None else 0,
                                                        _stream(ctl.tensor)), 'elx_step_begin_optimistic')


def step_commit(ctl: ControlBlock, cfg: ElxScalerCfg, chunk_flags: Optional[torch.Tensor] = None):
    """Adopt the single-pass update (the two state sets change roles) or, after an overflow, take the optimistic
    decision back and decide "skip" (``elx_step_commit``)."""
    with _DeviceGuard(ctl.tensor):
        _lib.check(_lib.get().elx_step_commit(ctl.ptr, cfg, _ptr(chunk_flags),
                                              chunk_flags.numel() if chunk_flags is not None else 0,
                                              _stream(ctl.tensor)), 'elx_step_commit')


def _check_two_sets(table: 'ChunkTable', other: 'ChunkTable'):
    if table.descs_dev is None or other.descs_dev is None:
        raise RuntimeError('finalize() both tables first')
    if other.n_chunks != table.n_chunks or other.tile_begin != table.tile_begin:
        raise ValueError('the two tables do not describe the same shards')
    if table.host_resident or other.host_resident:
        raise RuntimeError('the single-pass step runs on device-resident shards only')


def adam_multi_single_pass(table: 'ChunkTable', other: 'ChunkTable', ctl: ControlBlock,
                           chunk_flags: Optional[torch.Tensor] = None, first: int = 0, count: Optional[int] = None,
                           grads_table=None, gather_table=None, block_off: Optional[torch.Tensor] = None,
                           grads_mc: int = 0, gather_mc: int = 0):
    """Unscale + inf/nan detection + Adam/AdamW + working copy in one pass, out of place between the two state
    sets ``table`` (set 0) and ``other`` (set 1) (``elx_adam_multi_single_pass``).  With the peer tables and the
    multicast addresses of the ranks' gradient and gather slabs the same launch also reduce-scatters the gradients
    and all-gathers the working copies through the NVLink switch."""
    count = table.n_chunks - first if count is None else count
    _check_two_sets(table, other)
    sharded = gather_table is not None
    if sharded:
        _check_tensor(block_off, 'block_off', torch.int64)
        if block_off.numel() < table.n_chunks:
            raise ValueError('block_off is shorter than the table')
    with _DeviceGuard(table.descs_dev):
        _lib.check(
            _lib.get().elx_adam_multi_single_pass(
                _ptr(table.descs_dev), _ptr(other.descs_dev), first, count, table.tiles(first, count), table.code,
                _ptr(table.segs_dev), _ptr(table.hyper_dev), table.n_groups, ctl.ptr, _ptr(chunk_flags),
                grads_table if sharded else _no_peers(), gather_table if sharded else _no_peers(),
                _ptr(block_off) if sharded else None, ctypes.c_void_p(grads_mc) if sharded else None,
                ctypes.c_void_p(gather_mc) if sharded else None, _stream(table.descs_dev)),
            'elx_adam_multi_single_pass')


def adam_multi_repair(table: 'ChunkTable', other: 'ChunkTable', ctl: ControlBlock, first: int = 0,
                      count: Optional[int] = None, gather_table=None, block_off: Optional[torch.Tensor] = None):
    """Does nothing unless ``elx_step_commit`` asked for it; then rebuilds the working copies (and re-sends them to
    the gather blocks) from the current state set (``elx_adam_multi_repair``)."""
    count = table.n_chunks - first if count is None else count
    _check_two_sets(table, other)
    sharded = gather_table is not None
    with _DeviceGuard(table.descs_dev):
        _lib.check(
            _lib.get().elx_adam_multi_repair(_ptr(table.descs_dev), _ptr(other.descs_dev), first, count,
                                             table.tiles(first, count), table.code, ctl.ptr,
                                             gather_table if sharded else _no_peers(),
                                             _ptr(block_off) if sharded else None, None, _stream(table.descs_dev)),
            'elx_adam_multi_repair')


def pull_reduce_multi(table: ChunkTable, grads_table, block_off: torch.Tensor, ctl: Optional[ControlBlock],
                      chunk_flags: Optional[torch.Tensor] = None, first: int = 0, count: Optional[int] = None,
                      stage_off: Optional[torch.Tensor] = None):
    """NVLink pull reduce-scatter fused with the probe (``elx_pull_reduce_multi``).  ``grads_table`` is the
    ``ElxPeerTable`` of the ranks' gradient slabs, ``block_off`` (int64, device) the element offset of each
    chunk's block inside a slab."""
    count = table.n_chunks - first if count is None else count
    if table.host_resident:
        raise RuntimeError('the NVLink reduce-scatter writes device-resident shards only')
    _check_tensor(block_off, 'block_off', torch.int64)
    if block_off.numel() < table.n_chunks:
        raise ValueError('block_off is shorter than the table')
    if chunk_flags is not None:
        _check_tensor(chunk_flags, 'chunk_flags', torch.int32)
    with _DeviceGuard(table.descs_dev):
        _lib.check(
            _lib.get().elx_pull_reduce_multi(_ptr(table.descs_dev), first, count, table.tiles(first, count), table.code,
                                             grads_table, _ptr(block_off), _ptr(stage_off), _ptr(chunk_flags),
                                             ctl.ptr if ctl else None, _stream(table.descs_dev)),
            'elx_pull_reduce_multi')


def adam_multi_push(table: ChunkTable, ctl: ControlBlock, gather_table, block_off: torch.Tensor, first: int = 0,
                    count: Optional[int] = None):
    """Fused update whose refreshed low-precision tiles are also stored into every rank's gather slab
    (``elx_adam_multi_push``)."""
    count = table.n_chunks - first if count is None else count
    if table.host_resident:
        raise RuntimeError('the update fused with the push all-gather runs on device-resident shards only')
    _check_tensor(block_off, 'block_off', torch.int64)
    if block_off.numel() < table.n_chunks:
        raise ValueError('block_off is shorter than the table')
    with _DeviceGuard(table.descs_dev):
        _lib.check(
            _lib.get().elx_adam_multi_push(_ptr(table.descs_dev), first, count, table.tiles(first, count), table.code,
                                           _ptr(table.segs_dev), _ptr(table.hyper_dev), table.n_groups, ctl.ptr,
                                           gather_table, _ptr(block_off), _stream(table.descs_dev)),
            'elx_adam_multi_push')


def adam_multi_pull_push(table: ChunkTable, ctl: ControlBlock, grads_table, gather_table, block_off: torch.Tensor,
                         first: int = 0, count: Optional[int] = None):
    """Reduce-scatter, in-place update and all-gather in one launch over peer-mapped slabs
    (``elx_adam_multi_pull_push``); the decision must already exist."""
    count = table.n_chunks - first if count is None else count
    if table.host_resident:
        raise RuntimeError('the update fused with both collectives runs on device-resident shards only')
    _check_tensor(block_off, 'block_off', torch.int64)
    if block_off.numel() < table.n_chunks:
        raise ValueError('block_off is shorter than the table')
    with _DeviceGuard(table.descs_dev):
        _lib.check(
            _lib.get().elx_adam_multi_pull_push(_ptr(table.descs_dev), first, count, table.tiles(first, count), table.code,
                                                _ptr(table.segs_dev), _ptr(table.hyper_dev), table.n_groups, ctl.ptr,
                                                grads_table, gather_table, _ptr(block_off), _stream(table.descs_dev)),
            'elx_adam_multi_pull_push')


def multimem_reduce(dst: torch.Tensor, src_mc: int):
    """``dst[i]`` = the sum over all ranks of element i behind the multicast address ``src_mc``, as the NVLink
    switch forms it (``elx_multimem_reduce``)."""
    _check_tensor(dst, 'dst')
    with _DeviceGuard(dst):
        _lib.check(_lib.get().elx_multimem_reduce(ctypes.c_void_p(src_mc), _ptr(dst), dtype_code(dst.dtype), dst.numel(),
                                                  _stream(dst)), 'elx_multimem_reduce')


def copy_async(dst_ptr: int, src_ptr: int, nbytes: int, stream: torch.cuda.Stream):
    """One copy-engine transfer between raw device addresses (local or peer-mapped) on ``stream``."""
    _lib.check(_lib.get().elx_copy_async(ctypes.c_void_p(dst_ptr), ctypes.c_void_p(src_ptr), nbytes,
                                         ctypes.c_void_p(stream.cuda_stream)), 'elx_copy_async')
