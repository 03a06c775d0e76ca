"""Peer-mapped buffers for the NVLink paths: one process per GPU, every rank of a single-node group
maps every other rank's buffer into its own address space and the kernels read / write them directly.

Each rank allocates its buffer with ``elx_peer_alloc`` (cudaMalloc + an IPC handle), the handles travel
over the process group, and every rank opens the others' handles with ITS OWN device current
(``elx_ipc_open``) — that is what makes the mapping usable from kernels running on this rank's GPU.  torch
sees the local buffer through the CUDA array interface.  No multicast object is created and no NVLS is involved: the kernels use plain loads,
plain stores and non-multicast bulk stores only.
"""
import ctypes
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from . import _abi, _lib
from ._abi import ElxPeerTable

# IPC handle (bytes) -> base address of the mapping in this process.  A handle names a whole allocation of the
# exporter's caching allocator, which several buffers may share; it must be opened only once.
_OPENED: Dict[bytes, int] = {}


def _open_handle(handle: bytes, device: torch.device) -> int:
    base = _OPENED.get(handle)
    if base is None:
        out = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(handle, len(handle))
        with torch.cuda.device(device):
            _lib.check(_lib.get().elx_ipc_open(buf, ctypes.byref(out)), 'elx_ipc_open')
        base = out.value
        _OPENED[handle] = base
    return base


class _RawDeviceMemory:
    """A cudaMalloc'ed range owned by this object, exposed to torch through the CUDA array interface."""

    def __init__(self, nbytes: int, device: torch.device):
        self.nbytes = nbytes
        self.device = device
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(device):
            _lib.check(_lib.get().elx_peer_alloc(nbytes, ctypes.byref(ptr), handle), 'elx_peer_alloc')
        self.ptr = ptr.value
        self.handle = handle.raw
        self.__cuda_array_interface__ = dict(shape=(nbytes,), typestr='|u1', data=(self.ptr, False), version=2)

    def __del__(self):
        try:
            if getattr(self, 'ptr', None):
                with torch.cuda.device(self.device):
                    _lib.get().elx_peer_free(ctypes.c_void_p(self.ptr))
                self.ptr = None
        except Exception:    # interpreter shutdown
            pass


class PeerBuffer:
    """A buffer allocated identically on every rank plus the device addresses, valid in THIS process, of the
    other ranks' copies: ``local`` is this rank's tensor, ``table`` the ``ElxPeerTable`` of all addresses."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group, zero: bool = False):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > _abi.MAX_PEERS:
            raise ValueError(f'at most {_abi.MAX_PEERS} ranks per NVLink domain')
        device = torch.device(device)
        itemsize = torch.empty(0, dtype=dtype).element_size()
        nbytes = max(256, (numel * itemsize + 255) // 256 * 256)
        self._raw = _RawDeviceMemory(nbytes, device)
        self.local = torch.as_tensor(self._raw, device=device)[:numel * itemsize].view(dtype)
        assert self.local.data_ptr() == self._raw.ptr
        if zero:
            self.local.zero_()
        torch.cuda.synchronize(device)
        mine = (device.index, self._raw.handle, nbytes)
        gathered: List[Optional[tuple]] = [None] * self.world
        dist.all_gather_object(gathered, mine, group=group)
        table = ElxPeerTable()
        for j, (peer_device, peer_handle, peer_bytes) in enumerate(gathered):
            if peer_bytes != nbytes:
                raise RuntimeError('ranks disagree on the size of a peer buffer')
            if j == self.rank:
                table.base[j] = self._raw.ptr
            else:
                table.base[j] = _open_handle(peer_handle, device)
                word = ctypes.c_uint32()
                with torch.cuda.device(device):    # fail here, with a status code, rather than in a kernel
                    _lib.check(_lib.get().elx_peek_u32(ctypes.c_void_p(table.base[j]), ctypes.byref(word)),
                               f'peer buffer of rank {j} is not readable from {device}')
        table.rank, table.world = self.rank, self.world
        self.table = table
        dist.barrier(group=group)    # every rank has mapped every buffer before anyone uses them


class PeerBarrier:
    """Device-side barrier (and overflow agreement) between the ranks of a box: ``elx_peer_barrier``."""

    def __init__(self, device, group, timeout_ms: int = 20000):
        self.flags = PeerBuffer(256, torch.int32, device, group, zero=True)
        self.epoch = 0
        self.timeout_ms = timeout_ms
        self.device = torch.device(device)

    def __call__(self, ctl=None, exchange_overflow: bool = False):
        self.epoch += 1
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            _lib.check(
                _lib.get().elx_peer_barrier(self.flags.table, self.epoch, ctl.ptr if ctl is not None else None,
                                            int(exchange_overflow), self.timeout_ms, stream), 'elx_peer_barrier')


class SymmBuffer:
    """A buffer allocated identically on every rank of one NVLink domain and bound to a multicast object, so that
    the switch can serve one access for all ranks (``multimem`` instructions): ``local`` is this rank's tensor,
    ``table`` the ``ElxPeerTable`` of the ranks' copies as plain peer addresses, ``mc_ptr`` the multicast address
    that stands for all copies at once.  Allocation, handle exchange and the multicast binding are torch's
    symmetric memory (plumbing); the kernels that use the addresses are this library's."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group):
        import torch.distributed._symmetric_memory as symm
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > _abi.MAX_PEERS:
            raise ValueError(f'at most {_abi.MAX_PEERS} ranks per NVLink domain')
        device = torch.device(device)
        self.local = symm.empty(numel, dtype=dtype, device=device)
        self._handle = symm.rendezvous(self.local, group if group is not None else dist.group.WORLD)
        mc = int(getattr(self._handle, 'multicast_ptr', 0) or 0)
        if mc == 0:
            raise RuntimeError('this process group has no multicast address for symmetric memory '
                               '(the GPUs or the driver lack NVLink multicast): use the peer-mapped path instead')
        ptrs = list(self._handle.buffer_ptrs)
        if ptrs[self.rank] != self.local.data_ptr():
            raise RuntimeError('symmetric memory: the local buffer does not start at the exchanged address')
        table = ElxPeerTable()
        for j, ptr in enumerate(ptrs):
            table.base[j] = ptr
        table.rank, table.world = self.rank, self.world
        self.table = table
        self.mc_ptr = mc
        dist.barrier(group=group)
