"""TEST INFRASTRUCTURE — Python face of the CPU oracle ``elx_oracle.c``.

Only the test-suite, the smoke check and the CPU-baseline legs of the benchmark import this module;
no product code does.  Everything operates on CPU torch tensors (or numpy arrays) in place.  The
arithmetic each function follows is cited in ``elx_oracle.c``.

Parity status: state machine and shard geometry pinned against the reference's own Python code
(``tests/golden``); Adam arithmetic and loss scaler restate ColossalAI's published algorithm and are
pinned against ``torch.optim.Adam/AdamW`` — parity unpinned with respect to ColossalAI itself.
"""
import ctypes as C
import os
import subprocess
import sys

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(_HERE))
from elixir_b200 import _abi    # noqa: E402  (struct layouts are shared with the device ABI)
from elixir_b200._abi import ElxChunkDesc, ElxCtl, ElxHyper, ElxScalerCfg, ElxSeg    # noqa: E402,F401

_LIB = None
_CODES = {torch.float16: _abi.F16, torch.bfloat16: _abi.BF16, torch.float32: _abi.F32}


def build(force=False):
    so = os.path.join(_HERE, 'liboracle.so')
    src = os.path.join(_HERE, 'elx_oracle.c')
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(['make', '-C', _HERE, '-B'], check=True, capture_output=True)
    return so


def build_host_shim(force=False):
    """oracle/libelx_hostshim.so: the elx_* ABI on host memory (CPU-only tests of the host logic)."""
    so = os.path.join(_HERE, 'libelx_hostshim.so')
    srcs = [os.path.join(_HERE, 'elx_host_shim.c'), os.path.join(_HERE, 'elx_oracle.c')]
    if force or not os.path.exists(so) or os.path.getmtime(so) < max(os.path.getmtime(s) for s in srcs):
        subprocess.run(['make', '-C', _HERE, '-B', 'libelx_hostshim.so'], check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        L = C.CDLL(build())
        p, i, i64, f = C.c_void_p, C.c_int, C.c_int64, C.c_float
        L.orc_probe.restype, L.orc_probe.argtypes = i, [p, i, i64]
        L.orc_l2sq.restype, L.orc_l2sq.argtypes = C.c_double, [p, i, i64]
        L.orc_cast.restype, L.orc_cast.argtypes = None, [p, p, i, i64]
        L.orc_reduce_avg.restype, L.orc_reduce_avg.argtypes = None, [p, i, i, i64, p]
        L.orc_reduce_avg_f32acc.restype, L.orc_reduce_avg_f32acc.argtypes = None, [p, i, i, i64, p]
        L.orc_ctl_init.restype, L.orc_ctl_init.argtypes = None, [p, f]
        L.orc_step_begin.restype, L.orc_step_begin.argtypes = None, [p, ElxScalerCfg, p]
        for name in ('orc_adam_f32', 'orc_adam_f64'):
            fn = getattr(L, name)
            fn.restype, fn.argtypes = None, [p, p, p, p, i, i64, i64, ElxHyper, i, f]
        L.orc_step.restype, L.orc_step.argtypes = i, [p, i, p, p, i, p, ElxScalerCfg, i, i]
        L.orc_num_threads.restype, L.orc_num_threads.argtypes = i, []
        L.orc_f32_to_f16.restype, L.orc_f32_to_f16.argtypes = C.c_uint16, [f]
        L.orc_f32_to_bf16.restype, L.orc_f32_to_bf16.argtypes = C.c_uint16, [f]
        L.orc_f16_to_f32.restype, L.orc_f16_to_f32.argtypes = f, [C.c_uint16]
        L.orc_bf16_to_f32.restype, L.orc_bf16_to_f32.argtypes = f, [C.c_uint16]
        _LIB = L
    return _LIB


def _cpu(t, dtype=None):
    assert isinstance(t, torch.Tensor) and t.device.type == 'cpu' and t.is_contiguous()
    if dtype is not None:
        assert t.dtype == dtype, (t.dtype, dtype)
    return C.c_void_p(t.data_ptr())


def num_threads():
    return lib().orc_num_threads()


def probe(g, n_valid=None):
    n_valid = g.numel() if n_valid is None else n_valid
    assert 0 <= n_valid <= g.numel()
    return bool(lib().orc_probe(_cpu(g), _CODES[g.dtype], n_valid))


def l2sq(g, n_valid=None):
    n_valid = g.numel() if n_valid is None else n_valid
    assert 0 <= n_valid <= g.numel()
    return lib().orc_l2sq(_cpu(g), _CODES[g.dtype], n_valid)


def cast(master, dst):
    assert master.numel() == dst.numel()
    lib().orc_cast(_cpu(master, torch.float32), _cpu(dst), _CODES[dst.dtype], master.numel())


def reduce_avg(rank_tensors):
    out = torch.empty_like(rank_tensors[0])
    arr = (C.c_void_p * len(rank_tensors))(*[t.data_ptr() for t in rank_tensors])
    lib().orc_reduce_avg(arr, len(rank_tensors), _CODES[out.dtype], out.numel(), _cpu(out))
    return out


def reduce_avg_f32acc(rank_tensors):
    """The NVLink pull reduce: fp32 accumulation of x_r * (1/W) in rank order, one rounding."""
    out = torch.empty_like(rank_tensors[0])
    arr = (C.c_void_p * len(rank_tensors))(*[t.data_ptr() for t in rank_tensors])
    lib().orc_reduce_avg_f32acc(arr, len(rank_tensors), _CODES[out.dtype], out.numel(), _cpu(out))
    return out


def new_ctl(initial_scale=1.0):
    ctl = ElxCtl()
    lib().orc_ctl_init(C.byref(ctl), initial_scale)
    return ctl


def step_begin(ctl, cfg, norm_sq=None):
    ns = C.c_float(norm_sq) if norm_sq is not None else None
    lib().orc_step_begin(C.byref(ctl), cfg, C.byref(ns) if ns is not None else None)


def adam(master, exp_avg, exp_avg_sq, g, hyper, step, div_scale, begin=0, end=None, f64=False):
    end = master.numel() if end is None else end
    assert 0 <= begin <= end <= min(master.numel(), exp_avg.numel(), exp_avg_sq.numel(), g.numel()), 'range outside the tensors'
    fn = lib().orc_adam_f64 if f64 else lib().orc_adam_f32
    fn(_cpu(master, torch.float32), _cpu(exp_avg, torch.float32), _cpu(exp_avg_sq, torch.float32), _cpu(g),
       _CODES[g.dtype], begin, end, hyper, step, div_scale)


class ChunkSet:
    """Host-memory chunk set with the same tables as the device ABI, stepped by ``orc_step``."""

    def __init__(self, dtype):
        self.dtype = dtype
        self.descs, self.segs, self.keep = [], [], []
        self.tile = 0

    def add_chunk(self, master, exp_avg, exp_avg_sq, grad_param, n_valid, segments=()):
        for t in (master, exp_avg, exp_avg_sq):
            _cpu(t, torch.float32)
        _cpu(grad_param, self.dtype)
        n = master.numel()
        self.descs.append(
            ElxChunkDesc(master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), grad_param.data_ptr(), n, n_valid,
                         self.tile, len(self.segs), len(segments), _CODES[self.dtype], 0))
        self.segs.extend(ElxSeg(b, e, g, 0) for b, e, g in segments)
        self.keep.append((master, exp_avg, exp_avg_sq, grad_param))
        self.tile += (n + _abi.TILE - 1) // _abi.TILE

    def step(self, ctl, cfg, hypers, probe=True, f64=False):
        d = (ElxChunkDesc * len(self.descs))(*self.descs)
        s = (ElxSeg * max(1, len(self.segs)))(*self.segs)
        h = (ElxHyper * max(1, len(hypers)))(*hypers)
        return bool(lib().orc_step(d, len(self.descs), s, h, len(hypers), C.byref(ctl), cfg, int(probe), int(f64)))
