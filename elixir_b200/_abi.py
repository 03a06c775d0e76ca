"""ctypes view of ``include/elixir_b200.h``: the structs and the prototype of every entry point.

The table in :data:`PROTOTYPES` is the single Python-side statement of the C ABI; the loader in
``_lib.py`` applies it to ``libelixir_b200.so`` and the tests check that the library exports exactly
these symbols.
"""
import ctypes as C

ABI_VERSION = 2
TILE = 4096

F16, BF16, F32 = 0, 1, 2

OK = 0
ERR_NULL, ERR_ALIGN, ERR_SIZE, ERR_DTYPE, ERR_LAUNCH, ERR_ARG, ERR_NODEVICE, ERR_CAPACITY = range(-1, -9, -1)

STAT_LATE_INF = 1
STAT_BAD_DESC = 2
STAT_TIMEOUT = 4

MAX_GROUPS = 64


class ElxCtl(C.Structure):
    """Device-resident control block (128 bytes)."""
    _fields_ = [
        ('scale', C.c_float),
        ('found_inf', C.c_uint32),
        ('growth_step', C.c_int32),
        ('hysteresis_step', C.c_int32),
        ('step', C.c_int32),
        ('skip', C.c_uint32),
        ('div_scale', C.c_float),
        ('inv_div', C.c_float),
        ('skipped_steps', C.c_uint32),
        ('status', C.c_uint32),
        ('late_inf', C.c_uint32),
        ('forced_skips', C.c_uint32),
        ('clip_coef', C.c_float),
        ('grad_norm', C.c_float),
        ('cur_set', C.c_uint32),
        ('spec_state', C.c_uint32),
        ('repair', C.c_uint32),
        ('saved_scale', C.c_float),
        ('saved_growth_step', C.c_int32),
        ('saved_hysteresis_step', C.c_int32),
        ('saved_step', C.c_int32),
        ('reserved', C.c_uint32 * 11),
    ]


class ElxScalerCfg(C.Structure):
    _fields_ = [
        ('dynamic', C.c_int32),
        ('growth_factor', C.c_float),
        ('backoff_factor', C.c_float),
        ('min_scale', C.c_float),
        ('max_scale', C.c_float),
        ('growth_interval', C.c_int32),
        ('hysteresis', C.c_int32),
        ('max_norm', C.c_float),
    ]


class ElxHyper(C.Structure):
    _fields_ = [
        ('lr', C.c_float),
        ('beta1', C.c_float),
        ('beta2', C.c_float),
        ('eps', C.c_float),
        ('weight_decay', C.c_float),
        ('adamw_mode', C.c_int32),
        ('bias_correction', C.c_int32),
        ('reserved', C.c_int32),
    ]


class ElxSeg(C.Structure):
    _fields_ = [
        ('begin', C.c_int64),
        ('end', C.c_int64),
        ('group', C.c_int32),
        ('reserved', C.c_int32),
    ]


class ElxChunkDesc(C.Structure):
    _fields_ = [
        ('master', C.c_void_p),
        ('exp_avg', C.c_void_p),
        ('exp_avg_sq', C.c_void_p),
        ('grad_param', C.c_void_p),
        ('n_shard', C.c_int64),
        ('n_valid', C.c_int64),
        ('tile_begin', C.c_int64),
        ('seg_first', C.c_int32),
        ('seg_count', C.c_int32),
        ('dtype', C.c_int32),
        ('reserved', C.c_int32),
        ('grad_src', C.c_void_p),
    ]


MAX_PEERS = 16


class ElxPeerTable(C.Structure):
    _fields_ = [
        ('base', C.c_void_p * MAX_PEERS),
        ('rank', C.c_int32),
        ('world', C.c_int32),
    ]


assert C.sizeof(ElxPeerTable) == 8 * MAX_PEERS + 8
assert C.sizeof(ElxCtl) == 128
assert C.sizeof(ElxScalerCfg) == 32
assert C.sizeof(ElxHyper) == 32
assert C.sizeof(ElxSeg) == 24
assert C.sizeof(ElxChunkDesc) == 80

_p = C.c_void_p
_i = C.c_int
_i64 = C.c_int64
_f = C.c_float

# name -> (restype, argtypes); order and types as declared in include/elixir_b200.h
PROTOTYPES = {
    'elx_version': (_i, []),
    'elx_strerror': (C.c_char_p, [_i]),
    'elx_last_cuda_error': (C.c_char_p, []),
    'elx_set_tuning': (_i, [C.c_char_p, _i]),
    'elx_probe_scratch_elems': (_i64, [_i64]),
    'elx_ctl_init': (_i, [_p, _f, _p]),
    'elx_step_begin': (_i, [_p, ElxScalerCfg, _p, _p, _i, _p]),
    'elx_grad_check': (_i, [_p, _i, _i64, _p, _p, _p, _p, _i64, _p]),
    'elx_grad_check_static': (_i, [_p, _i, _i64, _p, _p, _p, _p]),
    'elx_grad_check_static_max_elems': (_i64, []),
    'elx_reduce_epilogue': (_i, [_p, _p, _i, _i64, _i64, _p, _p, _p, _p, _i64, _p]),
    'elx_widen': (_i, [_p, _i, _p, _i64, _p]),
    'elx_narrow_epilogue': (_i, [_p, _p, _i, _i64, _i64, _p, _p, _p]),
    'elx_grad_check_multi': (_i, [_p, _i, _i, _i64, _i, _p, _p, _p, _p, _p, _i64, _p]),
    'elx_adam_multi': (_i, [_p, _i, _i, _i64, _i, _p, _p, _i, _p, _p]),
    'elx_adam_multi_hostmem': (_i, [_p, _i, _i, _i64, _i, _p, _p, _i, _p, _p]),
    'elx_adam_multi_shadow': (_i, [_p, _p, _i, _i, _i64, _i, _p, _p, _i, _p, _p]),
    'elx_step_begin_optimistic': (_i, [_p, ElxScalerCfg, _p, _i, _p]),
    'elx_step_commit': (_i, [_p, ElxScalerCfg, _p, _i, _p]),
    'elx_adam_multi_single_pass': (_i, [_p, _p, _i, _i, _i64, _i, _p, _p, _i, _p, _p, ElxPeerTable, ElxPeerTable, _p, _p,
                                        _p, _p]),
    'elx_adam_multi_repair': (_i, [_p, _p, _i, _i, _i64, _i, _p, ElxPeerTable, _p, _p, _p]),
    'elx_enable_peer_access': (_i, [_i]),
    'elx_peer_alloc': (_i, [_i64, C.POINTER(C.c_void_p), _p]),
    'elx_peer_free': (_i, [_p]),
    'elx_ipc_open': (_i, [_p, C.POINTER(C.c_void_p)]),
    'elx_ipc_close': (_i, [_p]),
    'elx_peek_u32': (_i, [_p, C.POINTER(C.c_uint32)]),
    'elx_peer_barrier': (_i, [ElxPeerTable, C.c_uint32, _p, _i, _i, _p]),
    'elx_pull_reduce_multi': (_i, [_p, _i, _i, _i64, _i, ElxPeerTable, _p, _p, _p, _p, _p]),
    'elx_multimem_reduce': (_i, [_p, _p, _i, _i64, _p]),
    'elx_copy_async': (_i, [_p, _p, _i64, _p]),
    'elx_adam_multi_push': (_i, [_p, _i, _i, _i64, _i, _p, _p, _i, _p, ElxPeerTable, _p, _p]),
    'elx_adam_multi_pull_push': (_i, [_p, _i, _i, _i64, _i, _p, _p, _i, _p, ElxPeerTable, ElxPeerTable, _p, _p]),
    'elx_adam_chunk': (_i, [_p, _p, _p, _p, _i, _i64, _i64, ElxHyper, _p, _p]),
    'elx_cast_copyback': (_i, [_p, _p, _i, _i64, _p]),
}


def apply_prototypes(cdll):
    """Set restype/argtypes of every entry point on a loaded library; raise if one is missing."""
    for name, (restype, argtypes) in PROTOTYPES.items():
        try:
            fn = getattr(cdll, name)
        except AttributeError as exc:
            raise RuntimeError(f'{getattr(cdll, "_name", cdll)} does not export {name}') from exc
        fn.restype = restype
        fn.argtypes = argtypes
    return cdll
