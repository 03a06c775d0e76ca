"""Loader of the native library.  There is no fallback: without ``libelixir_b200.so`` every
operation of this package raises."""
import ctypes
import os

from . import _abi

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'libelixir_b200.so')
_LIB = None
# True only while a test has substituted a host-memory implementation of the ABI (tests/_dist_workers.py does).
_HOST_MEMORY = False


class ElixirB200Error(RuntimeError):
    """A native entry point returned a non-zero status."""

    def __init__(self, status, where, detail=''):
        self.status = status
        super().__init__(f'{where}: status {status} ({detail})')


def lib_path():
    return _LIB_PATH


def get():
    """The loaded library with prototypes applied."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f'{_LIB_PATH} is missing: build it with `python -m elixir_b200.build` '
                               '(needs nvcc); elixir_b200 has no CPU or PyTorch fallback for its kernels')
        cdll = ctypes.CDLL(_LIB_PATH)
        _abi.apply_prototypes(cdll)
        version = cdll.elx_version()
        if version != _abi.ABI_VERSION:
            raise RuntimeError(f'{_LIB_PATH} has ABI version {version}, this package expects {_abi.ABI_VERSION}')
        _LIB = cdll
        _apply_env_tuning(cdll)
    return _LIB


def _apply_env_tuning(cdll):
    """``ELX_TUNING="knob=value,knob=value"`` sets launch-shape knobs (see ``elx_set_tuning``) at load time."""
    spec = os.environ.get('ELX_TUNING', '').strip()
    for item in filter(None, (part.strip() for part in spec.split(','))):
        name, _, value = item.partition('=')
        status = cdll.elx_set_tuning(name.strip().encode(), int(value))
        if status != _abi.OK:
            raise RuntimeError(f'ELX_TUNING: bad entry {item!r}')


def host_memory_backend():
    return _HOST_MEMORY


def check(status, where):
    if status != _abi.OK:
        lib = get()
        detail = lib.elx_strerror(status).decode()
        if status == _abi.ERR_LAUNCH:
            detail += ': ' + lib.elx_last_cuda_error().decode()
        raise ElixirB200Error(status, where, detail)
