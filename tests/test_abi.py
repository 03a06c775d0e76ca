"""The C-ABI library loads without a GPU, exports exactly the symbols the header declares, and rejects
bad arguments with status codes before touching a device."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, 'include', 'elixir_b200.h')


@pytest.fixture(scope='module')
def lib():
    from elixir_b200 import _lib, build
    build.build()
    return _lib.get()


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(elx_[a-z0-9_]+)\s*\(', text)))


def test_header_and_python_prototypes_agree():
    from elixir_b200 import _abi
    assert _declared_functions() == sorted(_abi.PROTOTYPES)


def test_library_exports_every_declared_symbol(lib):
    from elixir_b200 import _lib
    out = subprocess.run(['nm', '-D', '--defined-only', _lib.lib_path()], capture_output=True, text=True, check=True)
    exported = {line.split()[-1] for line in out.stdout.splitlines() if ' T ' in line}
    declared = set(_declared_functions())
    assert declared <= exported
    assert {s for s in exported if s.startswith('elx_')} == declared


def test_struct_layouts_match_the_header():
    """Compile a tiny C program against the header and compare sizeof/offsetof with the ctypes mirror."""
    from elixir_b200 import _abi
    fields = {
        'ElxCtl': ['scale', 'found_inf', 'growth_step', 'hysteresis_step', 'step', 'skip', 'div_scale', 'inv_div',
                   'skipped_steps', 'status', 'late_inf', 'forced_skips', 'clip_coef', 'grad_norm', 'cur_set', 'spec_state',
                   'repair', 'saved_scale', 'saved_growth_step', 'saved_hysteresis_step', 'saved_step', 'reserved'],
        'ElxScalerCfg': ['dynamic', 'growth_factor', 'backoff_factor', 'min_scale', 'max_scale', 'growth_interval',
                         'hysteresis', 'max_norm'],
        'ElxHyper': ['lr', 'beta1', 'beta2', 'eps', 'weight_decay', 'adamw_mode', 'bias_correction', 'reserved'],
        'ElxSeg': ['begin', 'end', 'group', 'reserved'],
        'ElxChunkDesc': ['master', 'exp_avg', 'exp_avg_sq', 'grad_param', 'n_shard', 'n_valid', 'tile_begin',
                         'seg_first', 'seg_count', 'dtype', 'reserved', 'grad_src'],
    }
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "elixir_b200.h"', 'int main(void){']
    for s, fs in fields.items():
        lines.append(f'printf("{s} %zu\\n", sizeof({s}));')
        for f in fs:
            lines.append(f'printf("{s}.{f} %zu\\n", offsetof({s}, {f}));')
    lines.append('printf("TILE %d\\nVERSION %d\\n", ELX_TILE, ELX_ABI_VERSION); return 0;}')
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        src, exe = os.path.join(tmp, 'layout.c'), os.path.join(tmp, 'layout')
        open(src, 'w').write('\n'.join(lines))
        subprocess.run(['gcc', '-I', os.path.join(ROOT, 'include'), src, '-o', exe], check=True)
        out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout
    got = dict(line.split() for line in out.splitlines())
    for s, fs in fields.items():
        cls = getattr(_abi, s)
        assert int(got[s]) == ctypes.sizeof(cls)
        for f in fs:
            assert int(got[f'{s}.{f}']) == getattr(cls, f).offset, (s, f)
    assert int(got['TILE']) == _abi.TILE and int(got['VERSION']) == _abi.ABI_VERSION


def test_version_strerror_and_argument_checks_need_no_gpu(lib):
    from elixir_b200 import _abi
    assert lib.elx_version() == _abi.ABI_VERSION
    assert lib.elx_strerror(0) == b'ok'
    assert b'NULL' in lib.elx_strerror(_abi.ERR_NULL)
    assert lib.elx_probe_scratch_elems(10) == 10
    # validation happens before any CUDA call
    assert lib.elx_ctl_init(None, 1.0, None) == _abi.ERR_NULL
    assert lib.elx_grad_check(None, 0, 1, None, None, None, None, 0, None) == _abi.ERR_NULL
    assert lib.elx_adam_multi(None, 0, 1, 1, 0, None, None, 1, None, None) == _abi.ERR_NULL
    assert lib.elx_adam_multi_hostmem(None, 0, 1, 1, 0, None, None, 1, None, None) == _abi.ERR_NULL
    assert lib.elx_cast_copyback(ctypes.c_void_p(64), ctypes.c_void_p(128), 9, 1, None) == _abi.ERR_DTYPE
    assert lib.elx_set_tuning(b'adam_threads', 512) == _abi.OK
    assert lib.elx_set_tuning(b'adam_threads', -1) == _abi.OK


def test_product_refuses_cpu_tensors():
    import torch
    from elixir_b200 import kernels
    with pytest.raises(RuntimeError, match='no CPU path'):
        kernels.cast_copyback(torch.zeros(8), torch.zeros(8, dtype=torch.float16))


def test_product_does_not_import_the_oracle():
    """Nothing under elixir_b200/ may reference the oracle package."""
    pkg = os.path.join(ROOT, 'elixir_b200')
    for dirpath, _, files in os.walk(pkg):
        for name in files:
            if name.endswith(('.py', '.cu', '.h')):
                text = open(os.path.join(dirpath, name)).read()
                assert 'oracle' not in text.replace('tests/conftest.py', ''), os.path.join(dirpath, name)
