"""In-tree build of ``libelixir_b200.so`` (the CUDA kernels and their C ABI) with nvcc for sm_100a.

Run ``python -m elixir_b200.build``.  nvcc cross-compiles, so no GPU is needed to build.
"""
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT_DIR = os.path.dirname(PKG_DIR)
SOURCES = [os.path.join(PKG_DIR, 'csrc', name) for name in ('elx_control.cu', 'elx_adam.cu', 'elx_probe.cu', 'elx_peer.cu')]
HEADERS = [os.path.join(ROOT_DIR, 'include', 'elixir_b200.h'), os.path.join(PKG_DIR, 'csrc', 'elx_common.cuh')]
LIB_PATH = os.path.join(PKG_DIR, 'libelixir_b200.so')

NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17', '-shared', '-Xcompiler', '-fPIC'
]


def _nvcc():
    exe = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(exe):
        raise RuntimeError('nvcc not found: the elixir_b200 CUDA library cannot be built')
    return exe


def needs_build():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(src) > built for src in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """Compile the library if it is missing or older than its sources.  Returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    cmd = [_nvcc()] + NVCC_FLAGS + ['--threads', '4', '-I', os.path.join(ROOT_DIR, 'include'), '-o', LIB_PATH] + SOURCES
    if verbose:
        cmd.insert(1, '-Xptxas')
        cmd.insert(2, '-v')
        print(' '.join(cmd))
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError('nvcc failed:\n' + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
