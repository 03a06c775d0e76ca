"""elixir_b200 — the chunk-level mixed-precision optimizer step of hpcaitech/Elixir, rebuilt for
NVIDIA B200 as hand-written sm_100a kernels behind a C ABI (``include/elixir_b200.h``).

``elixir_b200.kernels`` binds the ABI to torch tensors; ``elixir_b200.chunk`` and
``elixir_b200.wrapper`` mirror ``elixir.chunk`` and ``elixir.wrapper`` of the reference for this
path.  Nothing here computes on the CPU: without the native library every operation raises.
"""
from . import _abi, _lib, kernels    # noqa: F401

__version__ = '0.1.0'
