"""The allocation-free probe entry point, exercised last.

Some users of the C ABI cannot give the library scratch memory: a plain-C or ctypes host that owns no
device allocator, or code that runs where allocating is not allowed.  ``elx_grad_check_static`` serves
them from an array built into the library.  This file checks, through the raw C ABI, that it returns
exactly what ``elx_grad_check`` returns with caller-provided scratch — on two calls in a row, because
the built-in array is shared between calls and keeps the previous call's contents.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _both(lib, g, n_valid, code):
    """(flag, l2 bits) from the entry point with caller scratch and from the allocation-free one."""
    dev = g.device
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    out = []
    n_tiles = (n_valid + 4095) // 4096
    scratch = torch.empty(max(1, n_tiles), dtype=torch.float32, device=dev)
    for static in (False, True):
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        l2 = torch.full((1,), -1.0, dtype=torch.float32, device=dev)
        if static:
            rc = lib.elx_grad_check_static(_p(g), code, n_valid, _p(flag), None, _p(l2), stream)
        else:
            rc = lib.elx_grad_check(_p(g), code, n_valid, _p(flag), None, _p(l2), _p(scratch), scratch.numel(), stream)
        assert rc == 0, lib.elx_strerror(rc)
        torch.cuda.synchronize()
        out.append((int(flag.item()), l2.view(torch.int32).item(), l2.item()))
    return out


def test_static_scratch_entry_matches_the_scratch_taking_one_twice_in_a_row(cuda, oracle):
    from elixir_b200 import _abi, _lib
    lib = _lib.get()
    assert lib.elx_grad_check_static_max_elems() == 16384 * 4096
    gen = torch.Generator().manual_seed(42)
    # first call: a large shard, clean.  second call: a smaller one with an inf — it must not see
    # anything the first call left in the shared array.
    big = (torch.randn(5 * 1024 * 1024 + 77, generator=gen) * 4).half()
    small = (torch.randn(3 * 4096 + 5, generator=gen) * 2).to(torch.bfloat16)
    small[4097] = float('inf')
    small[7] = float('nan')
    for g, n_valid, code in ((big, big.numel() - 3, _abi.F16), (small, small.numel(), _abi.BF16),
                             (small, 7, _abi.BF16)):
        plain, static = _both(lib, g.to(cuda), n_valid, code)
        assert plain[0] == static[0] == int(oracle.probe(g, n_valid))
        assert plain[1] == static[1]    # same bits: same kernels, same reduction order
        want = oracle.l2sq(g, n_valid)
        if want == want and want != float('inf'):
            assert abs(static[2] - want) <= 1e-5 * max(want, 1e-30)


def test_static_scratch_entry_rejects_oversized_requests(cuda):
    from elixir_b200 import _abi, _lib
    lib = _lib.get()
    g = torch.zeros(4096, dtype=torch.float16, device=cuda)
    flag = torch.zeros(1, dtype=torch.int32, device=cuda)
    l2 = torch.zeros(1, dtype=torch.float32, device=cuda)
    too_many = lib.elx_grad_check_static_max_elems() + 1
    assert lib.elx_grad_check_static(_p(g), _abi.F16, too_many, _p(flag), None, _p(l2), None) == _abi.ERR_CAPACITY
    assert b'capacity' in lib.elx_strerror(_abi.ERR_CAPACITY)


def test_static_scratch_entry_without_a_norm_has_no_size_limit(cuda):
    """The limit belongs to the built-in array, and only the sum of squares uses it: a plain overflow probe of a
    shard larger than the limit goes through."""
    from elixir_b200 import _abi, _lib
    lib = _lib.get()
    n = lib.elx_grad_check_static_max_elems() + 4096 + 3
    g = torch.zeros(n, dtype=torch.float16, device=cuda)
    g[n - 2] = float('inf')
    flag = torch.zeros(1, dtype=torch.int32, device=cuda)
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)
    assert lib.elx_grad_check_static(_p(g), _abi.F16, n - 2, _p(flag), None, None, stream) == _abi.OK
    assert flag.item() == 0
    assert lib.elx_grad_check_static(_p(g), _abi.F16, n, _p(flag), None, None, stream) == _abi.OK
    assert flag.item() == 1
