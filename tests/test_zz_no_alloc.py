"""The allocation-free decode entry point, called through the C ABI.

Some hosts cannot allocate device memory when they call a linear layer: the serving
framework around them has already taken the whole GPU into its own pool, or the call sits
in a loop where a device-synchronising cudaMalloc is not acceptable.  For them the library
keeps its split-K scratch in a fixed array of its own.  This test checks that the entry
point gives the same output as the regular one (which takes a caller-provided workspace),
on two calls in a row -- the second call finds the scratch as the first one left it.

Collected last on purpose (file name), so a run that stops at the first failure has already
run every other test.  It passes alone in a fresh process and after the other tests.
"""
import ctypes

import numpy as np
import pytest
import torch

from locomp_b200 import _lib
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu


def _call(fn, *args):
    rc = fn(*args)
    assert rc == 0, (rc, _lib.lib().lcq_last_error())


@pytest.mark.parametrize("m,n,k", [(1, 4096, 2048), (4, 2048, 8192), (16, 1000, 1024)])
def test_noalloc_matches_workspace_entry_twice(m, n, k):
    lib = _lib.lib()
    rng = np.random.default_rng(m * 7 + n)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    wd, sd = torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda()
    F16 = _lib.F16
    st = torch.cuda.current_stream().cuda_stream
    ws_bytes = lib.lcq_matmul_workspace_bytes(4, m, n, k, 32, F16, F16, F16, _lib.ALGO_GEMV_TC)
    assert 0 < ws_bytes <= lib.lcq_noalloc_scratch_bytes()
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    for rep in range(2):      # two calls in a row, fresh activations each time
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(rep)).half().cuda()
        ref = torch.empty(m, n, dtype=torch.float16, device="cuda")
        got = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        _call(lib.lcq_matmul_int4, x.data_ptr(), wd.data_ptr(), sd.data_ptr(), ref.data_ptr(), m, n, k, 32,
              F16, F16, F16, _lib.ALGO_GEMV_TC, ws.data_ptr(), ws.numel(), st)
        _call(lib.lcq_matmul_int4_noalloc, x.data_ptr(), wd.data_ptr(), sd.data_ptr(), got.data_ptr(), m, n, k, 32,
              F16, F16, F16, st)
        torch.cuda.synchronize()
        # same kernel, same summation order: within the tolerance of the other parity tests (rtol/atol 1e-2)
        torch.testing.assert_close(got.float(), ref.float(), rtol=1e-2, atol=1e-2)
        oracle = O.matmul_int4(x.float().cpu().numpy(), wp, s, 32)
        assert np.all(np.abs(got.float().cpu().numpy() - oracle) <= 1e-2 + 1e-2 * np.abs(oracle))
    assert lib.lcq_check_device_status(None) == 0


def test_noalloc_rejects_what_does_not_fit():
    lib = _lib.lib()
    one = ctypes.c_void_p(256)
    F16 = _lib.F16
    # a plan larger than the built-in scratch: clear error, nothing launched
    rc = lib.lcq_matmul_int4_noalloc(one, one, one, one, 16, 128256, 8192, 32, F16, F16, F16, None)
    assert rc == _lib.ERR_WORKSPACE and b"scratch" in lib.lcq_last_error()
    # outside the decode kernel's domain
    rc = lib.lcq_matmul_int4_noalloc(one, one, one, one, 64, 1024, 1024, 32, F16, F16, F16, None)
    assert rc == _lib.ERR_UNSUPPORTED
    rc = lib.lcq_matmul_int4_noalloc(one, one, one, one, 1, 1024, 96, 32, F16, F16, F16, None)
    assert rc == _lib.ERR_UNSUPPORTED
