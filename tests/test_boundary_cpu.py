"""Host-side checks that need no GPU: the shared library loads and exports the whole C ABI,
arguments are validated before the device is touched, and the GEMV work plan is sound."""
import ctypes
import os
import re

import numpy as np
import pytest

import locomp_b200 as L
from locomp_b200 import _lib
from locomp_b200.build import LIB_PATH, build, needs_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module", autouse=True)
def _built():
    if needs_build():
        build()
    assert os.path.exists(LIB_PATH)


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "locomp_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lcq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared_functions()
    assert len(names) >= 12
    handle = ctypes.CDLL(LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_status_strings():
    lib = _lib.lib()
    assert lib.lcq_version() >= 100
    assert lib.lcq_status_string(0) == b"ok"
    assert b"workspace" in lib.lcq_status_string(_lib.ERR_WORKSPACE)


def test_c_abi_rejects_bad_problems_without_a_device():
    lib = _lib.lib()
    one = ctypes.c_void_p(256)
    # K not a multiple of the group size
    assert lib.lcq_matmul_int4(one, one, one, one, 1, 8, 40, 32, 0, 0, 0, 0, None, 0, None) == _lib.ERR_BAD_ARG
    assert b"group_size" in lib.lcq_last_error()
    # odd K for int4
    assert lib.lcq_dequant_int4(one, one, one, 4, 7, 7, 0, 0, None) == _lib.ERR_BAD_ARG
    # bad dtype code
    assert lib.lcq_dequant_int8(one, one, one, 4, 8, 8, 9, 0, None) == _lib.ERR_BAD_ARG
    # null pointers
    assert lib.lcq_matmul_int8(None, one, one, one, 1, 8, 64, 32, 0, 0, 0, 0, None, 0, None) == _lib.ERR_BAD_ARG
    # empty problems are fine and touch nothing
    assert lib.lcq_matmul_int4(None, None, None, None, 0, 8, 64, 32, 0, 0, 0, 0, None, 0, None) == 0
    assert lib.lcq_dequant_int4(None, None, None, 0, 64, 32, 0, 0, None) == 0
    assert lib.lcq_matmul_workspace_bytes(4, 1, 8, 40, 32, 1, 1, 1, 0) == (1 << 64) - 1


def test_algo_selection():
    lib = _lib.lib()
    sel = lib.lcq_matmul_select_algo
    assert sel(4, 1, 2048, 2048, 32, _lib.F16, _lib.F16, _lib.F16) == _lib.ALGO_GEMV_TC
    assert sel(4, 16, 2048, 8192, 32, _lib.F16, _lib.F16, _lib.F16) == _lib.ALGO_GEMV_TC
    assert sel(4, 4, 1536, 576, 32, _lib.F16, _lib.F16, _lib.F16) == _lib.ALGO_GEMV_TC   # K % 256 != 0: partial last k tile
    assert sel(4, 1, 49152, 576, 32, _lib.F16, _lib.F16, _lib.F16) == _lib.ALGO_GEMV_TC  # the lm_head
    assert sel(4, 1, 1536, 576, 32, _lib.F16, _lib.F16, _lib.F16) == _lib.ALGO_SIMT      # one row x a tiny weight: latency-bound
    assert sel(4, 1, 1536, 96, 32, _lib.F16, _lib.F16, _lib.F16) == _lib.ALGO_SIMT       # K % 64 != 0
    assert sel(4, 1, 4096, 4096, 32, _lib.F32, _lib.F32, _lib.F32) == _lib.ALGO_SIMT     # reference dtypes
    assert sel(8, 1, 1536, 576, 576, _lib.F32, _lib.F32, _lib.F32) == _lib.ALGO_SIMT     # the reference's int8 shape: 0.9 MB, latency-bound
    assert sel(8, 1, 49152, 2048, 64, _lib.F32, _lib.F32, _lib.F32) == _lib.ALGO_GEMV_W8
    assert sel(8, 1, 64, 40, 8, _lib.F32, _lib.F32, _lib.F32) == _lib.ALGO_SIMT          # K % 16 != 0
    assert lib.lcq_matmul_workspace_bytes(8, 1, 1536, 576, 576, 0, 0, 0, 0) == 0
    assert lib.lcq_matmul_workspace_bytes(4, 1, 2048, 2048, 32, 1, 1, 1, 0) > 0


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
def test_gemv_plan_covers_every_tile_once(M):
    lib = _lib.lib()
    f = (ctypes.c_int * 8)()
    for N in (1, 100, 128, 192, 1024, 2048, 8192, 16032, 49152, 128256):
        for K in (64, 256, 576, 768, 2048, 8192, 28672):
            for sms in (148, 132, 7, 1):
                rc = lib.lcq_gemv_tc_plan_check(M, N, K, sms, f)
                assert rc == 0, (M, N, K, sms, lib.lcq_last_error())
                assert f[0] <= max(2 * sms, f[2]) and f[6] <= 227 * 1024   # CTAs never wait on each other


def test_small_problems_plan_into_clusters_and_large_ones_do_not():
    lib = _lib.lib()
    plan = lib.lcq_gemv_tc_plan_cluster
    assert plan(1, 2048, 2048, 148) == 8          # 16 row blocks x 8 k tiles: one tile per CTA
    assert plan(4, 8192, 2048, 148) == 4          # 64 row blocks: 4 CTAs each keep all 256 resident
    assert plan(16, 2048, 8192, 148) == 4         # x per CTA is a share of K: no k ranges needed; one CTA per SM: clusters of 4
    assert plan(1, 4096, 4096, 148) == 4          # 32 row blocks x 8 would fill more than 3/4 of the CTA slots
    assert plan(1, 49152, 2048, 148) == 1         # enough tiles per CTA: stream-K
    assert plan(1, 128256, 8192, 148) == 1
    assert plan(1, 192, 64, 148) == 1             # a single k tile cannot be shared
    for M in (1, 3, 8, 16):                       # whatever the plan, a cluster never exceeds 8 CTAs
        for N in (100, 1024, 5000, 16032):
            for K in (64, 576, 2048, 28672):
                c = plan(M, N, K, 148)
                assert c in (1, 2, 4, 8), (M, N, K, c)


def test_python_validation_happens_before_the_gpu():
    x = np.zeros(64, np.float32)
    with pytest.raises(ValueError, match="K=64"):
        L.gpu_matvec_int4(x, np.zeros((4, 31), np.uint8), np.zeros((4, 2), np.float32))
    with pytest.raises(ValueError, match="scales"):
        L.gpu_matvec_int4(x, np.zeros((4, 32), np.uint8), np.zeros((4, 3), np.float32))
    with pytest.raises(TypeError, match="uint8"):
        L.gpu_matvec_int4(x, np.zeros((4, 32), np.int8), np.zeros((4, 2), np.float32))
    with pytest.raises(TypeError, match="int8"):
        L.gpu_matvec_int8(x, np.zeros((4, 64), np.uint8), np.zeros((4, 2), np.float32))
    with pytest.raises(ValueError, match="group_size"):
        L.gpu_matvec_int8(x, np.zeros((4, 64), np.int8), np.zeros((4, 2), np.float32), group_size=48)
    with pytest.raises(TypeError):
        L.gpu_matvec_int4("nope", np.zeros((4, 32), np.uint8), np.zeros((4, 2), np.float32))
    with pytest.raises(TypeError, match="float"):
        L.gpu_matvec_int4(x.astype(np.int32), np.zeros((4, 32), np.uint8), np.zeros((4, 2), np.float32))
    with pytest.raises(ValueError, match="bytes"):
        L.gpu_dequant_int4(np.zeros(100, np.uint8), np.zeros(8, np.float32), 4, 64)
    with pytest.raises(ValueError, match="grid"):
        L.dequant_int4[(5,), (128,)](np.zeros(128, np.uint8), np.zeros(8, np.float32), np.zeros(256, np.float32),
                                     64, 32, 2, 32)
    with pytest.raises(ValueError, match="HALF_K"):
        L.dequant_matvec_int4[(4,), (128,)](x, np.zeros(128, np.uint8), np.zeros(8, np.float32),
                                            np.zeros(4, np.float32), 64, 31, 2, 32)
    with pytest.raises(TypeError, match="missing"):
        L.dequant_matvec_int8[(4,), (128,)](x, np.zeros(256, np.int8))
    with pytest.raises(TypeError):
        L.dequant_int8(np.zeros(4, np.int8))


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        L.gpu_matvec_int4(np.zeros(64, np.float32), np.zeros((4, 32), np.uint8), np.zeros((4, 2), np.float32))


def test_foreign_cuda_tensor_objects_are_validated():
    """Objects shaped like the reference's CUDATensor (_cuda_ptr / dtype / shape) are accepted by the
    argument normaliser and checked like any other operand -- before any launch."""
    from locomp_b200.tensor import resolve

    class FakeCUDATensor:
        def __init__(self, ptr, shape, dtype):
            self._cuda_ptr, self.shape, self.dtype, self.size = ptr, shape, np.dtype(dtype), int(np.prod(shape))

    op = resolve(FakeCUDATensor(0x1000, (4, 32), np.uint8), "w")
    assert op.ptr == 0x1000 and op.kind == "u8" and op.shape == (4, 32) and op.size == 128
    assert resolve(FakeCUDATensor(0x2000, (64,), np.float16), "x", bf16=True).kind == "bf16"
    with pytest.raises(TypeError):
        resolve(FakeCUDATensor(0x1000, (4,), np.float64), "x")
    with pytest.raises(TypeError):
        resolve(object(), "x")
    # shape errors surface before the device is touched, also for foreign tensors
    with pytest.raises(ValueError, match="K=64"):
        L.gpu_matvec_int4(FakeCUDATensor(0x1000, (64,), np.float32), FakeCUDATensor(0x2000, (4, 31), np.uint8),
                          FakeCUDATensor(0x3000, (4, 2), np.float32))


def test_sharding_argument_checks():
    from locomp_b200.shard import shard_rows
    assert shard_rows(49152, 8, 7) == (43008, 49152)
    with pytest.raises(ValueError):
        L.ShardedQuantLinear(np.zeros((4, 32), np.uint8), np.zeros((4, 2), np.float16), gather="smoke-signals")
