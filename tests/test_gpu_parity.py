"""Parity of the CUDA kernels (called through the C ABI via the Python operators) with the
NumPy oracle and with the golden vectors produced by the reference's own functions.

Bars: integer unpacking and dequantised weights bit-exact; matmul outputs within
rtol 1e-2 / atol 1e-2 for 16-bit activations, 1e-4 (relative to the output scale) for float32.
"""
import numpy as np
import pytest
import torch

import locomp_b200 as L
from locomp_b200 import _lib
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu

RTOL16, ATOL16 = 1e-2, 1e-2


def _bits(a):
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32}[a.dtype.itemsize])


def _assert_f32_close(got, exp):
    exp = np.asarray(exp, np.float64)
    scale = float(np.sqrt(np.mean(exp ** 2))) if exp.size else 1.0
    np.testing.assert_allclose(np.asarray(got, np.float64), exp, rtol=1e-4, atol=1e-4 * scale)


def _device_status_ok():
    assert _lib.lib().lcq_check_device_status(None) == 0, _lib.lib().lcq_last_error()


# --------------------------------------------------------------------------- dequantize
@pytest.mark.parametrize("shape", [(64, 256), (128, 512)])
def test_dequant_int4_golden_bit_exact(golden, shape):
    n, k = shape
    out = L.gpu_dequant_int4(golden[f"dq4_{n}x{k}_packed"], golden[f"dq4_{n}x{k}_scales"], n, k, 32)
    assert out.dtype == np.float32 and out.shape == (n, k)
    assert np.array_equal(_bits(out), _bits(golden[f"dq4_{n}x{k}_expected"]))


def test_dequant_int8_golden_bit_exact(golden):
    out = L.gpu_dequant_int8(golden["dq8_64x256_w8"], golden["dq8_64x256_scales"], 64, 256, 32)
    assert np.array_equal(_bits(out), _bits(golden["dq8_64x256_expected"]))


def test_dequant_full_byte_table(golden):
    out = L.gpu_dequant_int4(golden["tbl_packed"], golden["tbl_scales"], 4, 128, 32)
    assert np.array_equal(_bits(out), _bits(golden["tbl_expected"]))


@pytest.mark.parametrize("n,k,g", [(5, 64, 32), (3, 6, 2), (7, 96, 16), (1, 32, 32), (33, 200, 8), (2, 1000, 500),
                                   (129, 4096, 128), (17, 34, 34)])
@pytest.mark.parametrize("sdt", [np.float32, np.float16])
def test_dequant_ragged_shapes_bit_exact(n, k, g, sdt):
    rng = np.random.default_rng(n * 1000 + k)
    wp, s = O.make_w4(rng, n, k, g, sdt)
    assert np.array_equal(_bits(L.gpu_dequant_int4(wp, s, n, k, g)), _bits(O.dequant_int4(wp, s, g)))
    w8, s8 = O.make_w8(rng, n, k, g, sdt)
    assert np.array_equal(_bits(L.gpu_dequant_int8(w8, s8, n, k, g)), _bits(O.dequant_int8(w8, s8, g)))


@pytest.mark.parametrize("odt", ["f16", "bf16"])
def test_dequant_16bit_outputs_are_rne_of_the_f32_value(odt):
    rng = np.random.default_rng(5)
    wp, s = O.make_w4(rng, 96, 512, 32, np.float16)
    got = L.dequantize(wp, s, 96, 512, 32, bits=4, out_dtype=odt).float().cpu().numpy()
    exp = O.round_to(O.dequant_int4(wp, s, 32), odt).astype(np.float32)
    assert np.array_equal(_bits(got), _bits(exp))
    w8, s8 = O.make_w8(rng, 31, 100, 20, np.float32)
    got = L.dequantize(w8, s8, 31, 100, 20, bits=8, out_dtype=odt).float().cpu().numpy()
    exp = O.round_to(O.dequant_int8(w8, s8, 20), odt).astype(np.float32)
    assert np.array_equal(_bits(got), _bits(exp))


def test_dequant_empty_and_flat_inputs():
    assert L.gpu_dequant_int4(np.zeros((0, 32), np.uint8), np.zeros((0, 2), np.float32), 0, 64).shape == (0, 64)
    rng = np.random.default_rng(9)
    wp, s = O.make_w4(rng, 16, 256, 32, np.float32)
    out = L.gpu_dequant_int4(wp.flatten(), s.flatten(), 16, 256, 32)   # as the reference wrapper passes them
    assert np.array_equal(_bits(out), _bits(O.dequant_int4(wp, s, 32)))


def test_dequant_full_size_properties():
    """Largest prefill weight (4096 x 14336): sampled rows against the oracle, exact linearity in
    the scales (powers of two), and idempotent repeat."""
    n, k = 4096, 14336
    rng = np.random.default_rng(0)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    wd, sd = torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda()
    a = L.dequantize(wd, sd, n, k, 32)
    rows = rng.choice(n, size=64, replace=False)
    assert np.array_equal(_bits(a[rows].cpu().numpy()), _bits(O.dequant_int4(wp[rows], s[rows], 32)))
    b = L.dequantize(wd, sd * 4, n, k, 32)
    assert torch.equal(b, a * 4)
    assert torch.equal(L.dequantize(wd, sd, n, k, 32), a)
    assert float(a.abs().max()) <= 8 * float(s.max())


# --------------------------------------------------------------------------- float32 matvec (reference dtypes)
@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_matvec_f32_golden(golden, tag):
    g = int(golden[f"mv_{tag}_g"])
    x = golden[f"mv_{tag}_x"]
    y4 = L.gpu_matvec_int4(x, golden[f"mv_{tag}_p4"], golden[f"mv_{tag}_s4"], g)
    y8 = L.gpu_matvec_int8(x, golden[f"mv_{tag}_w8"], golden[f"mv_{tag}_s8"], g)
    assert y4.dtype == np.float32 and y4.shape == (golden[f"mv_{tag}_p4"].shape[0],)
    _assert_f32_close(y4, golden[f"mv_{tag}_fast4"])
    _assert_f32_close(y8, golden[f"mv_{tag}_fast8"])


def test_config1_int8_per_channel(golden):
    rng = np.random.default_rng(0)
    w8 = rng.integers(-127, 128, size=(1536, 576), dtype=np.int8)
    s = (np.abs(rng.standard_normal((1536, 1))) * 0.01).astype(np.float32)
    x = rng.standard_normal(576).astype(np.float32)
    y = L.gpu_matvec_int8(x, w8, s, 576)
    _assert_f32_close(y, golden["cfg1_expected"])
    _assert_f32_close(y, O.matmul_int8(x, w8, s, 576))


@pytest.mark.parametrize("n,k,g,m", [(9, 64, 32, 1), (40, 34, 2, 3), (130, 96, 16, 5), (8, 4096, 128, 2),
                                     (257, 576, 32, 1), (64, 256, 256, 7)])
def test_simt_ragged_shapes(n, k, g, m):
    rng = np.random.default_rng(n + k)
    wp, s = O.make_w4(rng, n, k, g, np.float32)
    w8, s8 = O.make_w8(rng, n, k, g, np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    _assert_f32_close(L.gpu_matvec_int4(x, wp, s, g), O.matmul_int4(x, wp, s, g))
    _assert_f32_close(L.gpu_matvec_int8(x, w8, s8, g), O.matmul_int8(x, w8, s8, g))
    if m == 1:
        _assert_f32_close(L.gpu_matvec_int4(x[0], wp, s, g), O.matmul_int4(x[0], wp, s, g))


def test_kernel_object_forms(golden):
    p4, s4, x = golden["mv_a_p4"], golden["mv_a_s4"], golden["mv_a_x"]
    n, k = 256, 256
    X, W, S, Out = L.tensor(x), L.tensor(p4), L.tensor(s4), L.empty(n)
    assert Out.shape == (n,) and Out.dtype == np.float32 and isinstance(Out._cuda_ptr, int)
    L.dequant_matvec_int4[(n,), (128,)](X, W, S, Out, k, k // 2, k // 32, 32)
    _assert_f32_close(Out.numpy(), golden["mv_a_fast4"])
    W8, S8, O8 = L.tensor(golden["mv_a_w8"]), L.tensor(golden["mv_a_s8"]), L.zeros(n)
    L.dequant_matvec_int8[(n,), (128,)](X, W8, S8, O8, K_dim=k, NUM_SCALES=k // 32, GROUP_SIZE=32)
    _assert_f32_close(O8.numpy(), golden["mv_a_fast8"])
    # dequantize with flattened device tensors, as the reference wrapper does
    Wf, Sf, Of = L.tensor(p4.flatten()), L.tensor(s4.flatten()), L.empty(n * k)
    L.dequant_int4[(n,), (128,)](Wf, Sf, Of, k, k // 2, k // 32, 32)
    assert np.array_equal(_bits(Of.numpy().reshape(n, k)), _bits(O.dequant_int4(p4, s4, 32)))
    O8f = L.empty(n * k)
    L.dequant_int8[(n,), (128,)](W8, S8, O8f, k, k // 32, 32)
    assert np.array_equal(_bits(O8f.numpy().reshape(n, k)), _bits(O.dequant_int8(golden["mv_a_w8"], golden["mv_a_s8"], 32)))
    for t in (X, W, S, Out, Wf, Sf, Of):
        t.free()
    with pytest.raises((RuntimeError, ValueError)):
        L.dequant_int4[(n,), (128,)](Wf, Sf, Of, k, k // 2, k // 32, 32)


# --------------------------------------------------------------------------- W4A16 (fp16/bf16 activations)
def _w4a16_case(n, k, m, seed=0, xdt=np.float16):
    rng = np.random.default_rng(seed)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    x = rng.standard_normal((16, k)).astype(np.float16)[:m]
    return wp, s, np.ascontiguousarray(x)


def _oracle_blocked(x, wp, s, rows=4096):
    outs = [O.matmul_int4(x.astype(np.float32), wp[i:i + rows], s[i:i + rows], 32) for i in range(0, wp.shape[0], rows)]
    return np.concatenate(outs, axis=-1)


def _check16(y, ref):
    y = np.asarray(y, np.float64)
    bad = np.abs(y - ref) > ATOL16 + RTOL16 * np.abs(ref)
    assert not bad.any(), f"{bad.sum()} of {bad.size} outside tolerance; max err {np.abs(y - ref).max():.4g}"


@pytest.mark.parametrize("algo", ["gemv_tc", "simt"])
@pytest.mark.parametrize("n,k", [(128, 256), (100, 512), (333, 768), (2048, 2048), (130, 8192)])
@pytest.mark.parametrize("m", [1, 2, 4, 7, 8, 9, 16])
def test_w4a16_small_shapes(algo, n, k, m):
    wp, s, x = _w4a16_case(n, k, m, seed=n + k + m)
    y = L.quantized_matmul(torch.from_numpy(x).cuda(), torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda(),
                           32, algo=algo)
    assert y.dtype == torch.float16 and tuple(y.shape) == (m, n)
    ref = _oracle_blocked(x, wp, s)
    _check16(y.float().cpu().numpy(), ref)
    _device_status_ok()


@pytest.mark.parametrize("k,n", [(2048, 2048), (2048, 8192), (8192, 2048), (2048, 49152)])
@pytest.mark.parametrize("m", [1, 4, 16])
def test_w4a16_config2_full_shapes(k, n, m):
    """The SmolLM2-1.7B projection shapes at full size, AUTO dispatch, float32 output as well."""
    wp, s, x = _w4a16_case(n, k, m, seed=0)
    xd, wd, sd = torch.from_numpy(x).cuda(), torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda()
    assert _lib.lib().lcq_matmul_select_algo(4, m, n, k, 32, _lib.F16, _lib.F16, _lib.F16) == _lib.ALGO_GEMV_TC
    ref = _oracle_blocked(x, wp, s)
    y16 = L.quantized_matmul(xd, wd, sd, 32)
    _check16(y16.float().cpu().numpy(), ref)
    y32 = L.quantized_matmul(xd, wd, sd, 32, out_dtype="f32")
    # float32 output exposes the kernel's own error: products are exact, sums are float32
    np.testing.assert_allclose(y32.cpu().numpy(), ref, rtol=2e-4, atol=2e-4 * float(np.sqrt(np.mean(ref ** 2))))
    # running it again on the reused (self-cleaning) workspace gives the same bits
    assert torch.equal(L.quantized_matmul(xd, wd, sd, 32), y16)
    _device_status_ok()


def test_w4a16_bf16_activations_and_linearity():
    n, k, m = 1000, 4096, 5
    rng = np.random.default_rng(7)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    xb = torch.randn(m, k, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    wd, sd = torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda()
    y = L.quantized_matmul(xb.cuda(), wd, sd, 32, out_dtype="f32")
    ref = _oracle_blocked(xb.float().numpy(), wp, s)
    np.testing.assert_allclose(y.cpu().numpy(), ref, rtol=2e-4, atol=2e-4 * float(np.sqrt(np.mean(ref ** 2))))
    yb = L.quantized_matmul(xb.cuda(), wd, sd, 32)
    assert yb.dtype == torch.bfloat16
    _check16(yb.float().cpu().numpy(), ref)
    # linearity in x for power-of-two factors (float32 output): exact up to the fp16 residual of
    # the zero-point term, which may fall into the subnormal range
    y2 = L.quantized_matmul((xb * 2).cuda(), wd, sd, 32, out_dtype="f32")
    torch.testing.assert_close(y2, y * 2, rtol=1e-5, atol=1e-5)


def test_w4a16_zero_point_and_extremes():
    """All-zero nibbles (value -8), all-15 nibbles (+7) and zero scales."""
    n, k = 256, 512
    x = np.ones((3, k), np.float16)
    s = np.full((n, k // 32), 0.5, np.float16)
    s[5] = 0
    for byte, val in ((0x00, -8.0), (0xFF, 7.0), (0x88, 0.0)):
        wp = np.full((n, k // 2), byte, np.uint8)
        y = L.quantized_matmul(torch.from_numpy(x).cuda(), torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda(),
                               32, out_dtype="f32", algo="gemv_tc").cpu().numpy()
        exp = np.full((3, n), val * 0.5 * k, np.float32)
        exp[:, 5] = 0
        assert np.array_equal(y, exp), (byte, y[0, :8])


def test_host_wrapper_with_fp16_inputs_returns_host_array():
    wp, s, x = _w4a16_case(512, 1024, 1, seed=3)
    y = L.gpu_matvec_int4(x[0], wp, s, 32)
    assert isinstance(y, np.ndarray) and y.dtype == np.float16 and y.shape == (512,)
    _check16(y, _oracle_blocked(x, wp, s)[0])


# --------------------------------------------------------------------------- W4A16 prefill GEMM (tcgen05)
def _gemm_ref(x32, wp, s):
    wd = O.dequant_int4(wp, s, 32).astype(np.float64)
    return x32.astype(np.float64) @ wd.T


@pytest.mark.parametrize("m,n,k", [(32, 128, 256), (64, 256, 512), (256, 128, 1024), (300, 200, 768),
                                   (17, 1000, 256), (512, 384, 2048)])
@pytest.mark.parametrize("xdt", ["f16", "bf16"])
def test_w4a16_gemm_tc_small_shapes(m, n, k, xdt):
    rng = np.random.default_rng(m + n + k)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    xt = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).to(torch.float16 if xdt == "f16" else torch.bfloat16)
    wd, sd = torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda()
    y = L.quantized_matmul(xt.cuda(), wd, sd, 32, algo="gemm_tc", out_dtype="f32")
    _device_status_ok()
    ref = _gemm_ref(xt.float().numpy(), wp, s)
    _check16(y.cpu().numpy(), ref)
    y16 = L.quantized_matmul(xt.cuda(), wd, sd, 32, algo="gemm_tc")
    assert y16.dtype == xt.dtype and tuple(y16.shape) == (m, n)
    _check16(y16.float().cpu().numpy(), ref)
    _device_status_ok()


def test_w4a16_gemm_tc_split_k_sharded_70b_shape():
    """M = 64 on one eighth of the (8192, 28672) projection: few output tiles, so K is split and the
    float partials are summed by the reduce kernel; AUTO dispatch must pick the tcgen05 kernel."""
    m, k, n = 64, 8192, 28672 // 8
    rng = np.random.default_rng(64)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(2)).half()
    assert _lib.lib().lcq_matmul_select_algo(4, m, n, k, 32, _lib.F16, _lib.F16, _lib.F16) == _lib.ALGO_GEMM_TC
    wd, sd = torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda()
    y = L.quantized_matmul(x.cuda(), wd, sd, 32)
    ref = _gemm_ref(x.float().numpy(), wp, s)
    _check16(y.float().cpu().numpy(), ref)
    assert torch.equal(L.quantized_matmul(x.cuda(), wd, sd, 32), y)      # fixed summation order
    _device_status_ok()


def test_w4a16_gemm_tc_matches_decode_kernel():
    """Same inputs through the decode kernel (M <= 16 chunks) and the tcgen05 kernel."""
    rng = np.random.default_rng(11)
    n, k, m = 640, 1024, 48
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(1)).half().cuda()
    wd, sd = torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda()
    a = L.quantized_matmul(x, wd, sd, 32, algo="gemv_tc", out_dtype="f32")
    b = L.quantized_matmul(x, wd, sd, 32, algo="gemm_tc", out_dtype="f32")
    torch.testing.assert_close(a, b, rtol=2e-3, atol=2e-2)


# --------------------------------------------------------------------------- layers
def test_fused_projections_equal_separate_ones():
    rng = np.random.default_rng(21)
    k = 576
    parts = [O.make_w4(rng, n, k, 32, np.float16) for n in (576, 192, 192)]
    dev_parts = [(torch.from_numpy(w).cuda(), torch.from_numpy(s).cuda()) for w, s in parts]
    x = torch.from_numpy(rng.standard_normal((1, k)).astype(np.float16)).cuda()
    fused, splits = L.fuse_rows(dev_parts)
    y = fused(x)
    assert tuple(y.shape) == (1, 960) and splits == [(0, 576), (576, 768), (768, 960)]
    for (w, s), (a, b), (wn, sn) in zip(dev_parts, splits, parts):
        sep = L.QuantLinear(w, s)(x)
        assert torch.equal(y[:, a:b], sep)                       # rows are independent: bit-identical
        _check16(sep.float().cpu().numpy(), O.matmul_int4(x.float().cpu().numpy(), wn, sn, 32))


def test_decode_stack_counts_and_graph():
    st = L.DecodeStack(layers=2, fused=False)
    assert len(st.calls) == 2 * 7 + 1 and st.calls[-1][0].out_features == 49152
    fu = L.DecodeStack(layers=2, fused=True)
    assert len(fu.calls) == 2 * 4 + 1 and fu.weight_bytes == st.weight_bytes
    st.step()
    eager = [c[2].clone() for c in st.calls]
    st.capture()
    for c in st.calls:
        c[2].zero_()
    st.replay()
    torch.cuda.synchronize()
    for a, c in zip(eager, st.calls):
        assert torch.equal(a, c[2])
    _device_status_ok()


def test_w4a16_gemm_tc_unaligned_n_and_caller_workspace():
    """N not a multiple of 8 (scalar epilogue stores) and a caller-provided scratch buffer."""
    m, n, k = 48, 100, 512
    rng = np.random.default_rng(5)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    wd, sd = torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda()
    from locomp_b200.ops import matmul_workspace_bytes
    need = matmul_workspace_bytes(m, n, k, 32, 4, "bf16", "f16", "bf16", "gemm_tc")
    assert need > 0
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    y = L.quantized_matmul(x.cuda(), wd, sd, 32, algo="gemm_tc", workspace_buf=ws)
    _check16(y.float().cpu().numpy(), _gemm_ref(x.float().numpy(), wp, s))
    with pytest.raises(ValueError):
        L.quantized_matmul(x.cuda(), wd, sd, 32, algo="gemm_tc", workspace_buf=ws[: need // 2])
    _device_status_ok()


# --------------------------------------------------------------------------- int8 decode kernel (TMA-staged)
@pytest.mark.parametrize("n,k,g,m", [(1536, 576, 576, 1), (33, 256, 32, 1), (100, 1040, 16, 3), (2048, 4096, 128, 8),
                                     (31, 16, 16, 2), (4096, 2048, 64, 5)])
@pytest.mark.parametrize("xdt", ["f32", "f16"])
def test_int8_tma_kernel_matches_oracle_and_simt(n, k, g, m, xdt):
    """The TMA-staged int8 kernel (K % 16 == 0, G % 16 == 0, M <= 8; AUTO picks it from N = 16384 up) against the
    oracle, and against the CUDA-core kernel on the same inputs; partial last k tile, N tails."""
    rng = np.random.default_rng(n * 7 + k + m)
    w8, s8 = O.make_w8(rng, n, k, g, np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32 if xdt == "f32" else np.float16)
    code = _lib.F32 if xdt == "f32" else _lib.F16
    xd, wd, sd = torch.from_numpy(x).cuda(), torch.from_numpy(w8).cuda(), torch.from_numpy(s8).cuda()
    y = L.quantized_matmul(xd, wd, sd, g, bits=8, out_dtype="f32", algo="gemv_w8")
    ref = O.matmul_int8(x.astype(np.float32), w8, s8, g)
    _assert_f32_close(y.cpu().numpy(), ref)
    y_simt = L.quantized_matmul(xd, wd, sd, g, bits=8, out_dtype="f32", algo="simt")
    _assert_f32_close(y.cpu().numpy(), y_simt.cpu().numpy())
    if xdt == "f16":
        y16 = L.quantized_matmul(xd, wd, torch.from_numpy(s8.astype(np.float16)).cuda(), g, bits=8, algo="gemv_w8")
        assert y16.dtype == torch.float16
        _check16(y16.float().cpu().numpy(), O.matmul_int8(x.astype(np.float32), w8, s8.astype(np.float16), g))
    _device_status_ok()


def test_c_abi_sharding_context_with_one_rank():
    """lcq_shard_ctx_* at world = 1 (the two-rank form runs in tests/sharded_worker.py): create,
    no handles to exchange, two consecutive calls (the two regions alternate), destroy."""
    import ctypes
    lib = _lib.lib()
    n, k = 384 + 32, 2048
    rng = np.random.default_rng(11)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    wd, sd = torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda()
    ctx = ctypes.c_void_p()
    handles = ctypes.create_string_buffer(128)
    _lib.check(lib.lcq_shard_ctx_create(0, 1, 16 * n * 2, ctypes.byref(ctx), handles))
    try:
        torch.cuda.synchronize()
        for m in (1, 16):
            x = rng.standard_normal((m, k)).astype(np.float16)
            xd = torch.from_numpy(x).cuda()
            out_ptr = ctypes.c_void_p()
            _lib.check(lib.lcq_sharded_matmul_int4(ctx, xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), ctypes.byref(out_ptr),
                                                   m, n, k, 32, _lib.F16, _lib.F16, _lib.F16, _lib.ALGO_AUTO, None))
            torch.cuda.synchronize()

            class _Mem:
                __cuda_array_interface__ = {"shape": (m * n,), "typestr": "<f2", "data": (out_ptr.value, False), "version": 3}
            got = torch.as_tensor(_Mem(), device="cuda").cpu().numpy().reshape(m, n).astype(np.float32)
            ref = O.matmul_int4(x.astype(np.float32), wp, s, 32)
            assert np.all(np.abs(got - ref) <= 1e-2 + 1e-2 * np.abs(ref)), float(np.abs(got - ref).max())
        assert lib.lcq_check_device_status(None) == 0
        bad = ctypes.c_void_p()
        assert lib.lcq_sharded_matmul_int4(ctx, xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), ctypes.byref(bad), 32, n, k, 32,
                                           _lib.F16, _lib.F16, _lib.F16, _lib.ALGO_AUTO, None) == _lib.ERR_BAD_ARG   # slice over the limit
    finally:
        _lib.check(lib.lcq_shard_ctx_destroy(ctx))
