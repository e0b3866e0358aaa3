"""Parity at the FULL shapes of the benchmark configurations: the SmolLM2-135M decode shapes
(K = 576 / 1536, vocabulary 49152), the Llama-3-8B-like prefill shapes (M up to 8192) and the
70B-class shapes (K = 28672, N = 128256 and its eighth 16032).

Each case draws its inputs from np.random.default_rng(0) in the order weights, scales,
activations, feeds identical bytes to the kernel and to the checkers, and is checked twice:
  * exactly, against the float64-accumulating NumPy oracle, on a sample of weight rows (always
    including the first and last rows, i.e. the N tail) and, for large M, of activation rows;
  * in full, against a float64 matmul (on the GPU) of the dequantised weights, which the
    dequantize kernel produces and whose sampled rows are compared bit for bit with the oracle.
Bar: |err| <= 1e-2 + 1e-2 |ref| for 16-bit activations and outputs.
"""
import functools

import numpy as np
import pytest
import torch

import locomp_b200 as L
from locomp_b200 import _lib
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu

RTOL16, ATOL16 = 1e-2, 1e-2
ALGO_NAMES = {_lib.ALGO_SIMT: "simt", _lib.ALGO_GEMV_TC: "gemv_tc", _lib.ALGO_GEMM_TC: "gemm_tc"}


def _bits32(a):
    return np.ascontiguousarray(a).view(np.uint32)


def _check16(y, ref, what=""):
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    bad = np.abs(y - ref) > ATOL16 + RTOL16 * np.abs(ref)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance; max err {np.abs(y - ref).max():.4g}"


@functools.lru_cache(maxsize=2)
def _weights(k, n):
    """Seeded weights of one shape: host arrays and their device copies."""
    rng = np.random.default_rng(0)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    return wp, s, torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda(), rng


def _sample_rows(n, count, seed):
    rng = np.random.default_rng(seed)
    count = min(count, n)
    rows = set(rng.choice(n, size=count, replace=False).tolist())
    rows.update(range(min(8, n)))
    rows.update(range(max(0, n - 8), n))        # the N tail (last, possibly partial, row block)
    return np.array(sorted(rows))


def _full_reference(x_dev, wd, sd, n, k):
    """float64 X @ dequant(W)^T on the GPU, in row blocks of W; the dequantised rows come from
    the dequantize kernel (bit-exact against the oracle, asserted on sampled rows by the caller)."""
    out = torch.empty(x_dev.shape[0], n, dtype=torch.float64, device="cuda")
    xd = x_dev.double()
    step = 8192
    for r0 in range(0, n, step):
        r1 = min(n, r0 + step)
        wdq = L.dequantize(wd[r0:r1], sd[r0:r1], r1 - r0, k, 32)            # float32 [rows, K]
        out[:, r0:r1] = xd @ wdq.double().T
    return out


def _run_case(k, n, m, x_host_f32, x_dev, expect_algo, seed):
    wp, s, wd, sd, _ = _weights(k, n)
    code = _lib.F16 if x_dev.dtype == torch.float16 else _lib.BF16
    algo = _lib.lib().lcq_matmul_select_algo(4, m, n, k, 32, code, _lib.F16, code)
    assert ALGO_NAMES[algo] == expect_algo
    y = L.quantized_matmul(x_dev, wd, sd, 32)
    assert y.dtype == x_dev.dtype and tuple(y.shape) == (m, n)
    assert _lib.lib().lcq_check_device_status(None) == 0, _lib.lib().lcq_last_error()
    # exact oracle on sampled weight rows x sampled activation rows
    wrows = _sample_rows(n, 256, seed)
    xrows = _sample_rows(m, 64, seed + 1)
    ref = O.matmul_int4(x_host_f32[xrows], wp[wrows], s[wrows], 32)
    got = y[torch.from_numpy(xrows).cuda()][:, torch.from_numpy(wrows).cuda()].float().cpu().numpy()
    _check16(got, ref, "sampled rows vs NumPy oracle")
    # the dequantised weights used by the full check are bit-exact on the same sampled rows
    wdq = L.dequantize(wd[torch.from_numpy(wrows).cuda()].contiguous(), sd[torch.from_numpy(wrows).cuda()].contiguous(),
                       len(wrows), k, 32)
    assert np.array_equal(_bits32(wdq.cpu().numpy()), _bits32(O.dequant_int4(wp[wrows], s[wrows], 32)))
    # full output
    full = _full_reference(x_dev, wd, sd, n, k)
    err = (y.double() - full).abs()
    bad = err > ATOL16 + RTOL16 * full.abs()
    assert not bool(bad.any()), f"full output: {int(bad.sum())} of {bad.numel()} outside tolerance; max err {float(err.max()):.4g}"
    # a second run on the reused workspace gives the same bits
    assert torch.equal(L.quantized_matmul(x_dev, wd, sd, 32), y)
    assert _lib.lib().lcq_check_device_status(None) == 0


# --------------------------------------------------------------------------- prefill shapes (bf16)
CFG4_SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096)]


@pytest.mark.parametrize("m", [512, 2048, 8192])
@pytest.mark.parametrize("k,n", CFG4_SHAPES)          # innermost decorator = slowest: one weight draw per shape
def test_prefill_shapes_bf16(k, n, m):
    """M in {512, 2048, 8192} x the Llama-3-8B-like shapes, bf16 in and out, tcgen05 kernel by
    AUTO dispatch.  M = 8192 makes every CTA walk many output tiles (multi-wave persistent loop)."""
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    _run_case(k, n, m, x.float().numpy(), x.cuda(), "gemm_tc", seed=m + n)


@pytest.mark.parametrize("m,n,k", [(2048, 4096, 512), (512, 14336, 256), (1000, 3000, 256)])
@pytest.mark.parametrize("xdt", [torch.float16, torch.bfloat16])
def test_prefill_kernel_more_tiles_than_sms(m, n, k, xdt):
    """More output tiles than SMs with a small K: the persistent loop of every CTA runs past its
    first tile (accumulator hand-off phases, ring counters carried across tiles), N tile tails."""
    rng = np.random.default_rng(m + n + k)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(1)).to(xdt)
    wd, sd = torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda()
    y = L.quantized_matmul(x.cuda(), wd, sd, 32, algo="gemm_tc")
    ref = x.float().numpy().astype(np.float64) @ O.dequant_int4(wp, s, 32).astype(np.float64).T
    _check16(y.float().cpu().numpy(), ref, "tcgen05 kernel, many tiles per CTA")
    assert _lib.lib().lcq_check_device_status(None) == 0


# --------------------------------------------------------------------------- 70B-class shapes (fp16)
CFG5_SHAPES = [(8192, 28672), (28672, 8192), (8192, 128256), (8192, 16032)]


@pytest.mark.parametrize("m", [1, 16, 64])
@pytest.mark.parametrize("k,n", CFG5_SHAPES)
def test_70b_class_shapes_fp16(k, n, m):
    """(K, N) of the column-sharded configuration unsharded, plus the eighth of the vocabulary
    projection (N = 16032, not a multiple of the 128-row tile).  M = 1 and 16 go through the
    decode kernel -- K = 28672 is its longest float32 group-sum chain and most k ranges --,
    M = 64 through the tcgen05 kernel, except at K = 28672, where AUTO keeps the decode kernel in
    16-row chunks (the fp16 weight tiles of the tcgen05 kernel are not accurate enough there)."""
    _, _, _, _, rng = _weights(k, n)
    xs = getattr(test_70b_class_shapes_fp16, "_x", {})
    if (k, n) not in xs:                       # one activation draw per shape; M rows are its first M
        xs.clear()
        xs[(k, n)] = rng.standard_normal((64, k)).astype(np.float16)
        test_70b_class_shapes_fp16._x = xs
    x = np.ascontiguousarray(xs[(k, n)][:m])
    _run_case(k, n, m, x.astype(np.float32), torch.from_numpy(x).cuda(),
              "gemv_tc" if (m <= 16 or k > 16384) else "gemm_tc", seed=m + n)


# --------------------------------------------------------------------------- SmolLM2-135M decode shapes
CFG3_SHAPES = [(576, 576), (576, 192), (576, 1536), (1536, 576), (576, 49152)]     # (K, N)


@pytest.mark.parametrize("k,n", CFG3_SHAPES)
@pytest.mark.parametrize("m", [1, 4])
def test_decode_stack_shapes_fp16(k, n, m):
    """q/o, k/v, gate/up, down and the lm_head of the 30-layer stack, fp16, against the oracle in
    full (these weights are small enough for NumPy)."""
    rng = np.random.default_rng(0)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    x = rng.standard_normal((4, k)).astype(np.float16)[:m]
    y = L.quantized_matmul(torch.from_numpy(np.ascontiguousarray(x)).cuda(), torch.from_numpy(wp).cuda(),
                           torch.from_numpy(s).cuda(), 32)
    assert y.dtype == torch.float16 and tuple(y.shape) == (m, n)
    ref = np.concatenate([O.matmul_int4(x.astype(np.float32), wp[i:i + 8192], s[i:i + 8192], 32)
                          for i in range(0, n, 8192)], axis=-1)
    _check16(y.float().cpu().numpy(), ref, f"(K,N)=({k},{n}) M={m}")
    assert _lib.lib().lcq_check_device_status(None) == 0


@pytest.mark.parametrize("fused", [False, True])
def test_decode_stack_step_against_oracle(fused):
    """Every linear of a (2-layer) DecodeStack step, eager and replayed from its CUDA graph,
    against the oracle on that linear's own weights and input."""
    st = L.DecodeStack(layers=2, fused=fused, seed=3)
    st.step()
    torch.cuda.synchronize()
    refs = []
    for lin, x, out in st.calls:
        ref = O.matmul_int4(x.float().cpu().numpy(), lin.w.cpu().numpy(), lin.scales.cpu().numpy(), 32)
        _check16(out.float().cpu().numpy(), ref, f"eager, N={lin.out_features} K={lin.in_features}")
        refs.append(ref)
    st.capture()
    for c in st.calls:
        c[2].zero_()
    st.replay()
    torch.cuda.synchronize()
    for (lin, x, out), ref in zip(st.calls, refs):
        _check16(out.float().cpu().numpy(), ref, f"graph, N={lin.out_features} K={lin.in_features}")
    assert _lib.lib().lcq_check_device_status(None) == 0


# --------------------------------------------------------------------------- decode kernel, M > 16 in chunks
def test_decode_kernel_with_a_tail_chunk_sizes_its_workspace():
    """M = 24 through the decode kernel: a 16-row chunk and an 8-row tail whose plan needs more
    scratch than the full chunk's; the size query covers both."""
    m, n, k = 24, 2048, 8192
    rng = np.random.default_rng(24)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    x = rng.standard_normal((m, k)).astype(np.float16)
    from locomp_b200.ops import matmul_workspace_bytes
    need = matmul_workspace_bytes(m, n, k, 32, 4, "f16", "f16", "f16", "gemv_tc")
    assert need >= matmul_workspace_bytes(8, n, k, 32, 4, "f16", "f16", "f16", "gemv_tc")
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    y = L.quantized_matmul(torch.from_numpy(x).cuda(), torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda(), 32,
                           algo="gemv_tc", workspace_buf=ws)
    _check16(y.float().cpu().numpy(), O.matmul_int4(x.astype(np.float32), wp, s, 32), "M=24 decode kernel")
    assert _lib.lib().lcq_check_device_status(None) == 0


# --------------------------------------------------------------------------- activation range (bf16)
@pytest.mark.parametrize("scale", [1e-3, 1.0, 1e3])
@pytest.mark.parametrize("m", [3, 48])
def test_bf16_activation_range(scale, m):
    """bf16 activations scaled by 1e-3 and 1e3 through the tensor-core kernels, which convert them
    to fp16 (and the decode kernel divides half of them by 16, into fp16's subnormal range at
    1e-3): results stay inside the tolerance relative to the oracle."""
    n, k = 512, 2048
    rng = np.random.default_rng(17)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    x = (torch.randn(m, k, generator=torch.Generator().manual_seed(4)) * scale).to(torch.bfloat16)
    y = L.quantized_matmul(x.cuda(), torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda(), 32, out_dtype="f32")
    ref = O.matmul_int4(x.float().numpy(), wp, s, 32)
    err = np.abs(y.cpu().numpy() - ref)
    # scale-invariant form of the bar: 1e-2 relative plus 1e-2 of the output's RMS magnitude
    tol = 1e-2 * np.abs(ref) + 1e-2 * float(np.sqrt(np.mean(ref ** 2)))
    assert np.all(err <= tol), f"scale {scale}: max err {err.max():.4g}"


_CLUSTER_CASE = r"""
import sys
import numpy as np, torch
sys.path.insert(0, {root!r})
import locomp_b200 as L
from oracle import qmm_oracle as O
outs = {{}}
for (n, k, m) in ((2048, 2048, 1), (2048, 8192, 4), (1000, 2048, 8), (2048, 2048, 16), (640, 576, 3)):
    rng = np.random.default_rng(n + k + m)
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    x = rng.standard_normal((m, k)).astype(np.float16)
    y = L.quantized_matmul(torch.from_numpy(x).cuda(), torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda(), 32,
                           out_dtype="f32", algo="gemv_tc")
    outs[f"{{n}}_{{k}}_{{m}}"] = y.float().cpu().numpy()
np.savez({path!r}, **outs)
"""


def test_cluster_mode_and_scratch_mode_agree(tmp_path):
    """The small-problem plans with cluster mode on (partial sums meet in the cluster leader's shared
    memory) and with LCQ_GEMV_CLUSTER=0 (whole row blocks per CTA, or global scratch) differ only in
    how the float32 partial sums are associated: outputs agree to float32 round-off.  The switch is
    read once per process, hence two child processes."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = _lib.lib()
    assert lib.lcq_gemv_tc_plan_cluster(1, 2048, 2048, 148) > 1      # the first case does run as clusters
    results = []
    for cluster in ("1", "0"):
        path = str(tmp_path / f"cluster_{cluster}.npz")
        env = dict(os.environ, LCQ_GEMV_CLUSTER=cluster)
        out = subprocess.run([sys.executable, "-c", _CLUSTER_CASE.format(root=root, path=path)], capture_output=True,
                             text=True, timeout=300, env=env, cwd=root)
        assert out.returncode == 0, out.stderr[-800:]
        results.append(np.load(path))
    for key in results[0].files:
        a, b = results[0][key], results[1][key]
        scale = float(np.sqrt(np.mean(a.astype(np.float64) ** 2)))
        assert np.abs(a - b).max() <= 2e-5 * scale, (key, float(np.abs(a - b).max()), scale)
