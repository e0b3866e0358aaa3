"""The quantized operators, with the reference's Python call surface.

Reference surface reproduced here (same names, argument order, defaults and result types):

  gpu_matvec_int4(x, w_packed, scales, group_size=32) -> np.ndarray[N]      examples/38_quantized_matmul.py:141-155
  gpu_matvec_int8(x, w_int8,  scales, group_size=32) -> np.ndarray[N]       examples/38_quantized_matmul.py:158-171
  gpu_dequant_int4(w_packed, scales, N, K, group_size=32) -> np.ndarray[N,K] examples/52_dequantize.py:81-93
  gpu_dequant_int8(w_int8,  scales, N, K, group_size=32) -> np.ndarray[N,K]  examples/52_dequantize.py:96-107
  dequant_matvec_int4[(N,), (128,)](X, W, scales, O, K_dim, HALF_K, NUM_SCALES, GROUP_SIZE)   examples/38...:30-39, :154
  dequant_matvec_int8[(N,), (128,)](X, W, scales, O, K_dim, NUM_SCALES, GROUP_SIZE)           examples/38...:94-102, :170
  dequant_int4[(N,), (128,)](W, SCALES, OUT, K, HALF_K, NUM_SCALES, GROUP_SIZE)               examples/52...:27-30, :90
  dequant_int8[(N,), (128,)](W, SCALES, OUT, K, NUM_SCALES, GROUP_SIZE)                       examples/52...:60-63, :104

Differences, all by extension: K need only be a multiple of group_size (the reference asserts
K % 256 / K % 128); x may be [M, K]; 16-bit activations, scales and outputs are accepted;
results can stay on the device.  `quantized_matmul` / `dequantize` are the device-resident
forms a decode or prefill loop calls.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from . import _lib
from .tensor import (KIND_TO_CODE, KIND_TO_TORCH, DeviceTensor, Operand, _require_cuda, current_stream_ptr,
                     resolve, workspace)

_ALGOS = {None: _lib.ALGO_AUTO, "auto": _lib.ALGO_AUTO, "simt": _lib.ALGO_SIMT,
          "gemv_tc": _lib.ALGO_GEMV_TC, "gemm_tc": _lib.ALGO_GEMM_TC, "gemv_w8": _lib.ALGO_GEMV_W8}


def _float_kind(op: Operand, name: str) -> int:
    if op.kind not in KIND_TO_CODE:
        raise TypeError(f"{name} must be float32, float16 or bfloat16, got {op.kind}")
    return KIND_TO_CODE[op.kind]


def _same_device(*ops: Operand) -> int:
    dev = ops[0].device
    for o in ops[1:]:
        if o.device != dev:
            raise ValueError("all operands must live on one device")
    return dev


# ------------------------------------------------------------------------------------------
# device-resident forms
# ------------------------------------------------------------------------------------------
def quantized_matmul(x, w, scales, group_size: int = 32, *, bits: int = 4, out=None, out_dtype: Optional[str] = None,
                     algo: Optional[str] = None, stream=None, bf16: bool = False,
                     workspace_buf: Optional[torch.Tensor] = None):
    """out[m, n] = sum_k x[m, k] * dequant(w)[n, k], float32 accumulation.

    x: [K] or [M, K] (f32 / f16 / bf16); w: uint8 [N, K/2] (bits=4) or int8 [N, K] (bits=8);
    scales: [N, K/group_size].  Returns a torch CUDA tensor [N] or [M, N] (or `out`).
    Stream-ordered on `stream` (default: torch's current stream); no host synchronisation.
    workspace_buf: a zero-initialised uint8 CUDA tensor to use as scratch instead of the
    per-stream buffer this module keeps (needed under CUDA-graph capture, where nothing may be
    allocated; see matmul_workspace_bytes).
    """
    xo = resolve(x, "x", bf16)
    wo = resolve(w, "w")
    so = resolve(scales, "scales")
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    if wo.kind != ("u8" if bits == 4 else "i8"):
        raise TypeError(f"int{bits} weights must be {'uint8' if bits == 4 else 'int8'}, got {wo.kind}")
    if len(xo.shape) not in (1, 2):
        raise ValueError(f"x must be [K] or [M, K], got shape {xo.shape}")
    squeeze = len(xo.shape) == 1
    M = 1 if squeeze else xo.shape[0]
    K = xo.shape[-1]
    if len(wo.shape) != 2:
        raise ValueError(f"weights must be 2-D [N, K{'/2' if bits == 4 else ''}], got shape {wo.shape}")
    N = wo.shape[0]
    wk = wo.shape[1] * (2 if bits == 4 else 1)
    if wk != K:
        raise ValueError(f"x has K={K} but the weights hold K={wk}")
    if group_size <= 0 or K % group_size:
        raise ValueError(f"K={K} must be a multiple of group_size={group_size}")
    if so.size != N * (K // group_size):
        raise ValueError(f"scales must hold N*K/group_size = {N * (K // group_size)} values, got {so.size}")
    xk, sk = _float_kind(xo, "x"), _float_kind(so, "scales")
    okind = out_dtype or xo.kind
    if okind not in KIND_TO_CODE:
        raise ValueError(f"out_dtype must be one of f32/f16/bf16, got {okind}")
    dev = _same_device(xo, wo, so)
    host_out = None
    _require_cuda()
    if out is None:
        res = torch.empty((M, N), dtype=KIND_TO_TORCH[okind], device=torch.device("cuda", dev))
        oo = resolve(res, "out")
    else:
        oo = resolve(out, "out", bf16 and okind == "bf16")
        if oo.size != M * N:
            raise ValueError(f"out must hold M*N = {M * N} values, got {oo.size}")
        if out_dtype is None:
            okind = oo.kind
        elif oo.kind != okind:
            raise TypeError(f"out is {oo.kind} but out_dtype={okind}")
        res = out
        host_out = oo.host
    L = _lib.lib()
    sp = current_stream_ptr(stream)
    a = _ALGOS[algo]
    if stream is not None and any(o.host is not None for o in (xo, wo, so, oo)):
        torch.cuda.current_stream().synchronize()   # host uploads ran on torch's current stream
    with torch.cuda.device(dev):
        ws_bytes = L.lcq_matmul_workspace_bytes(bits, M, N, K, group_size, xk, sk, KIND_TO_CODE[okind], a)
        if ws_bytes == (1 << 64) - 1:
            raise _lib.LcqError(_lib.ERR_UNSUPPORTED, f"algo {algo!r} does not cover this problem")
        if ws_bytes and workspace_buf is not None:
            if workspace_buf.numel() * workspace_buf.element_size() < ws_bytes or workspace_buf.device.index != dev:
                raise ValueError(f"workspace_buf must hold {ws_bytes} bytes on cuda:{dev}")
            ws = workspace_buf
        else:
            ws = workspace(ws_bytes, dev, sp) if ws_bytes else None
        fn = L.lcq_matmul_int4 if bits == 4 else L.lcq_matmul_int8
        _lib.check(fn(xo.ptr, wo.ptr, so.ptr, oo.ptr, M, N, K, group_size, xk, sk, KIND_TO_CODE[okind], a,
                      ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, sp))
    if host_out is not None:          # a NumPy output: copy the result back in place
        torch.cuda.current_stream().synchronize()
        host_out[...] = oo.keepalive.cpu().numpy().reshape(host_out.shape)
        return host_out
    if out is None and squeeze:
        return res[0]
    return res


def matmul_workspace_bytes(M: int, N: int, K: int, group_size: int = 32, bits: int = 4, x_kind: str = "f16",
                           scale_kind: str = "f16", out_kind: Optional[str] = None, algo: Optional[str] = None) -> int:
    """Scratch bytes quantized_matmul needs for this problem (0 if none)."""
    n = _lib.lib().lcq_matmul_workspace_bytes(bits, M, N, K, group_size, KIND_TO_CODE[x_kind], KIND_TO_CODE[scale_kind],
                                              KIND_TO_CODE[out_kind or x_kind], _ALGOS[algo])
    if n == (1 << 64) - 1:
        raise ValueError("no kernel covers this problem")
    return int(n)


def dequantize(w, scales, N: Optional[int] = None, K: Optional[int] = None, group_size: int = 32, *, bits: int = 4,
               out=None, out_dtype: str = "f32", stream=None):
    """out[r, k] = dequant(w)[r, k]; returns a torch CUDA tensor [N, K] (or `out`).
    w and scales may be flat, as the reference's wrappers pass them (examples/52_dequantize.py:86-87)."""
    wo = resolve(w, "w")
    so = resolve(scales, "scales")
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    if wo.kind != ("u8" if bits == 4 else "i8"):
        raise TypeError(f"int{bits} weights must be {'uint8' if bits == 4 else 'int8'}, got {wo.kind}")
    if N is None or K is None:
        if len(wo.shape) != 2:
            raise ValueError("N and K are required when the weights are flat")
        N, K = wo.shape[0], wo.shape[1] * (2 if bits == 4 else 1)
    N, K = int(N), int(K)
    per_row = K // 2 if bits == 4 else K
    if wo.size != N * per_row:
        raise ValueError(f"weights must hold {N * per_row} bytes for N={N}, K={K}, got {wo.size}")
    if group_size <= 0 or K % group_size or (bits == 4 and K % 2):
        raise ValueError(f"K={K} must be even and a multiple of group_size={group_size}")
    if so.size != N * (K // group_size):
        raise ValueError(f"scales must hold {N * (K // group_size)} values, got {so.size}")
    sk = _float_kind(so, "scales")
    dev = _same_device(wo, so)
    host_out = None
    _require_cuda()
    if out is None:
        if out_dtype not in KIND_TO_CODE:
            raise ValueError(f"out_dtype must be one of f32/f16/bf16, got {out_dtype}")
        res = torch.empty((N, K), dtype=KIND_TO_TORCH[out_dtype], device=torch.device("cuda", dev))
        oo = resolve(res, "out")
    else:
        oo = resolve(out, "out")
        if oo.size != N * K:
            raise ValueError(f"out must hold N*K = {N * K} values, got {oo.size}")
        res = out
        host_out = oo.host
    ok = _float_kind(oo, "out")
    L = _lib.lib()
    sp = current_stream_ptr(stream)
    with torch.cuda.device(dev):
        fn = L.lcq_dequant_int4 if bits == 4 else L.lcq_dequant_int8
        _lib.check(fn(wo.ptr, so.ptr, oo.ptr, N, K, group_size, sk, ok, sp))
    if host_out is not None:
        torch.cuda.current_stream().synchronize()
        host_out[...] = oo.keepalive.cpu().numpy().reshape(host_out.shape)
        return host_out
    return res


# ------------------------------------------------------------------------------------------
# the reference's wrapper functions (host arrays in, host arrays out)
# ------------------------------------------------------------------------------------------
def _to_host(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.float16).cpu().numpy()
    return t.cpu().numpy()


def gpu_matvec_int4(x, w_packed, scales, group_size=32, **kw):
    """INT4 quantized matvec. x:[K], w_packed:[N,K//2] uint8, scales:[N,K//G] -> host array [N].
    (examples/38_quantized_matmul.py:141-155; x may also be [M, K] -> [M, N].)
    Keyword extensions: return_device=True keeps the result on the GPU; out_dtype, algo, stream."""
    return_device = kw.pop("return_device", False)
    y = quantized_matmul(x, w_packed, scales, group_size, bits=4, **kw)
    return y if return_device else _to_host(y)


def gpu_matvec_int8(x, w_int8, scales, group_size=32, **kw):
    """INT8 quantized matvec. x:[K], w_int8:[N,K] int8, scales:[N,K//G] -> host array [N].
    (examples/38_quantized_matmul.py:158-171)"""
    return_device = kw.pop("return_device", False)
    y = quantized_matmul(x, w_int8, scales, group_size, bits=8, **kw)
    return y if return_device else _to_host(y)


def gpu_dequant_int4(w_packed, scales, N, K, group_size=32, **kw):
    """Dequantize INT4 packed weights -> host float32 [N, K] (examples/52_dequantize.py:81-93)."""
    return_device = kw.pop("return_device", False)
    y = dequantize(w_packed, scales, N, K, group_size, bits=4, **kw)
    return y if return_device else _to_host(y)


def gpu_dequant_int8(w_int8, scales, N, K, group_size=32, **kw):
    """Dequantize INT8 weights -> host float32 [N, K] (examples/52_dequantize.py:96-107)."""
    return_device = kw.pop("return_device", False)
    y = dequantize(w_int8, scales, N, K, group_size, bits=8, **kw)
    return y if return_device else _to_host(y)


# ------------------------------------------------------------------------------------------
# the reference's kernel-object call form: kernel[(grid,), (threadgroup,)](tensors..., constexprs...)
# ------------------------------------------------------------------------------------------
class _KernelCall:
    def __init__(self, kernel: "_Kernel", grid, tg):
        self.kernel, self.grid, self.tg = kernel, grid, tg

    def __call__(self, *args, **kwargs):
        names = self.kernel.params
        if len(args) > len(names):
            raise TypeError(f"{self.kernel.name} takes {len(names)} arguments, got {len(args)}")
        bound = dict(zip(names, args))
        for k, v in kwargs.items():
            if k not in names:
                raise TypeError(f"{self.kernel.name} has no parameter {k!r}")
            if k in bound:
                raise TypeError(f"{self.kernel.name} got multiple values for {k!r}")
            bound[k] = v
        missing = [n for n in names if n not in bound]
        if missing:
            raise TypeError(f"{self.kernel.name} missing arguments: {', '.join(missing)}")
        grid0 = self.grid[0] if isinstance(self.grid, (tuple, list)) else int(self.grid)
        self.kernel.run(int(grid0), bound)
        # the reference synchronises the device after every launch (locomp/api.py:852-854)
        torch.cuda.current_stream().synchronize()


class _Kernel:
    """`kernel[grid, threadgroup](...)`, as locomp.KernelLauncher.__getitem__ (locomp/api.py:480-487).
    The grid must equal the number of rows; the threadgroup size is accepted and ignored."""

    def __init__(self, name, params, run):
        self.name, self.params, self.run = name, params, run

    def __getitem__(self, launch):
        if not isinstance(launch, tuple) or len(launch) != 2:
            raise TypeError(f"{self.name}[grid, threadgroup] expects two entries")
        return _KernelCall(self, launch[0], launch[1])

    def __call__(self, *a, **k):
        raise TypeError(f"{self.name} must be launched as {self.name}[(grid,), (threadgroup,)](...)")


def _flat_rows(size: int, per_row: int, what: str) -> int:
    if per_row <= 0 or size % per_row:
        raise ValueError(f"{what}: {size} elements is not a whole number of rows of {per_row}")
    return size // per_row


def _run_matvec(bits: int):
    def run(grid0: int, a: dict):
        K, G, ns = int(a["K_dim"]), int(a["GROUP_SIZE"]), int(a["NUM_SCALES"])
        if G <= 0 or K % G or ns != K // G:
            raise ValueError(f"NUM_SCALES={ns} must equal K_dim/GROUP_SIZE = {K}/{G}")
        if bits == 4 and int(a["HALF_K"]) != K // 2:
            raise ValueError(f"HALF_K={a['HALF_K']} must equal K_dim/2 = {K // 2}")
        wo = resolve(a["W"], "W")
        N = _flat_rows(wo.size, K // 2 if bits == 4 else K, "W")
        if grid0 != N:
            raise ValueError(f"grid ({grid0},) must equal the number of weight rows N={N}")
        xo = resolve(a["X"], "X")
        if xo.size != K:
            raise ValueError(f"X must hold K_dim={K} values, got {xo.size}")
        w2 = _view(a["W"], wo, (N, K // 2 if bits == 4 else K))
        x1 = _view(a["X"], xo, (K,))
        quantized_matmul(x1, w2, a["scales"], G, bits=bits, out=a["O"])
    return run


def _run_dequant(bits: int):
    def run(grid0: int, a: dict):
        K, G, ns = int(a["K"]), int(a["GROUP_SIZE"]), int(a["NUM_SCALES"])
        if G <= 0 or K % G or ns != K // G:
            raise ValueError(f"NUM_SCALES={ns} must equal K/GROUP_SIZE = {K}/{G}")
        if bits == 4 and int(a["HALF_K"]) != K // 2:
            raise ValueError(f"HALF_K={a['HALF_K']} must equal K/2 = {K // 2}")
        wo = resolve(a["W"], "W")
        N = _flat_rows(wo.size, K // 2 if bits == 4 else K, "W")
        if grid0 != N:
            raise ValueError(f"grid ({grid0},) must equal the number of weight rows N={N}")
        dequantize(a["W"], a["SCALES"], N, K, G, bits=bits, out=a["OUT"])
    return run


def _view(orig, op: Operand, shape):
    """Reshape a flat operand without copying (device objects) or by NumPy reshape (host)."""
    if isinstance(orig, np.ndarray):
        return orig.reshape(shape)
    if isinstance(orig, DeviceTensor):
        return orig.torch().view(shape)
    if isinstance(orig, torch.Tensor):
        return orig.view(shape)

    class _Shim:   # foreign CUDATensor: same pointer, new shape
        _cuda_ptr, dtype = op.ptr, getattr(orig, "dtype")
    s = _Shim()
    s.shape = tuple(shape)
    s._owner = orig
    return s


dequant_matvec_int4 = _Kernel("dequant_matvec_int4",
                              ["X", "W", "scales", "O", "K_dim", "HALF_K", "NUM_SCALES", "GROUP_SIZE"], _run_matvec(4))
dequant_matvec_int8 = _Kernel("dequant_matvec_int8",
                              ["X", "W", "scales", "O", "K_dim", "NUM_SCALES", "GROUP_SIZE"], _run_matvec(8))
dequant_int4 = _Kernel("dequant_int4", ["W", "SCALES", "OUT", "K", "HALF_K", "NUM_SCALES", "GROUP_SIZE"],
                       _run_dequant(4))
dequant_int8 = _Kernel("dequant_int8", ["W", "SCALES", "OUT", "K", "NUM_SCALES", "GROUP_SIZE"], _run_dequant(8))
