"""The decode-step operators on either side of the quantized linears, and the weight quantisers.

Reference surface reproduced here (same names, argument order and launch form):

  rms_norm_kernel[(rows,), (128,)](X, W, O, N, EPS_X1000)      examples/54_smollm2_inference.py:40-73, :488-489
  silu_mul_kernel[(N,)](gate, up, O, N)                        examples/54_smollm2_inference.py:113-120, :549
  add_inplace_kernel[(N,)](A, B, N)                            examples/54_smollm2_inference.py:164-167, :530
  embed_lookup(token_ids, table, out, seq_len, dim)            locomp/api.py:1025-1038
  quantize_int4(weights, group_size=32) -> (packed, scales)    examples/38_quantized_matmul.py:248-271
  quantize_int8(weights, group_size=32) -> (w_int8, scales)    examples/38_quantized_matmul.py:274-293
  quantize_int4_ref(w, group_size=32)   -> (packed, scales)    examples/52_dequantize.py:110-126

plus the device-resident forms a decode loop calls (`rms_norm`, `residual_rms_norm`, `silu_mul`,
`add_inplace`, `argmax`, `quantize`) and `QuantizedWeight`, the container of a packed weight.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib
from .ops import _Kernel, _float_kind
from .tensor import KIND_TO_TORCH, Operand, _require_cuda, current_stream_ptr, resolve


def _same(*ops: Operand) -> Tuple[int, int]:
    kind, dev = ops[0].kind, ops[0].device
    for o in ops[1:]:
        if o.kind != kind:
            raise TypeError(f"all tensors of the call must share one dtype, got {kind} and {o.kind}")
        if o.device != dev:
            raise ValueError("all operands must live on one device")
    return kind, dev


def _finish(out_op: Operand, res):
    """Copy a NumPy output back in place (host callers), else return the device result."""
    if out_op.host is not None:
        torch.cuda.current_stream().synchronize()
        out_op.host[...] = out_op.keepalive.cpu().numpy().reshape(out_op.host.shape)
        return out_op.host
    return res


# ------------------------------------------------------------------------------------------ norm / activation / residual
def rms_norm(x, weight, eps: float = 1e-5, *, out=None, stream=None, bf16: bool = False):
    """out[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * weight; x is [n] or [rows, n]."""
    xo, wo = resolve(x, "x", bf16), resolve(weight, "weight", bf16)
    n = xo.shape[-1] if xo.shape else 0
    if wo.size != n:
        raise ValueError(f"weight must hold n = {n} values, got {wo.size}")
    rows = xo.size // n if n else 0
    _require_cuda()
    if out is None:
        res = torch.empty(xo.shape, dtype=KIND_TO_TORCH[xo.kind], device=torch.device("cuda", xo.device))
        oo = resolve(res, "out")
    else:
        oo, res = resolve(out, "out", bf16), out
        if oo.size != xo.size:
            raise ValueError(f"out must hold {xo.size} values, got {oo.size}")
    kind, dev = _same(xo, wo, oo)
    code = _float_kind(xo, "x")
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().lcq_rms_norm(xo.ptr, wo.ptr, oo.ptr, rows, n, float(eps), code, current_stream_ptr(stream)))
    return _finish(oo, res)


def residual_rms_norm(hidden, delta, weight, eps: float = 1e-5, *, out=None, stream=None, bf16: bool = False):
    """hidden += delta (in place), then out = rms_norm(hidden, weight): the residual add and the
    norm that follows it in the layer (examples/54_smollm2_inference.py:529-534) as one launch.
    `hidden` must be device-resident (it is updated in place).  Returns out."""
    ho, do, wo = resolve(hidden, "hidden", bf16), resolve(delta, "delta", bf16), resolve(weight, "weight", bf16)
    if ho.host is not None:
        raise TypeError("hidden is updated in place and must be a device tensor")
    n = ho.shape[-1] if ho.shape else 0
    if do.size != ho.size or wo.size != n:
        raise ValueError("delta must match hidden and weight must hold its last dimension")
    rows = ho.size // n if n else 0
    _require_cuda()
    if out is None:
        res = torch.empty(ho.shape, dtype=KIND_TO_TORCH[ho.kind], device=torch.device("cuda", ho.device))
        oo = resolve(res, "out")
    else:
        oo, res = resolve(out, "out", bf16), out
        if oo.size != ho.size:
            raise ValueError(f"out must hold {ho.size} values, got {oo.size}")
    kind, dev = _same(ho, do, wo, oo)
    code = _float_kind(ho, "hidden")
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().lcq_residual_rms_norm(ho.ptr, do.ptr, wo.ptr, oo.ptr, rows, n, float(eps), code,
                                                    current_stream_ptr(stream)))
    return _finish(oo, res)


def silu_mul(gate, up, *, out=None, stream=None, bf16: bool = False):
    """out = gate * sigmoid(gate) * up, elementwise."""
    go, uo = resolve(gate, "gate", bf16), resolve(up, "up", bf16)
    if go.size != uo.size:
        raise ValueError("gate and up must have the same number of elements")
    _require_cuda()
    if out is None:
        res = torch.empty(go.shape, dtype=KIND_TO_TORCH[go.kind], device=torch.device("cuda", go.device))
        oo = resolve(res, "out")
    else:
        oo, res = resolve(out, "out", bf16), out
        if oo.size != go.size:
            raise ValueError(f"out must hold {go.size} values, got {oo.size}")
    kind, dev = _same(go, uo, oo)
    code = _float_kind(go, "gate")
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().lcq_silu_mul(go.ptr, uo.ptr, oo.ptr, go.size, code, current_stream_ptr(stream)))
    return _finish(oo, res)


def add_inplace(a, b, *, stream=None, bf16: bool = False):
    """a += b, elementwise; `a` must be device-resident.  Returns a."""
    ao, bo = resolve(a, "a", bf16), resolve(b, "b", bf16)
    if ao.host is not None:
        raise TypeError("a is updated in place and must be a device tensor")
    if ao.size != bo.size:
        raise ValueError("a and b must have the same number of elements")
    kind, dev = _same(ao, bo)
    code = _float_kind(ao, "a")
    _require_cuda()
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().lcq_add_inplace(ao.ptr, bo.ptr, ao.size, code, current_stream_ptr(stream)))
    return a


# ------------------------------------------------------------------------------------------ embedding / sampling
def embed_lookup(token_ids, table, out, seq_len: int, dim: int, *, stream=None, bf16: bool = False) -> None:
    """out[i] = table[token_ids[i]] for i in range(seq_len) (locomp.embed_lookup, locomp/api.py:1025-1038).
    token_ids: int32 [seq_len]; table: [vocab, dim]; out: [seq_len * dim], same dtype as table."""
    io, to, oo = resolve(token_ids, "token_ids"), resolve(table, "table", bf16), resolve(out, "out", bf16)
    if io.kind != "i32":
        raise TypeError(f"token_ids must be int32, got {io.kind}")
    seq_len, dim = int(seq_len), int(dim)
    if io.size < seq_len:
        raise ValueError(f"token_ids holds {io.size} ids, seq_len is {seq_len}")
    if dim <= 0 or to.size % dim:
        raise ValueError(f"table of {to.size} values is not a whole number of rows of dim {dim}")
    if oo.size < seq_len * dim:
        raise ValueError(f"out must hold seq_len * dim = {seq_len * dim} values, got {oo.size}")
    kind, dev = _same(to, oo)
    code = _float_kind(to, "table")
    _require_cuda()
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().lcq_embed_lookup(io.ptr, to.ptr, oo.ptr, seq_len, to.size // dim, dim, code,
                                               current_stream_ptr(stream)))
    _finish(oo, None)


def argmax(x, *, out=None, stream=None, bf16: bool = False):
    """Index of the first maximum of each row of x ([n] or [rows, n]) as int32, computed on the
    device: the host-side np.argmax of examples/54_smollm2_inference.py:606 without the download."""
    xo = resolve(x, "x", bf16)
    if not xo.shape or xo.shape[-1] == 0:
        raise ValueError("argmax needs at least one element per row")
    n = xo.shape[-1]
    rows = xo.size // n
    code = _float_kind(xo, "x")
    _require_cuda()
    if out is None:
        res = torch.empty(xo.shape[:-1], dtype=torch.int32, device=torch.device("cuda", xo.device))
        oo = resolve(res, "out")
    else:
        oo, res = resolve(out, "out"), out
        if oo.kind != "i32" or oo.size != rows:
            raise ValueError(f"out must be int32 with {rows} elements")
    with torch.cuda.device(xo.device):
        _lib.check(_lib.lib().lcq_argmax(xo.ptr, oo.ptr, rows, n, code, current_stream_ptr(stream)))
    return _finish(oo, res)


# ------------------------------------------------------------------------------------------ kernel-object forms
def _run_rms_norm(grid0: int, a: dict):
    n = int(a["N"])
    xo = resolve(a["X"], "X")
    if n <= 0 or xo.size < grid0 * n:
        raise ValueError(f"X must hold grid * N = {grid0 * n} values")
    eps = int(a["EPS_X1000"]) * 0.000001          # the kernel's own scaling (examples/54_smollm2_inference.py:46)
    code = _float_kind(xo, "X")
    wo, oo = resolve(a["W"], "W"), resolve(a["O"], "O")
    _same(xo, wo, oo)
    _require_cuda()
    with torch.cuda.device(xo.device):
        _lib.check(_lib.lib().lcq_rms_norm(xo.ptr, wo.ptr, oo.ptr, grid0, n, eps, code, current_stream_ptr(None)))
    _finish(oo, None)


def _run_silu_mul(grid0: int, a: dict):
    n = int(a["N"])
    if grid0 != n:
        raise ValueError(f"grid ({grid0},) must equal N={n}")
    go, uo, oo = resolve(a["gate"], "gate"), resolve(a["up"], "up"), resolve(a["O"], "O")
    _same(go, uo, oo)
    _require_cuda()
    with torch.cuda.device(go.device):
        _lib.check(_lib.lib().lcq_silu_mul(go.ptr, uo.ptr, oo.ptr, n, _float_kind(go, "gate"), current_stream_ptr(None)))
    _finish(oo, None)


def _run_add_inplace(grid0: int, a: dict):
    n = int(a["N"])
    if grid0 != n:
        raise ValueError(f"grid ({grid0},) must equal N={n}")
    ao, bo = resolve(a["A"], "A"), resolve(a["B"], "B")
    _same(ao, bo)
    _require_cuda()
    with torch.cuda.device(ao.device):
        _lib.check(_lib.lib().lcq_add_inplace(ao.ptr, bo.ptr, n, _float_kind(ao, "A"), current_stream_ptr(None)))
    _finish(ao, None)


class _Kernel1(_Kernel):
    """Kernel object that also accepts the one-entry launch form `kernel[(N,)](...)` the reference
    uses for its elementwise kernels (threadgroup defaults, locomp/api.py:480-487)."""

    def __getitem__(self, launch):
        if isinstance(launch, tuple) and len(launch) == 1 and isinstance(launch[0], int):
            launch = ((launch[0],), (1,))                    # kernel[(N,)]  ==  kernel[N,]
        elif isinstance(launch, tuple) and len(launch) == 1:
            launch = (launch[0], (1,))
        elif isinstance(launch, int):
            launch = ((launch,), (1,))
        return super().__getitem__(launch)


rms_norm_kernel = _Kernel1("rms_norm_kernel", ["X", "W", "O", "N", "EPS_X1000"], _run_rms_norm)
silu_mul_kernel = _Kernel1("silu_mul_kernel", ["gate", "up", "O", "N"], _run_silu_mul)
add_inplace_kernel = _Kernel1("add_inplace_kernel", ["A", "B", "N"], _run_add_inplace)


# ------------------------------------------------------------------------------------------ quantisers
@dataclass
class QuantizedWeight:
    """A quantized weight in the wire layout of the reference's operators: `w` uint8 [N, K/2]
    (low nibble = even k, stored value q + 8) or int8 [N, K]; `scales` [N, K/group_size]."""
    w: torch.Tensor
    scales: torch.Tensor
    group_size: int
    bits: int

    @property
    def shape(self) -> Tuple[int, int]:
        return self.w.shape[0], self.w.shape[1] * (2 if self.bits == 4 else 1)

    def save(self, path: str) -> None:
        """Write the packed bytes and scales as an .npz file (host copy)."""
        np.savez(path, w=self.w.cpu().numpy(), scales=self.scales.cpu().numpy(),
                 group_size=np.int64(self.group_size), bits=np.int64(self.bits))

    @staticmethod
    def load(path: str, device="cuda") -> "QuantizedWeight":
        d = np.load(path if str(path).endswith(".npz") else str(path) + ".npz")
        return QuantizedWeight(torch.from_numpy(d["w"]).to(device), torch.from_numpy(d["scales"]).to(device),
                               int(d["group_size"]), int(d["bits"]))

    def linear(self):
        from .linear import QuantLinear
        return QuantLinear(self.w, self.scales, self.group_size, self.bits)


def quantize(weights, group_size: int = 32, *, bits: int = 4, style: str = "ex38", scale_dtype: Optional[str] = None,
             stream=None) -> QuantizedWeight:
    """Quantize a float weight [N, K] on the device; returns a QuantizedWeight (device-resident).
    style "ex38": quantize_int4 / quantize_int8 of examples/38_quantized_matmul.py:248-293;
    style "ex52": quantize_int4_ref of examples/52_dequantize.py:110-126.
    Scales are float32 as in the reference; scale_dtype="f16" additionally rounds them to fp16
    (the W4A16 kernels' scale type)."""
    wo = resolve(weights, "weights")
    if len(wo.shape) != 2:
        raise ValueError(f"weights must be 2-D [N, K], got shape {wo.shape}")
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    if style not in ("ex38", "ex52"):
        raise ValueError("style must be 'ex38' or 'ex52'")
    n, k = wo.shape
    if group_size <= 0 or k % group_size or (bits == 4 and group_size % 2):
        raise ValueError(f"K={k} must be a multiple of group_size={group_size} (even for int4)")
    code = _float_kind(wo, "weights")
    _require_cuda()
    dev = torch.device("cuda", wo.device)
    q = torch.empty((n, k // 2) if bits == 4 else (n, k), dtype=torch.uint8 if bits == 4 else torch.int8, device=dev)
    s = torch.empty((n, k // group_size), dtype=torch.float32, device=dev)
    fn = _lib.lib().lcq_quantize_int4 if bits == 4 else _lib.lib().lcq_quantize_int8
    with torch.cuda.device(wo.device):
        _lib.check(fn(wo.ptr, q.data_ptr(), s.data_ptr(), n, k, group_size, code, 0 if style == "ex38" else 1,
                      current_stream_ptr(stream)))
    if scale_dtype not in (None, "f32"):
        s = s.to(KIND_TO_TORCH[scale_dtype])
    return QuantizedWeight(q, s, group_size, bits)


def quantize_int4(weights, group_size=32):
    """float32 [N, K] -> (packed uint8 [N, K/2], scales float32 [N, K/G]) as host arrays
    (examples/38_quantized_matmul.py:248-271)."""
    qw = quantize(np.ascontiguousarray(weights, dtype=np.float32), group_size, bits=4, style="ex38")
    return qw.w.cpu().numpy(), qw.scales.cpu().numpy()


def quantize_int8(weights, group_size=32):
    """float32 [N, K] -> (int8 [N, K], scales float32 [N, K/G]) as host arrays
    (examples/38_quantized_matmul.py:274-293)."""
    qw = quantize(np.ascontiguousarray(weights, dtype=np.float32), group_size, bits=8, style="ex38")
    return qw.w.cpu().numpy(), qw.scales.cpu().numpy()


def quantize_int4_ref(w, group_size=32):
    """The packer of examples/52_dequantize.py:110-126 (amax floored at 1e-10, divisor scale + 1e-10)."""
    qw = quantize(np.ascontiguousarray(w, dtype=np.float32), group_size, bits=4, style="ex52")
    return qw.w.cpu().numpy(), qw.scales.cpu().numpy()
