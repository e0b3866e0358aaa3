"""Device tensors for the quantized operators.

`DeviceTensor` has the attribute set of the reference's CUDATensor
(locomp/backends/cuda_runtime.py:52-97: `_cuda_ptr`, `size`, `dtype`, `shape`, `.numpy()`,
`.free()`), and `tensor` / `empty` / `zeros` mirror the factories the reference's wrappers
call (locomp/api.py:323-402).  Memory is owned by a torch CUDA tensor; torch is used for
allocation and copies only.

`resolve` turns anything the reference's launcher accepts (locomp/api.py:826-843) -- a
device tensor, a NumPy array (uploaded for the call), plus torch CUDA tensors and any
object exposing `_cuda_ptr`/`dtype`/`shape` -- into a raw pointer plus metadata.  Unlike the
reference, which uploads bytes as they are and lets a kernel misread a wrong dtype, the
dtype is checked here.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import numpy as np
import torch

from . import _lib

_NP_TO_TORCH = {
    np.dtype(np.float32): torch.float32,
    np.dtype(np.float16): torch.float16,
    np.dtype(np.uint8): torch.uint8,
    np.dtype(np.int8): torch.int8,
    np.dtype(np.int32): torch.int32,
}
_TORCH_TO_KIND = {
    torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16",
    torch.uint8: "u8", torch.int8: "i8", torch.int32: "i32",
}
_NP_TO_KIND = {np.dtype(np.float32): "f32", np.dtype(np.float16): "f16", np.dtype(np.uint8): "u8",
               np.dtype(np.int8): "i8", np.dtype(np.int32): "i32"}
KIND_TO_CODE = {"f32": _lib.F32, "f16": _lib.F16, "bf16": _lib.BF16}
KIND_TO_TORCH = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16,
                 "u8": torch.uint8, "i8": torch.int8}


def _require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("locomp_b200 needs a CUDA device; there is no CPU fallback")


class DeviceTensor:
    """A device-resident array; same public surface as the reference's CUDATensor."""

    def __init__(self, storage: torch.Tensor, bf16_carrier: bool = False):
        if not storage.is_cuda:
            raise ValueError("DeviceTensor wraps CUDA memory only")
        self._t = storage.contiguous()
        self._freed = False
        # reference convention: bf16 values travel in a float16-typed array (examples/55_bfloat16_kernels.py:25-41)
        self.bf16_carrier = bool(bf16_carrier)

    @property
    def _cuda_ptr(self) -> int:
        if self._freed:
            raise RuntimeError("tensor was freed")
        return self._t.data_ptr()

    @property
    def size(self) -> int:
        return self._t.numel()

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(self._t.shape)

    @property
    def dtype(self) -> np.dtype:
        if self._t.dtype == torch.bfloat16:
            return np.dtype(np.float16)   # carrier dtype; see bf16_carrier
        return np.dtype(torch.empty(0, dtype=self._t.dtype).numpy().dtype)

    @property
    def kind(self) -> str:
        if self.bf16_carrier and self._t.dtype == torch.float16:
            return "bf16"
        return _TORCH_TO_KIND[self._t.dtype]

    def torch(self) -> torch.Tensor:
        """The backing torch tensor (zero copy)."""
        return self._t

    def numpy(self) -> np.ndarray:
        """Copy device memory to the host (CUDATensor.numpy, cuda_runtime.py:78-80)."""
        if self._freed:
            raise RuntimeError("tensor was freed")
        t = self._t
        if t.dtype == torch.bfloat16:
            t = t.view(torch.float16)
        return t.cpu().numpy()

    def free(self) -> None:
        if not self._freed:
            self._t = torch.empty(0, device=self._t.device, dtype=self._t.dtype)
            self._freed = True

    def __repr__(self) -> str:
        return f"DeviceTensor(shape={self.shape}, dtype={self.dtype})"


def tensor(data, dtype=np.float32, device: Optional[int] = None) -> DeviceTensor:
    """Upload a list / NumPy array (locomp.tensor, locomp/api.py:323-339).  As in the
    reference, an ndarray keeps its own dtype and `dtype` applies to other inputs."""
    _require_cuda()
    arr = data if isinstance(data, np.ndarray) else np.asarray(data, dtype=dtype)
    arr = np.ascontiguousarray(arr)
    if arr.dtype not in _NP_TO_TORCH:
        raise TypeError(f"unsupported dtype {arr.dtype}")
    dev = torch.device("cuda", torch.cuda.current_device() if device is None else device)
    return DeviceTensor(torch.from_numpy(arr).to(dev, non_blocking=False))


def empty(shape, dtype=np.float32, device: Optional[int] = None) -> DeviceTensor:
    """Uninitialised device tensor (locomp.empty, locomp/api.py:342-364)."""
    _require_cuda()
    if isinstance(shape, int):
        shape = (shape,)
    dev = torch.device("cuda", torch.cuda.current_device() if device is None else device)
    return DeviceTensor(torch.empty(tuple(shape), dtype=_NP_TO_TORCH[np.dtype(dtype)], device=dev))


def zeros(shape, dtype=np.float32, device: Optional[int] = None) -> DeviceTensor:
    """Zero-filled device tensor (locomp.zeros, locomp/api.py:367-389)."""
    t = empty(shape, dtype, device)
    t.torch().zero_()
    return t


class Operand:
    """One normalised operator argument.  A NumPy argument is uploaded lazily, on first use
    of `.ptr`, so that shape and dtype validation happens before the GPU is touched."""

    def __init__(self, ptr, kind, shape, size, device, keepalive, host=None):
        self._ptr = ptr
        self.kind = kind              # "f32" | "f16" | "bf16" | "u8" | "i8" | "i32"
        self.shape = tuple(shape)
        self.size = int(size)
        self.device = device
        self.keepalive = keepalive    # object that owns the memory for the duration of the call
        self.host = host              # set when the caller passed a NumPy array

    @property
    def ptr(self) -> int:
        if self._ptr is None:
            _require_cuda()
            src = np.ascontiguousarray(self.host)
            self.keepalive = torch.from_numpy(src).to(torch.device("cuda", self.device), non_blocking=True)
            self._ptr = self.keepalive.data_ptr()
        return self._ptr


def resolve(arg, name: str, bf16: bool = False) -> Operand:
    """Normalise one operator argument.  NumPy arrays are uploaded (and, if they are outputs,
    copied back by the caller); device objects are used in place."""
    if isinstance(arg, DeviceTensor):
        t = arg.torch()
        if arg._freed:
            raise ValueError(f"{name}: tensor was freed")
        return Operand(t.data_ptr(), "bf16" if (bf16 and t.dtype == torch.float16) else arg.kind,
                       tuple(t.shape), t.numel(), t.device.index, arg)
    if isinstance(arg, torch.Tensor):
        if not arg.is_cuda:
            raise TypeError(f"{name}: torch tensor must live on a CUDA device")
        if not arg.is_contiguous():
            raise ValueError(f"{name}: tensor must be contiguous")
        if arg.dtype not in _TORCH_TO_KIND:
            raise TypeError(f"{name}: unsupported dtype {arg.dtype}")
        kind = _TORCH_TO_KIND[arg.dtype]
        if bf16 and kind == "f16":
            kind = "bf16"
        return Operand(arg.data_ptr(), kind, tuple(arg.shape), arg.numel(), arg.device.index, arg)
    if isinstance(arg, np.ndarray):
        if arg.dtype not in _NP_TO_KIND:
            raise TypeError(f"{name}: unsupported dtype {arg.dtype}")
        kind = _NP_TO_KIND[arg.dtype]
        if bf16 and kind == "f16":
            kind = "bf16"
        dev = torch.cuda.current_device() if torch.cuda.is_available() else 0
        return Operand(None, kind, tuple(arg.shape), arg.size, dev, None, host=arg)
    if hasattr(arg, "_cuda_ptr") and hasattr(arg, "dtype") and hasattr(arg, "shape"):
        # the reference's own CUDATensor or a look-alike
        dt = np.dtype(arg.dtype)
        if dt not in _NP_TO_KIND:
            raise TypeError(f"{name}: unsupported dtype {dt}")
        kind = _NP_TO_KIND[dt]
        if bf16 and kind == "f16":
            kind = "bf16"
        shape = tuple(arg.shape)
        size = int(np.prod(shape)) if shape else 1
        dev = torch.cuda.current_device() if torch.cuda.is_available() else 0
        return Operand(int(arg._cuda_ptr), kind, shape, size, dev, arg)
    raise TypeError(f"Unsupported argument type for {name}: {type(arg)}")


def current_stream_ptr(stream=None) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    return int(stream)


_workspaces = {}


def workspace(nbytes: int, device: int, stream_ptr: int) -> torch.Tensor:
    """Zero-initialised scratch buffer, one per (device, stream); the kernels leave it zeroed."""
    key = (device, stream_ptr)
    buf = _workspaces.get(key)
    need = max(int(nbytes), 256)
    if buf is None or buf.numel() < need:
        if buf is not None:
            # work queued on the old buffer must finish before the allocator may reuse it
            torch.cuda.synchronize(device)
        buf = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=torch.device("cuda", device))
        torch.cuda.synchronize(device)   # zero-fill ran on torch's stream; the caller's may differ
        _workspaces[key] = buf
    return buf
