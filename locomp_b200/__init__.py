"""locomp_b200: B200-native weight-quantized matmul / dequantize operators.

A drop-in, for NVIDIA B200 (sm_100a), for the quantized operators of Zyora-Dev/locomp
(examples/38_quantized_matmul.py, examples/52_dequantize.py): same Python call surface,
same packed-weight and scale layout, hand-written CUDA kernels behind a C-ABI shared
library (include/locomp_b200.h).  There is no CPU fallback.
"""
from ._lib import LcqError
from .ops import (dequant_int4, dequant_int8, dequant_matvec_int4, dequant_matvec_int8, dequantize,
                  gpu_dequant_int4, gpu_dequant_int8, gpu_matvec_int4, gpu_matvec_int8, quantized_matmul)
from .decode_ops import (QuantizedWeight, add_inplace, add_inplace_kernel, argmax, embed_lookup, quantize, quantize_int4,
                         quantize_int4_ref, quantize_int8, residual_rms_norm, rms_norm, rms_norm_kernel, silu_mul,
                         silu_mul_kernel)
from .linear import DecodeStack, QuantLinear, fuse_rows
from .shard import PeerGather, ShardedQuantLinear, shard_rows
from .tensor import DeviceTensor, empty, tensor, zeros

__all__ = [
    "LcqError", "DeviceTensor", "tensor", "empty", "zeros",
    "gpu_matvec_int4", "gpu_matvec_int8", "gpu_dequant_int4", "gpu_dequant_int8",
    "dequant_matvec_int4", "dequant_matvec_int8", "dequant_int4", "dequant_int8",
    "quantized_matmul", "dequantize", "rms_norm", "residual_rms_norm", "silu_mul", "add_inplace", "embed_lookup", "argmax",
    "rms_norm_kernel", "silu_mul_kernel", "add_inplace_kernel", "quantize", "quantize_int4", "quantize_int8",
    "quantize_int4_ref", "QuantizedWeight", "ShardedQuantLinear", "PeerGather", "shard_rows", "QuantLinear", "fuse_rows", "DecodeStack",
]
__version__ = "0.1.0"
