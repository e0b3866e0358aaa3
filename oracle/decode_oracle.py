"""CPU oracle for the decode-step operators next to the quantized linears.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module.

It restates, in NumPy, the arithmetic of these reference functions:

* rms_norm           kernel examples/54_smollm2_inference.py:40-73; NumPy form
                     rms_norm_np, examples/29_rms_norm.py:60-63
* silu_mul           kernel examples/54_smollm2_inference.py:113-120; NumPy form
                     silu_mul_np, examples/31_fused_silu.py:29-31
* add_inplace        kernel examples/54_smollm2_inference.py:164-167
* residual_rms_norm  NumPy form fused_residual_rms_norm_np, examples/34_fused_residual_norm.py:63-68
* embed_lookup       kernels locomp/_builtin_kernels.py:8-25 (out[i] = table[ids[i]])
* argmax             np.argmax on the logits, examples/54_smollm2_inference.py:606
* quantize_int4_ex52 examples/52_dequantize.py:110-126

Parity status: pinned.  tests/golden/make_golden.py imports the reference's NumPy functions
named above and stores their outputs on seeded inputs in tests/golden/glue_vectors.npz;
tests/test_oracle_golden.py compares this module with them.  embed_lookup, add_inplace and
argmax are exact operations (a copy, one float32 addition, np.argmax itself).
"""
from __future__ import annotations

import numpy as np

from .qmm_oracle import pack_int4


def rms_norm(x, w, eps: float = 1e-5) -> np.ndarray:
    """x * (1 / sqrt(mean(x^2, last axis) + eps)) * w, in float64; cast by the caller."""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    mean_sq = np.mean(x ** 2, axis=-1, keepdims=True)
    return x * (1.0 / np.sqrt(mean_sq + eps)) * w


def silu_mul(gate, up) -> np.ndarray:
    """gate * sigmoid(gate) * up, in float64."""
    g = np.asarray(gate, dtype=np.float64)
    return g * (1.0 / (1.0 + np.exp(-g))) * np.asarray(up, dtype=np.float64)


def add(a, b, dtype=np.float32) -> np.ndarray:
    """a + b with one rounding in the storage type (what the in-place add stores)."""
    return (np.asarray(a, dtype=np.float64) + np.asarray(b, dtype=np.float64)).astype(dtype)


def residual_rms_norm(residual, hidden, w, eps: float = 1e-5, dtype=np.float32):
    """(h, rms_norm(h) * w) with h = residual + hidden rounded to the storage type first."""
    h = add(residual, hidden, dtype)
    return h, rms_norm(h, w, eps)


def embed_lookup(token_ids, table) -> np.ndarray:
    return np.asarray(table)[np.asarray(token_ids, dtype=np.int64)]


def argmax(x) -> np.ndarray:
    return np.argmax(np.asarray(x), axis=-1).astype(np.int32)


def quantize_int4_ex52(w, group_size: int = 32):
    """The packer of examples/52_dequantize.py:110-126: amax floored at 1e-10, scale = amax / 7,
    q = clip(round(w / (scale + 1e-10)) + 8, 0, 15), all in float32."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    g = w.reshape(n, k // group_size, group_size)
    absmax = np.maximum(np.abs(g).max(axis=2, keepdims=True), np.float32(1e-10)).astype(np.float32)
    scales = (absmax.reshape(n, k // group_size) / np.float32(7.0)).astype(np.float32)
    q = np.round(g / (scales.reshape(n, -1, 1) + np.float32(1e-10))) + 8
    q = np.clip(q, 0, 15).astype(np.uint8).reshape(n, k)
    return pack_int4(q), scales
