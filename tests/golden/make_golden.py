"""Generate the golden fixtures in this folder from the reference's own NumPy functions.

Run in a container that has the reference tree (it cannot run on the GPU box):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

It imports examples/38_quantized_matmul.py and examples/52_dequantize.py from the
reference, reproduces the seeded cases of their own self-checks
(examples/52_dequantize.py:146-172 and examples/38_quantized_matmul.py:312-375, seed 42)
plus a few small ragged cases, and stores inputs and reference outputs as .npz.
Every array stored is an OUTPUT OF REFERENCE CODE run on seeded random inputs.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(ref_root: str, rel: str, name: str):
    sys.path.insert(0, ref_root)
    spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root: str) -> None:
    sys.dont_write_bytecode = True
    ex38 = _load(ref_root, "examples/38_quantized_matmul.py", "ref_ex38")
    ex52 = _load(ref_root, "examples/52_dequantize.py", "ref_ex52")
    out = {}

    # --- dequantize self-check cases of the reference (seed 42, one RNG stream, g=32)
    np.random.seed(42)
    for n, k in [(64, 256), (128, 512)]:
        w = np.random.randn(n, k).astype(np.float32) * 0.5
        packed, scales = ex52.quantize_int4_ref(w, 32)
        out[f"dq4_{n}x{k}_w"] = w
        out[f"dq4_{n}x{k}_packed"] = packed
        out[f"dq4_{n}x{k}_scales"] = scales
        out[f"dq4_{n}x{k}_expected"] = ex52.dequant_int4_ref(packed, scales, n, k, 32)

    # int8 dequantize, formula of examples/52_dequantize.py:162-166
    np.random.seed(43)
    for n, k in [(64, 256)]:
        w = np.random.randn(n, k).astype(np.float32) * 0.5
        absmax = np.abs(w.reshape(n, k // 32, 32)).max(axis=2)
        scales = (absmax / 127.0).astype(np.float32)
        w8 = np.clip(np.round(w / (np.repeat(scales, 32, axis=1) + 1e-10)), -128, 127).astype(np.int8)
        out[f"dq8_{n}x{k}_w8"] = w8
        out[f"dq8_{n}x{k}_scales"] = scales
        out[f"dq8_{n}x{k}_expected"] = w8.astype(np.float32) * np.repeat(scales, 32, axis=1)

    # --- matvec cases of the reference benchmark (seed 42 per shape), smallest shape,
    #     plus ragged shapes and other group sizes
    for tag, n, k, g in [("a", 256, 256, 32), ("b", 48, 192, 32), ("c", 40, 128, 64), ("d", 24, 96, 16)]:
        np.random.seed(42)
        wf = np.random.randn(n, k).astype(np.float32) * 0.1
        x = np.random.randn(k).astype(np.float32) * 0.1
        p4, s4 = ex38.quantize_int4(wf, g)
        w8, s8 = ex38.quantize_int8(wf, g)
        out[f"mv_{tag}_wf"] = wf
        out[f"mv_{tag}_x"] = x
        out[f"mv_{tag}_g"] = np.int64(g)
        out[f"mv_{tag}_p4"] = p4
        out[f"mv_{tag}_s4"] = s4
        out[f"mv_{tag}_w8"] = w8
        out[f"mv_{tag}_s8"] = s8
        out[f"mv_{tag}_fast4"] = ex38.fast_numpy_matvec_int4(x, p4, s4, g)
        out[f"mv_{tag}_fast8"] = ex38.fast_numpy_matvec_int8(x, w8, s8, g)
        if n * k <= 48 * 192:
            out[f"mv_{tag}_loop4"] = ex38.numpy_matvec_int4(x, p4, s4, g)
            out[f"mv_{tag}_loop8"] = ex38.numpy_matvec_int8(x, w8, s8, g)
        # the two packers of the reference must agree (they define the wire layout)
        p4b, s4b = ex52.quantize_int4_ref(wf, g)
        out[f"mv_{tag}_p4_ex52"] = p4b

    # --- config-1 shape (int8, per-channel scales = group_size K), default_rng(0) draws
    rng = np.random.default_rng(0)
    w8 = rng.integers(-127, 128, size=(1536, 576), dtype=np.int8)
    s = (np.abs(rng.standard_normal((1536, 1))) * 0.01).astype(np.float32)
    x = rng.standard_normal(576).astype(np.float32)
    out["cfg1_w8_sha"] = np.frombuffer(__import__("hashlib").sha256(w8.tobytes()).digest(), dtype=np.uint8)
    out["cfg1_scales"] = s
    out["cfg1_x"] = x
    out["cfg1_expected"] = ex38.fast_numpy_matvec_int8(x, w8, s, 576)

    # --- all 256 byte values x a handful of scales: the complete unpack table
    allb = np.arange(256, dtype=np.uint8).reshape(4, 64)   # N=4, K=128
    sc = np.array([[0.5, 0.015625, 1.0, 3.0]] * 4, dtype=np.float32)
    out["tbl_packed"] = allb
    out["tbl_scales"] = sc
    out["tbl_expected"] = ex52.dequant_int4_ref(allb, sc, 4, 128, 32)

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/reference")
    main(sys.argv[1])
