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
    glue_vectors(ref_root)


def glue_vectors(ref_root: str) -> None:
    """Second fixture file: the reference's NumPy forms of the decode-step operators next to the
    quantized linears (examples/29_rms_norm.py:60-63, examples/31_fused_silu.py:29-31,
    examples/34_fused_residual_norm.py:63-68) at the SmolLM2-135M widths, and the scales of the
    examples/52 packer.  Every output stored is an OUTPUT OF REFERENCE CODE on seeded inputs."""
    ex29 = _load(ref_root, "examples/29_rms_norm.py", "ref_ex29")
    ex31 = _load(ref_root, "examples/31_fused_silu.py", "ref_ex31")
    ex34 = _load(ref_root, "examples/34_fused_residual_norm.py", "ref_ex34")
    ex52 = _load(ref_root, "examples/52_dequantize.py", "ref_ex52_b")
    out = {}
    rng = np.random.default_rng(54)
    for rows, n in [(1, 576), (4, 576), (3, 1000)]:
        x = rng.standard_normal((rows, n)).astype(np.float32)
        w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        r = rng.standard_normal((rows, n)).astype(np.float32)
        tag = f"{rows}x{n}"
        out[f"norm_{tag}_x"], out[f"norm_{tag}_w"], out[f"norm_{tag}_r"] = x, w, r
        out[f"norm_{tag}_expected"] = ex29.rms_norm_np(x, w, eps=1e-5)
        h, normed = ex34.fused_residual_rms_norm_np(r, x, w, eps=1e-5)
        out[f"resnorm_{tag}_h"], out[f"resnorm_{tag}_expected"] = h, normed
    for n in (1536, 1000):
        g = (3.0 * rng.standard_normal(n)).astype(np.float32)
        u = rng.standard_normal(n).astype(np.float32)
        out[f"silu_{n}_gate"], out[f"silu_{n}_up"] = g, u
        out[f"silu_{n}_expected"] = ex31.silu_mul_np(g, u)
    np.random.seed(42)
    for tag, n, k, g in [("a", 256, 256, 32), ("d", 24, 96, 16)]:
        wf = np.random.randn(n, k).astype(np.float32) * 0.1
        if tag == "d":
            wf[3, 16:32] = 0.0                      # an all-zero group: the floor at 1e-10 decides its scale
            wf[5] *= 1e-4                           # small scales: the + 1e-10 in the divisor changes bits
        p, s = ex52.quantize_int4_ref(wf, g)
        out[f"q52_{tag}_wf"], out[f"q52_{tag}_g"], out[f"q52_{tag}_p"], out[f"q52_{tag}_s"] = wf, np.int64(g), p, s
    path = os.path.join(HERE, "glue_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/reference")
    main(sys.argv[1])
