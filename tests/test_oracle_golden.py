"""The NumPy oracle against vectors produced by the reference's own functions
(tests/golden/make_golden.py).  CPU only."""
import hashlib

import numpy as np
import pytest

from oracle import qmm_oracle as O


@pytest.mark.parametrize("shape", [(64, 256), (128, 512)])
def test_dequant_int4_bit_exact(golden, shape):
    n, k = shape
    got = O.dequant_int4(golden[f"dq4_{n}x{k}_packed"], golden[f"dq4_{n}x{k}_scales"], 32)
    exp = golden[f"dq4_{n}x{k}_expected"]
    assert got.dtype == np.float32 and got.shape == (n, k)
    assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))


def test_dequant_int8_bit_exact(golden):
    got = O.dequant_int8(golden["dq8_64x256_w8"], golden["dq8_64x256_scales"], 32)
    assert np.array_equal(got.view(np.uint32), golden["dq8_64x256_expected"].view(np.uint32))


def test_full_byte_table(golden):
    got = O.dequant_int4(golden["tbl_packed"], golden["tbl_scales"], 32)
    assert np.array_equal(got.view(np.uint32), golden["tbl_expected"].view(np.uint32))
    q = O.unpack_int4(golden["tbl_packed"])
    b = golden["tbl_packed"].astype(np.int32)
    assert np.array_equal(q[:, 0::2], b & 15) and np.array_equal(q[:, 1::2], b >> 4)
    assert np.array_equal(O.pack_int4(q), golden["tbl_packed"])


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_quantisers_match_reference(golden, tag):
    g = int(golden[f"mv_{tag}_g"])
    wf = golden[f"mv_{tag}_wf"]
    p4, s4 = O.quantize_int4(wf, g)
    assert np.array_equal(p4, golden[f"mv_{tag}_p4"])
    assert np.array_equal(s4.view(np.uint32), golden[f"mv_{tag}_s4"].view(np.uint32))
    # both packers of the reference define the same wire layout
    assert np.array_equal(golden[f"mv_{tag}_p4"], golden[f"mv_{tag}_p4_ex52"])
    w8, s8 = O.quantize_int8(wf, g)
    assert np.array_equal(w8, golden[f"mv_{tag}_w8"])
    assert np.array_equal(s8.view(np.uint32), golden[f"mv_{tag}_s8"].view(np.uint32))


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_matvec_matches_reference(golden, tag):
    g = int(golden[f"mv_{tag}_g"])
    x = golden[f"mv_{tag}_x"]
    for kind, w, s in (("4", golden[f"mv_{tag}_p4"], golden[f"mv_{tag}_s4"]),
                       ("8", golden[f"mv_{tag}_w8"], golden[f"mv_{tag}_s8"])):
        fn = O.matmul_int4 if kind == "4" else O.matmul_int8
        exact = fn(x, w, s, g, exact=True)
        fast = fn(x, w, s, g, exact=False)
        ref_fast = golden[f"mv_{tag}_fast{kind}"]
        # float32 BLAS order is unspecified: compare at float32 round-off of the sum
        np.testing.assert_allclose(fast, ref_fast, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(exact, ref_fast, rtol=1e-5, atol=1e-6)
        if f"mv_{tag}_loop{kind}" in golden:
            loop = O.loop_matvec_int4 if kind == "4" else O.loop_matvec_int8
            ref_loop = golden[f"mv_{tag}_loop{kind}"]
            np.testing.assert_allclose(exact.astype(np.float32), ref_loop, rtol=2e-6, atol=1e-7)
            if w.shape[0] * x.shape[0] <= 24 * 96:
                assert np.array_equal(loop(x, w, s, g), ref_loop)


def test_config1_int8_per_channel(golden):
    rng = np.random.default_rng(0)
    w8 = rng.integers(-127, 128, size=(1536, 576), dtype=np.int8)
    s = (np.abs(rng.standard_normal((1536, 1))) * 0.01).astype(np.float32)
    x = rng.standard_normal(576).astype(np.float32)
    sha = np.frombuffer(hashlib.sha256(w8.tobytes()).digest(), dtype=np.uint8)
    assert np.array_equal(sha, golden["cfg1_w8_sha"]), "seeded generator drifted"
    assert np.array_equal(s, golden["cfg1_scales"]) and np.array_equal(x, golden["cfg1_x"])
    got = O.matmul_int8(x, w8, s, 576)
    exp = golden["cfg1_expected"]
    # "1e-4 relative" is read against the output scale: the reference's own float32 BLAS
    # sum carries round-off of ~1e-7 * sum|x*w|, which exceeds 1e-4 * |y| where y cancels to ~0.
    np.testing.assert_allclose(got, exp, rtol=1e-4, atol=1e-4 * float(np.sqrt(np.mean(exp ** 2))))


def test_round_to_bf16_is_rne():
    import torch
    v = np.random.default_rng(1).standard_normal(4096).astype(np.float32) * 3
    exp = torch.from_numpy(v).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(O.round_to(v, "bf16"), exp)
    assert np.array_equal(O.round_to(v, "f16"), v.astype(np.float16))


def test_ragged_and_empty():
    rng = np.random.default_rng(3)
    wp, s = O.make_w4(rng, 5, 64, 32)
    assert O.dequant_int4(wp, s, 32).shape == (5, 64)
    assert O.dequant_int4(wp[:0], s[:0], 32).shape == (0, 64)
    assert O.matmul_int4(np.zeros((0, 64), np.float16), wp, s).shape == (0, 5)
    with pytest.raises(ValueError):
        O.dequant_int4(wp, s, 48)
    with pytest.raises(ValueError):
        O.dequant_int4(wp.astype(np.int8), s, 32)


# --------------------------------------------------------------------------- decode-step operators
@pytest.fixture(scope="module")
def glue():
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    return dict(np.load(os.path.join(here, "golden", "glue_vectors.npz")))


@pytest.mark.parametrize("tag", ["1x576", "4x576", "3x1000"])
def test_decode_oracle_norms_match_reference_numpy_forms(glue, tag):
    from oracle import decode_oracle as D
    x, w, r = glue[f"norm_{tag}_x"], glue[f"norm_{tag}_w"], glue[f"norm_{tag}_r"]
    np.testing.assert_allclose(D.rms_norm(x, w, 1e-5), glue[f"norm_{tag}_expected"], rtol=2e-6, atol=1e-7)
    h, normed = D.residual_rms_norm(r, x, w, 1e-5)
    assert np.array_equal(h, glue[f"resnorm_{tag}_h"])                 # one float32 addition: exact
    np.testing.assert_allclose(normed, glue[f"resnorm_{tag}_expected"], rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("n", [1536, 1000])
def test_decode_oracle_silu_matches_reference_numpy_form(glue, n):
    from oracle import decode_oracle as D
    np.testing.assert_allclose(D.silu_mul(glue[f"silu_{n}_gate"], glue[f"silu_{n}_up"]), glue[f"silu_{n}_expected"],
                               rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("tag", ["a", "d"])
def test_ex52_quantiser_oracle_bit_exact(glue, tag):
    from oracle import decode_oracle as D
    p, s = D.quantize_int4_ex52(glue[f"q52_{tag}_wf"], int(glue[f"q52_{tag}_g"]))
    assert np.array_equal(p, glue[f"q52_{tag}_p"])
    assert np.array_equal(s.view(np.uint32), glue[f"q52_{tag}_s"].view(np.uint32))
