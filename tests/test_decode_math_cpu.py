"""NumPy model of the arithmetic the W4A16 decode kernel performs, checked against the oracle on
CPU.  It pins the three tricks the kernel relies on:

  1. a nibble q in bits 0-3 of a 16-bit lane is the fp16 subnormal q * 2^-24 (bits 4-7: q * 2^-20),
     so masking a packed word yields tensor-core operands without any conversion;
  2. the activations are paired to those operands as (e0,e4)(e1,e5)(e2,e6)(e3,e7) per 8-block with
     the odd-nibble slots pre-divided by 16;
  3. the zero point is a separate contraction  -8 * sum_g scale[n,g] * xsum[g,m]  with -8*xsum*2^-9
     split into an fp16 high part and an fp16 residual.
"""
import numpy as np

from oracle import qmm_oracle as O


def _masked_operands(w_packed):
    """[N, K/2] uint8 -> fp16 values [N, K] exactly as the kernel's four masks produce them."""
    words = np.ascontiguousarray(w_packed).view(np.uint32)            # 8 nibbles per word
    n, nw = words.shape
    vals = np.empty((n, nw, 8), dtype=np.float64)
    for shift, mask, (ea, eb) in ((0, 0x000F000F, (0, 4)), (0, 0x00F000F0, (1, 5)),
                                  (8, 0x000F000F, (2, 6)), (8, 0x00F000F0, (3, 7))):
        m = (words >> shift) & mask
        lo = (m & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float64)
        hi = (m >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
        vals[:, :, ea], vals[:, :, eb] = lo, hi
    return vals.reshape(n, nw * 8)


def test_masked_words_are_scaled_nibbles():
    rng = np.random.default_rng(0)
    wp, _ = O.make_w4(rng, 16, 256)
    a = _masked_operands(wp)
    q = O.unpack_int4(wp).astype(np.float64)
    k = np.arange(256)
    odd = (k % 2) == 1                     # odd k = high nibble of its byte = bits 4-7 of a 16-bit lane
    assert np.array_equal(a[:, ~odd], q[:, ~odd] * 2.0 ** -24)
    assert np.array_equal(a[:, odd], q[:, odd] * 2.0 ** -20)


def test_decode_arithmetic_matches_oracle():
    rng = np.random.default_rng(1)
    n, k, m = 64, 1024, 5
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    x = rng.standard_normal((m, k)).astype(np.float16)
    a = _masked_operands(wp)                                           # [N, K] subnormal-scaled nibbles
    odd = (np.arange(k) % 2) == 1
    xb = x.astype(np.float64)
    xb[:, odd] = (x[:, odd].astype(np.float32) * np.float32(0.0625)).astype(np.float16).astype(np.float64)
    # per 32-group: D = sum x*a (float32 accumulate in the MMA), acc += scale * D
    d = np.einsum("ngk,mgk->mng", a.reshape(n, k // 32, 32), xb.reshape(m, k // 32, 32)).astype(np.float32)
    acc = np.einsum("mng,ng->mn", d.astype(np.float64), s.astype(np.float64))
    # zero point: -8*xsum*2^-9 as fp16 hi + lo, contracted with the fp16 scales
    xsum = x.astype(np.float32).reshape(m, k // 32, 32).sum(axis=2)
    zp = np.float32(-0.015625) * xsum
    hi = zp.astype(np.float16)
    lo = (zp - hi.astype(np.float32)).astype(np.float16)
    cor = np.einsum("ng,mg->mn", s.astype(np.float64), hi.astype(np.float64) + lo.astype(np.float64))
    y = acc * 2.0 ** 24 + cor * 512.0
    ref = O.matmul_int4(x.astype(np.float32), wp, s, 32)
    np.testing.assert_allclose(y, ref, rtol=2e-5, atol=2e-5 * float(np.sqrt(np.mean(ref ** 2))))


def test_zero_point_split_survives_large_activations():
    """|x| up to the fp16 maximum: -8*xsum*2^-9 stays finite in fp16 and the hi+lo pair keeps ~21 bits."""
    xsum = np.float32(32 * 65504.0)
    zp = np.float32(-0.015625) * xsum
    hi = np.float16(zp)
    lo = np.float16(zp - np.float32(hi))
    assert np.isfinite(hi) and np.isfinite(lo)
    assert abs((float(hi) + float(lo)) - float(zp)) <= abs(float(zp)) * 2.0 ** -20
