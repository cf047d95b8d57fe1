"""The oracle's codecs against the reference's own known-answer tests.

Each test names the reference test it restates (paths inside the reference project).
"""
import numpy as np
import pytest


# ---- flare-loader/src/quantize.rs:886-960 (f16) -------------------------------------------
def test_f16_to_f32_known_values(orc):
    f = lambda b: float(orc.f16_to_f32(np.uint16(b))[0])
    assert abs(f(0x3C00) - 1.0) < 1e-6          # test_f16_to_f32
    assert f(0x0000) == 0.0
    assert abs(f(0xBC00) + 1.0) < 1e-6
    nz = orc.f16_to_f32(np.uint16(0x8000))[0]   # test_f16_to_f32_negative_zero
    assert nz == 0.0 and np.signbit(nz)
    assert np.isposinf(f(0x7C00))               # ..._positive_infinity
    assert np.isneginf(f(0xFC00))               # ..._negative_infinity
    assert np.isnan(f(0x7E00))                  # ..._nan
    sub = f(0x0001)                             # ..._subnormal
    assert 0.0 < sub < 1e-4
    assert abs(f(0x7BFF) - 65504.0) < 1.0       # ..._max_normal
    assert abs(f(0x4000) - 2.0) < 1e-6          # ..._two
    assert abs(f(0x3800) - 0.5) < 1e-6          # ..._half


def test_f16_to_f32_every_bit_pattern_matches_ieee(orc):
    bits = np.arange(65536, dtype=np.uint16)
    got = orc.f16_to_f32(bits)
    want = bits.view(np.float16).astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])
    assert np.all(np.isnan(got[nan]))
    # the reference keeps the NaN payload as mant << 13 (quantize.rs:524-527)
    mant = (bits[nan].astype(np.uint32) & 0x3FF) << 13
    assert np.array_equal(got.view(np.uint32)[nan] & 0x7FFFFF, mant)


# ---- flare-loader/src/quantize.rs:540-542, 962-995 (bf16) ----------------------------------
def test_bf16_to_f32(orc):
    L = orc.lib()
    assert abs(L.orc_bf16_to_f32(0x3F80) - 1.0) < 1e-6
    assert L.orc_bf16_to_f32(0x0000) == 0.0
    assert abs(L.orc_bf16_to_f32(0xBF80) + 1.0) < 1e-6
    assert abs(L.orc_bf16_to_f32(0x4000) - 2.0) < 1e-6
    assert np.isposinf(L.orc_bf16_to_f32(0x7F80))


# ---- f32 -> f16 RNE (half::f16::from_f32 as used at flare-gpu/src/kv_cache.rs:132) --------
def test_f32_to_f16_rne_matches_numpy(orc):
    rng = np.random.default_rng(7)
    xs = [rng.standard_normal(200000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 300.0, 7e4)]
    # every f16 value, the midpoints between neighbours and their f32 neighbours
    h = np.arange(0x7C00, dtype=np.uint16).view(np.float16).astype(np.float32)
    mids = ((h[:-1].astype(np.float64) + h[1:].astype(np.float64)) / 2).astype(np.float32)
    xs += [h, mids, np.nextafter(mids, np.float32(np.inf)), np.nextafter(mids, np.float32(-np.inf)),
           np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65519.9, 65520.0, 1e9, 5.96e-8, 2.98e-8, 2.99e-8],
                    dtype=np.float32)]
    x = np.concatenate(xs)
    x = np.concatenate([x, -x])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(orc.f32_to_f16(x), want)
    assert np.isnan(orc.f16_to_f32(orc.f32_to_f16(np.float32(np.nan)))[0])


def test_f32_to_bf16_rne(orc):
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(100000).astype(np.float32),
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, np.inf], dtype=np.float32)])
    got = orc.f32_to_bf16(x)
    u = x.view(np.uint32).astype(np.uint64)
    want = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    assert np.array_equal(got, want)


# ---- flare-loader/src/quantize.rs:1259-1353, 1694 (Q8_0 blocks) ---------------------------
def _q8_block(scale_bytes, qs):
    return bytes(scale_bytes) + bytes(qs)


def test_dequant_q8_0_short_block(orc):
    out = np.full(32, 55.0, dtype=np.float32)
    orc.dequant_q8_0_block(bytes([0x00, 0x3C, 0x01, 0x02]), out)
    assert np.all(np.abs(out - 55.0) < 1e-6)


def test_dequant_q8_0_zero_scale(orc):
    out = np.zeros(32, dtype=np.float32)
    orc.dequant_q8_0_block(_q8_block([0, 0], [0x7F] * 32), out)
    assert np.all(np.abs(out) < 1e-6)


def test_dequant_q8_0_positive_values(orc):
    out = np.zeros(32, dtype=np.float32)
    orc.dequant_q8_0_block(_q8_block([0x00, 0x3C], [42] + [0] * 31), out)
    assert abs(out[0] - 42.0) < 1e-4 and np.all(np.abs(out[1:]) < 1e-5)


def test_dequant_q8_0_negative_values(orc):
    out = np.zeros(32, dtype=np.float32)
    orc.dequant_q8_0_block(_q8_block([0x00, 0x3C], [0x80] + [0] * 31), out)
    assert abs(out[0] + 128.0) < 1e-4


def test_dequant_q8_0_mixed_signs(orc):
    out = np.zeros(32, dtype=np.float32)
    orc.dequant_q8_0_block(_q8_block([0x00, 0x3C], [0x01, 0xFF] + [0] * 30), out)
    assert abs(out[0] - 1.0) < 1e-4 and abs(out[1] + 1.0) < 1e-4


def test_dequant_q8_0_negative_scale(orc):
    out = np.zeros(32, dtype=np.float32)
    orc.dequant_q8_0_block(_q8_block([0x00, 0xC0], [0x02] + [0] * 31), out)
    assert abs(out[0] + 4.0) < 1e-4


def test_dequant_q8_0_ramp(orc):
    out = np.zeros(32, dtype=np.float32)
    orc.dequant_q8_0_block(_q8_block([0x00, 0x3C], list(range(32))), out)
    assert np.all(np.abs(out - np.arange(32)) < 1e-3)


# ---- flare-core/src/model.rs:5507-5527 (Q8_0 quantiser, x86_64 branch) --------------------
def test_quantize_q8_0_formula(orc):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((64, 64)).astype(np.float32)
    x[3, :32] = 0.0                      # a zero block: d = 0, id = 0
    x[5, 7] = 40.0
    blocks = orc.quantize_q8_0(x).reshape(64, 2, 34)
    xb = x.reshape(64, 2, 32)
    amax = np.abs(xb).max(axis=-1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        idv = np.where(d != 0, np.float32(127.0) / amax, np.float32(0)).astype(np.float32)
    prod = (xb * idv[..., None]).astype(np.float32)
    q = np.where(prod >= 0, np.floor(prod + np.float32(0.5)), np.ceil(prod - np.float32(0.5)))  # half away
    # (x*id) is at most 127 in magnitude, exactly representable +0.5 arithmetic in f32 is safe there
    assert np.array_equal(blocks[..., 2:].view(np.int8), q.astype(np.int8))
    assert np.array_equal(blocks[..., :2].copy().view(np.uint16)[..., 0], d.astype(np.float16).view(np.uint16))
    # dequantised block = i8 * f16 scale, one multiply (quantize.rs:188-197)
    deq = orc.dequant_q8_0(blocks.reshape(64, 68))
    want = blocks[..., 2:].view(np.int8).astype(np.float32) * d.astype(np.float16).astype(np.float32)[..., None]
    assert np.array_equal(deq.view(np.uint32), want.reshape(64, 64).view(np.uint32))
    assert np.max(np.abs(deq - x)) < 0.2


# ---- flare-core/src/kv_cache.rs:924-940 (test_pack_unpack_direct) -------------------------
def test_pack_unpack_direct(orc):
    values = np.array([0.0, 1.0, 2.0, 3.0, 0.5, 1.5, 2.5, 3.0], dtype=np.float32)
    packed, scale, mn = orc.q2_quantize_to_packed(values)
    assert packed.size == 2
    out = orc.q2_dequant_per_token(packed, scale, mn, 8)
    assert np.all(np.abs(values - out) <= 0.6)
    # range [0,3] -> scale 1, min 0; round() is half away from zero: 0.5->1, 1.5->2, 2.5->3
    assert scale == 1.0 and mn == 0.0
    codes = [(packed[i // 4] >> ((i % 4) * 2)) & 3 for i in range(8)]
    assert codes == [0, 1, 2, 3, 1, 2, 3, 3]


def test_q2_constant_vector_is_all_zero_codes(orc):
    packed, scale, mn = orc.q2_quantize_to_packed(np.full(8, 42.0, dtype=np.float32))
    assert scale == 0.0 and mn == 42.0 and not packed.any()
    assert np.all(orc.q2_dequant_per_token(packed, scale, mn, 8) == 42.0)


def test_q2_odd_length_packs_round_up(orc):
    packed, scale, mn = orc.q2_quantize_to_packed(np.array([0, 3, 1, 2, 3], dtype=np.float32))
    assert packed.size == 2 and packed[0] == (0 | 3 << 2 | 1 << 4 | 2 << 6) and packed[1] == 3


def test_q8_0_matvec_restatement(orc):
    """quantize_input_q8_0 + matvec_q8_0_preq_into (flare-core/src/model.rs:5507-5527, 8066-8100) on numbers that can
    be checked by hand: one block, weights 1..32 scaled by 0.5, input all ones -> quants 127, scale 1/127."""
    w = np.zeros(34, np.uint8)
    w[0:2] = [0x00, 0x38]                                  # f16 0.5
    w[2:] = np.arange(1, 33, dtype=np.int8).view(np.uint8)
    x = np.ones(32, np.float32)
    scales, quants = orc.quantize_input_q8_0(x)
    assert quants.tolist() == [127] * 32 and scales[0] == np.float32(1.0) / np.float32(127.0)
    got = orc.matvec_q8_0(w, x, 1)
    want = (np.float32(0.5) * scales[0]) * np.float32(127 * 528)           # sum 1..32 = 528
    assert got[0] == want and abs(got[0] - 264.0) < 1e-3
    # against a float64 evaluation of the same quantised operands on a random matrix
    rng = np.random.default_rng(3)
    rows, cols = 7, 256
    W = rng.standard_normal((rows, cols), dtype=np.float32)
    xb = rng.standard_normal(cols, dtype=np.float32)
    blocks = orc.quantize_q8_0(W)
    got = orc.matvec_q8_0(blocks, xb, rows)
    Wd = orc.dequant_q8_0(blocks).astype(np.float64)
    s, qv = orc.quantize_input_q8_0(xb)
    xd = (qv.reshape(-1, 32).astype(np.float64) * s[:, None].astype(np.float64)).reshape(-1)
    assert np.max(np.abs(got - Wd @ xd)) < 1e-4
    assert np.max(np.abs(got - W @ xb)) < 0.5            # and it is the product, up to the two quantisations
