"""The committed fixtures of tests/golden (made by tests/golden/make_golden.py): the CPU restatement must
still reproduce them bit for bit, and the CUDA path must match them — bit for bit for codecs and cache
planes, within the attention tolerance for attention outputs."""
import os

import numpy as np
import pytest

from util import assert_bits_equal, assert_close

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v1.npz")
DEC_SHAPES = [(2, 2, 2, 1), (2, 2, 2, 6), (4, 2, 4, 10), (32, 8, 64, 20), (8, 4, 64, 1), (1, 1, 3, 5),
              (8, 2, 64, 300), (4, 1, 128, 200)]


@pytest.fixture(scope="module")
def g():
    return np.load(GOLDEN)


# ------------------------------------------------------------------ CPU: the restatement has not drifted
def test_generator_reproduces_the_fixtures(g):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(os.path.dirname(GOLDEN), "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.DEC_SHAPES == DEC_SHAPES
    fresh = mod.build()
    assert sorted(fresh) == sorted(g.files)
    for name in g.files:
        assert_bits_equal(fresh[name], g[name], name)


def test_fixture_sanity(g):
    # a few facts that do not depend on any implementation
    back = g["f16_back"]
    x = g["f16_in"]
    finite = np.isfinite(x) & (np.abs(x) < 65504)
    assert np.all(np.abs(back[finite] - x[finite]) <= np.maximum(np.abs(x[finite]) * 2.0 ** -11, 2.0 ** -25))
    assert g["q8_blocks"].size == 64 * 34
    assert np.all(g["q8_dequant"][32:64] == 0.0)
    for i, (nh, nkv, hd, sl) in enumerate(DEC_SHAPES):
        v = g[f"dec_{i}_v"].reshape(sl, nkv, hd)
        out = g[f"dec_{i}_out"].reshape(nh, hd)
        for h in range(nh):        # a convex combination of the value rows
            col = v[:, h // (nh // nkv), :]
            assert np.all(out[h] <= col.max(axis=0) + 1e-5) and np.all(out[h] >= col.min(axis=0) - 1e-5)


# ------------------------------------------------------------------ GPU: the CUDA path against the fixtures
@pytest.fixture(scope="module")
def fb():
    import flarellm_b200 as fb
    return fb


@pytest.fixture(scope="module")
def eng(fb):
    e = fb.Engine(0)
    yield e
    e.close()


@pytest.mark.gpu
@pytest.mark.parametrize("i", range(len(DEC_SHAPES)))
def test_gpu_decode_matches_fixture(fb, eng, g, i):
    nh, nkv, hd, sl = DEC_SHAPES[i]
    be = fb.CudaBackend(0)
    got = be.grouped_query_attention(g[f"dec_{i}_q"], g[f"dec_{i}_k"], g[f"dec_{i}_v"], nh, nkv, hd, sl)
    assert_close(got, g[f"dec_{i}_out"], f"decode fixture {DEC_SHAPES[i]}")
    # and through the device-resident f32 ring
    kv = eng.kv_alloc(1, 1, max(32, sl), nkv, hd, fb.KV_F32)
    kv.append(0, 0, g[f"dec_{i}_k"], g[f"dec_{i}_v"])
    kv.advance(0, sl - 1)                                  # the newest token is "this step's" row
    got = eng.decode(kv, 0, nh, g[f"dec_{i}_q"].reshape(1, 1, nh, hd))
    assert_close(got, g[f"dec_{i}_out"], f"decode fixture {DEC_SHAPES[i]} (device ring)")
    kv.free()


@pytest.mark.gpu
def test_gpu_q8_cache_matches_fixture(fb, eng, g):
    """A Q8_0 cache row is the block stream of the fixture, byte for byte, and dequantises to the same values."""
    x = g["q8_in"].reshape(8, 256)                         # 8 tokens of 4 kv heads x 64
    kv = eng.kv_alloc(1, 1, 32, 4, 64, fb.KV_Q8_0)
    kv.append(0, 0, x, x)
    kv.advance(0, 8)
    blocks = kv.export_q8_0_blocks(0, 0, 0, 8)
    assert_bits_equal(blocks[0], g["q8_blocks"], "Q8_0 key blocks")
    assert_bits_equal(blocks[1], g["q8_blocks"], "Q8_0 value blocks")
    dk, dv = kv.export_dequant(0, 0)
    assert_bits_equal(dk[:8].reshape(-1), g["q8_dequant"], "Q8_0 dequantised keys")
    kv.free()


@pytest.mark.gpu
def test_gpu_prefill_matches_fixture(fb, eng, g):
    S, nh, nkv, hd = 70, 2, 1, 64
    for key, window in (("pre_out", 0), ("pre_out_w16", 16)):
        got = eng.prefill(g["pre_q"], g["pre_k"], g["pre_v"], 1, S, nh, nkv, hd, window=window)
        assert_close(got, g[key], f"prefill fixture window {window}")


@pytest.mark.gpu
def test_gpu_kivi_ref_cache_matches_fixture(fb, eng, g):
    nkv, hd, ms, n = 2, 32, 128, 70
    kv = eng.kv_alloc(1, 1, ms, nkv, hd, fb.KV_KIVI_REF)
    k, v = g["kivi_ref_k"], g["kivi_ref_v"]
    for t in range(n):
        kv.write(0, 0, t, k[t], v[t])
        kv.advance(0, 1)
    names = {"key_packed": "PLANE_K_Q", "value_packed": "PLANE_V_Q", "key_scales": "PLANE_K_SCALE", "key_mins": "PLANE_K_MIN",
             "value_scales": "PLANE_V_SCALE", "value_mins": "PLANE_V_MIN", "residual_keys": "PLANE_K_RES",
             "residual_values": "PLANE_V_RES"}
    for oname, pname in names.items():
        assert_bits_equal(kv.export_plane(0, 0, getattr(fb, pname)), g[f"kivi_ref_plane_{oname}"], oname)
    dk, dv = kv.export_dequant(0, 0)
    assert_bits_equal(dk.reshape(-1), g["kivi_ref_dk"], "KIVI key view")
    assert_bits_equal(dv.reshape(-1), g["kivi_ref_dv"], "KIVI value view")
    kv.free()


@pytest.mark.gpu
def test_gpu_g32_cache_matches_fixture(fb, eng, g):
    kvd, ms, n = 64, 256, 200
    kv = eng.kv_alloc(1, 1, ms, 1, kvd, fb.KV_KIVI_G32)
    k, v = g["g32_k"], g["g32_v"]
    kv.append(0, 0, k[:150], v[:150]); kv.advance(0, 150)
    for t in range(150, n):
        kv.write(0, 0, t, k[t], v[t]); kv.advance(0, 1)
    names = {"k_codes": "PLANE_K_Q", "k_meta": "PLANE_K_SCALE", "v_codes": "PLANE_V_Q", "v_meta": "PLANE_V_SCALE",
             "res_k": "PLANE_K_RES", "res_v": "PLANE_V_RES"}
    for oname, pname in names.items():
        assert_bits_equal(kv.export_plane(0, 0, getattr(fb, pname)), g[f"g32_plane_{oname}"], oname)
    dk, dv = kv.export_dequant(0, 0)
    assert_bits_equal(dk, g["g32_dk"], "group-32 key view")
    assert_bits_equal(dv, g["g32_dv"], "group-32 value view")
    kv.free()
