"""GPU parity for the two 2-bit caches: the reference's QuantizedKvCache bit for bit, and the
group-32 mode."""
import numpy as np
import pytest

from util import assert_bits_equal, assert_close, normal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fb():
    import flarellm_b200 as fb
    return fb


@pytest.fixture(scope="module")
def eng(fb):
    e = fb.Engine(0)
    yield e
    e.close()


REF_PLANES = [("key_packed", "PLANE_K_Q"), ("value_packed", "PLANE_V_Q"), ("key_scales", "PLANE_K_SCALE"),
              ("key_mins", "PLANE_K_MIN"), ("value_scales", "PLANE_V_SCALE"), ("value_mins", "PLANE_V_MIN"),
              ("residual_keys", "PLANE_K_RES"), ("residual_values", "PLANE_V_RES")]


def _compare_ref_planes(fb, kv, oc, layer, what):
    for oname, pname in REF_PLANES:
        got = kv.export_plane(layer, 0, getattr(fb, pname))
        assert_bits_equal(got, oc.plane(oname, layer), f"{what}: {oname}")


@pytest.mark.parametrize("ms,n_tokens", [(64, 50), (64, 64 + 37), (16, 40)])
def test_kivi_ref_cache_is_bit_exact_and_decodes_with_quirks(eng, fb, orc, ms, n_tokens):
    """Token-by-token decode steps against flare-core's QuantizedKvCache
    (flare-core/src/kv_cache.rs:121-250) and the call order of model.rs:2186-2247:
    write -> attend over len+1 slots of the dequantised view -> advance."""
    nh, nkv, hd, layers = 8, 2, 64, 2
    kv = eng.kv_alloc(layers, 1, ms, nkv, hd, fb.KV_KIVI_REF)
    oc = orc.QuantizedKvCache(layers, ms, nkv, hd)
    k = normal(61, (n_tokens, layers, nkv * hd))
    v = normal(62, (n_tokens, layers, nkv * hd))
    k[:, :, 5] *= 8
    q = normal(63, (n_tokens, 1, 1, nh, hd), 0.4)
    for t in range(n_tokens):
        for layer in range(layers):
            kv.write(layer, 0, t, k[t, layer], v[t, layer])
            oc.write(layer, k[t, layer], v[t, layer])
        if t % 7 == 0 or t >= n_tokens - 3:
            for layer in range(layers):
                _compare_ref_planes(fb, kv, oc, layer, f"t={t} layer={layer}")
                dk, dv = kv.export_dequant(layer, 0)
                assert_bits_equal(dk.reshape(-1), oc.dequant_keys(layer), f"dequant_keys t={t}")
                assert_bits_equal(dv.reshape(-1), oc.dequant_values(layer), f"dequant_values t={t}")
                seq_len = min(oc.len() + 1, ms)
                got = eng.decode(kv, layer, nh, q[t])
                want = orc.gqa_decode(q[t], oc.dequant_keys(layer), oc.dequant_values(layer), nh, nkv, hd, seq_len)
                assert_close(got, want, f"KIVI ref decode t={t} layer={layer}")
        kv.advance(); oc.advance()
        assert kv.state(0) == (oc.position(), oc.len())
    kv.free()


def test_kivi_ref_bulk_append_equals_sequential(eng, fb, orc):
    nh, nkv, hd, ms, n = 8, 2, 64, 128, 100
    kv = eng.kv_alloc(1, 1, ms, nkv, hd, fb.KV_KIVI_REF)
    oc = orc.QuantizedKvCache(1, ms, nkv, hd)
    k, v = normal(71, (n, nkv * hd)), normal(72, (n, nkv * hd))
    kv.append(0, 0, k[:60], v[:60]); kv.advance(0, 60)
    kv.append(0, 0, k[60:], v[60:]); kv.advance(0, n - 60)
    for t in range(n):
        oc.write(0, k[t], v[t]); oc.advance()
    _compare_ref_planes(fb, kv, oc, 0, "bulk")
    kv.free()


def test_kivi_ref_constant_rows_and_clear(eng, fb, orc):
    """kv_cache.rs:902-921: a constant vector has range 0, scale 0, all codes 0, and decodes to the constant."""
    kv = eng.kv_alloc(1, 1, 64, 1, 64, fb.KV_KIVI_REF)
    oc = orc.QuantizedKvCache(1, 64, 1, 64)
    for t in range(35):
        row = np.full(64, 42.0 if t == 0 else float(t), np.float32)
        kv.write(0, 0, t, row, row); kv.advance()
        oc.write(0, row, row); oc.advance()
    dk, dv = kv.export_dequant(0, 0)
    assert dv[0, 0] == 42.0 and not np.isnan(dv).any()
    assert_bits_equal(dv.reshape(-1), oc.dequant_values(0), "constant rows")
    kv.clear()
    assert kv.state(0) == (0, 0)
    for _, pname in REF_PLANES:
        assert not kv.export_plane(0, 0, getattr(fb, pname)).any()
    kv.free()


# ------------------------------------------------------------------ group-32 mode
G32_PLANES = [("k_codes", "PLANE_K_Q"), ("k_meta", "PLANE_K_SCALE"), ("v_codes", "PLANE_V_Q"),
              ("v_meta", "PLANE_V_SCALE"), ("res_k", "PLANE_K_RES"), ("res_v", "PLANE_V_RES")]


def _g32_oracle(orc, ms, kvd, k, v):
    oc = orc.G32Cache(ms, kvd)
    for t in range(k.shape[0]):
        oc.write_advance(k[t], v[t])
    return oc


def _g32_inputs(seed, n, kvd):
    k, v = normal(seed, (n, kvd)), normal(seed + 1, (n, kvd))
    rng = np.random.default_rng(seed + 2)
    outl = rng.choice(kvd, size=max(1, kvd // 100 + 1), replace=False)   # ~1 % outlier key channels, x8
    k[:, outl] *= 8
    return k, v


@pytest.mark.parametrize("ms,n,chunks", [(512, 300, [300]), (512, 450, [1] * 140 + [33, 200, 77]),
                                         (256, 256 + 200, [129, 127, 100, 100])])
def test_g32_planes_and_view_are_bit_exact(eng, fb, orc, ms, n, chunks):
    nkv, hd = 2, 64
    kvd = nkv * hd
    assert sum(chunks) == n
    k, v = _g32_inputs(81, n, kvd)
    kv = eng.kv_alloc(1, 1, ms, nkv, hd, fb.KV_KIVI_G32)
    t = 0
    for c in chunks:
        if c == 1:
            kv.write(0, 0, t, k[t], v[t])
        else:
            kv.append(0, 0, k[t:t + c], v[t:t + c])
        kv.advance(0, c)
        t += c
    oc = _g32_oracle(orc, ms, kvd, k, v)
    # ring rows: all 128; codes / meta: only groups that have been quantised and are still live
    for oname, pname in G32_PLANES[4:]:
        assert_bits_equal(kv.export_plane(0, 0, getattr(fb, pname)), oc.plane(oname), oname)
    dk, dv = kv.export_dequant(0, 0)
    ok, ov = oc.dequant()
    assert_bits_equal(dk, ok, "g32 key view")
    assert_bits_equal(dv, ov, "g32 value view")
    if n <= ms:      # before the wrap every quantised group is final: planes are byte-identical
        for oname, pname in G32_PLANES[:4]:
            assert_bits_equal(kv.export_plane(0, 0, getattr(fb, pname)), oc.plane(oname), oname)
    kv.free()


def test_g32_decode_step(eng, fb, orc):
    """Decode steps (write, attend over min(len+1, max), advance) at 32 q / 8 kv heads, head_dim 64."""
    nh, nkv, hd, ms, B = 32, 8, 64, 1024, 2
    kvd = nkv * hd
    n0 = 700
    kv = eng.kv_alloc(1, B, ms, nkv, hd, fb.KV_KIVI_G32)
    ks, vs = [], []
    for b in range(B):
        k, v = _g32_inputs(91 + 10 * b, n0 + 40, kvd)
        ks.append(k); vs.append(v)
        kv.append(0, b, k[:n0], v[:n0]); kv.advance(b, n0)
    for step in range(40):
        t = n0 + step
        q = normal(200 + step, (B, 1, nh, hd), 0.4)
        for b in range(B):
            kv.write(0, b, t, ks[b][t], vs[b][t])
        got = eng.decode(kv, 0, nh, q)
        if step % 13 == 0 or step == 39:
            for b in range(B):
                oc = _g32_oracle(orc, ms, kvd, ks[b][:t + 1], vs[b][:t + 1])
                ok, ov = oc.dequant()
                want = orc.gqa_decode(q[b], ok, ov, nh, nkv, hd, oc.attend_len())
                assert_close(got[b], want, f"g32 step {step} seq {b}")
        kv.advance()
    kv.free()


@pytest.mark.parametrize("nh,nkv,layers,B,n0", [(32, 8, 2, 2, 1500), (8, 4, 1, 3, 1100), (8, 8, 1, 1, 2000), (4, 2, 3, 2, 1333), (4, 1, 1, 2, 1200)])
def test_g32_long_context_decode_takes_the_tensor_core_path(eng, fb, orc, nh, nkv, layers, B, n0):
    """From 1024 attended tokens on, equal-length batches at head_dim 64 run the code-tile kernel for the
    quantised prefix plus the general kernel for the newest tokens; results must still match the CPU."""
    hd, ms = 64, 2048
    kvd = nkv * hd
    layer = layers - 1
    kv = eng.kv_alloc(layers, B, ms, nkv, hd, fb.KV_KIVI_G32)
    ks, vs = [], []
    for b in range(B):
        k, v = _g32_inputs(17 + 10 * b + nh, n0 + 36, kvd)
        ks.append(k); vs.append(v)
        kv.append(layer, b, k[:n0], v[:n0]); kv.advance(b, n0)
    for step in range(36):
        t = n0 + step
        q = normal(300 + step, (B, 1, nh, hd), 0.4)
        for b in range(B):
            kv.write(layer, b, t, ks[b][t], vs[b][t])
        got = eng.decode(kv, layer, nh, q)
        if step % 7 == 0 or step == 35:
            for b in range(B):
                oc = _g32_oracle(orc, ms, kvd, ks[b][:t + 1], vs[b][:t + 1])
                ok, ov = oc.dequant()
                want = orc.gqa_decode(q[b], ok, ov, nh, nkv, hd, oc.attend_len())
                assert_close(got[b], want, f"g32 long step {step} seq {b}")
        kv.advance()
    kv.free()


@pytest.mark.parametrize("extra", [[5, 63], [64, 127], [128, 200], [2048 + 1000, 31]])
def test_g32_wrapped_ring_stays_on_the_tensor_core_path(eng, fb, orc, extra):
    """A ring of 2048 slots that has wrapped (2048 + extra tokens written): the 128 ring tokens then sit in two or
    three tiles somewhere in the middle of the physical slots, possibly across the end of the ring, with the oldest
    2-bit tokens right behind them.  The call must still be served by the code-tile kernel and match the CPU; the
    second batch entry has another phase of the ring, and a third one has not wrapped at all."""
    nh, nkv, hd, ms = 32, 8, 64, 2048
    kvd = nkv * hd
    totals = [ms + extra[0], ms + extra[1], 1500]
    B = len(totals)
    kv = eng.kv_alloc(1, B, ms, nkv, hd, fb.KV_KIVI_G32)
    ks, vs = [], []
    for b, n in enumerate(totals):
        k, v = _g32_inputs(400 + 10 * b + extra[0], n + 3, kvd)
        ks.append(k); vs.append(v)
        done = 0
        while done < n:                        # in pieces, as prefill then decode steps would arrive
            c = min(777, n - done)
            kv.append(0, b, k[done:done + c], v[done:done + c]); kv.advance(b, c)
            done += c
    for step in range(3):
        q = normal(500 + step, (B, 1, nh, hd), 0.4)
        for b, n in enumerate(totals):
            kv.write(0, b, n + step, ks[b][n + step], vs[b][n + step])
        got = eng.decode(kv, 0, nh, q)
        assert eng.last_path() == fb.PATH_KIVI_TENSOR
        for b, n in enumerate(totals):
            oc = _g32_oracle(orc, ms, kvd, ks[b][:n + step + 1], vs[b][:n + step + 1])
            ok, ov = oc.dequant()
            want = orc.gqa_decode(q[b], ok, ov, nh, nkv, hd, oc.attend_len())
            assert_close(got[b], want, f"wrapped ring, extra {extra}, step {step}, seq {b}")
        kv.advance()
    kv.free()


def test_g32_ragged_batch_long_context(eng, fb, orc):
    """Sequences of different lengths (long, short, shorter than the residual ring) in one call."""
    nh, nkv, hd, ms, B = 8, 2, 64, 2048, 3
    kvd = nkv * hd
    lens = [1700, 300, 77]
    kv = eng.kv_alloc(1, B, ms, nkv, hd, fb.KV_KIVI_G32)
    q = normal(77, (B, 1, nh, hd), 0.4)
    for b in range(B):
        k, v = _g32_inputs(5 + b, lens[b] + 1, kvd)
        kv.append(0, b, k[:lens[b]], v[:lens[b]]); kv.advance(b, lens[b])
        kv.write(0, b, lens[b], k[lens[b]], v[lens[b]])
    got = eng.decode(kv, 0, nh, q)
    for b in range(B):
        k, v = _g32_inputs(5 + b, lens[b] + 1, kvd)
        oc = _g32_oracle(orc, ms, kvd, k, v)
        ok, ov = oc.dequant()
        assert_close(got[b], orc.gqa_decode(q[b], ok, ov, nh, nkv, hd, oc.attend_len()), f"ragged seq {b}")
    kv.free()


def test_g32_rollback_is_refused_after_eviction(eng, fb):
    kv = eng.kv_alloc(1, 1, 256, 1, 64, fb.KV_KIVI_G32)
    rows = normal(5, (200, 64))
    kv.append(0, 0, rows[:100], rows[:100]); kv.advance(0, 100)
    kv.truncate(0, 90)
    assert kv.state(0) == (90, 90)
    kv.append(0, 0, rows[:110], rows[:110]); kv.advance(0, 110)
    with pytest.raises(fb.FlareError) as e:
        kv.truncate(0, 150)
    assert e.value.status == fb.ERR_UNSUPPORTED
    kv.free()
