"""The oracle's attention and caches against the reference's own tests (restated)."""
import numpy as np
import pytest

# flare-core/src/model.rs:10427-10435
REF_SHAPES = [(2, 2, 2, 1), (2, 2, 2, 6), (4, 2, 4, 10), (32, 8, 64, 20), (8, 4, 64, 1), (1, 1, 3, 5)]


def ref_inputs(nh, nkv, hd, sl):
    """Closed-form inputs of test_fused_attention_matches_reference (model.rs:10438-10447):
    the index is turned into f32 first, then scaled, then sin/cos in f32."""
    i = np.arange(nh * hd, dtype=np.int64)
    q = np.sin(((i * 7 + 3).astype(np.float32) * np.float32(0.1)).astype(np.float32)).astype(np.float32)
    j = np.arange(sl * nkv * hd, dtype=np.int64)
    k = np.cos(((j * 11 + 5).astype(np.float32) * np.float32(0.05)).astype(np.float32)).astype(np.float32)
    v = np.sin(((j * 13 + 7).astype(np.float32) * np.float32(0.08)).astype(np.float32)).astype(np.float32)
    return q, k, v


def attention_f64(q, k, v, nh, nkv, hd, sl):
    q = q.astype(np.float64).reshape(nh, hd)
    k = k.astype(np.float64).reshape(-1, nkv, hd)[:sl]
    v = v.astype(np.float64).reshape(-1, nkv, hd)[:sl]
    out = np.zeros((nh, hd))
    for h in range(nh):
        g = h // (nh // nkv)
        s = k[:, g] @ q[h] / np.sqrt(np.float64(hd))
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ v[:, g]
    return out.reshape(-1)


@pytest.mark.parametrize("nh,nkv,hd,sl", REF_SHAPES)
def test_fused_attention_matches_reference(orc, nh, nkv, hd, sl):
    """model.rs:10369-10463: online softmax vs the in-test 3-pass routine, tol max(|ref|*1e-4, 1e-5)."""
    q, k, v = ref_inputs(nh, nkv, hd, sl)
    ref = orc.gqa_decode_three_pass(q, k, v, nh, nkv, hd, sl)
    fused = orc.gqa_decode(q, k, v, nh, nkv, hd, sl)
    tol = np.maximum(np.abs(ref) * 1e-4, 1e-5)
    assert np.all(np.abs(ref - fused) <= tol)
    # and both against float64
    f64 = attention_f64(q, k, v, nh, nkv, hd, sl)
    assert np.max(np.abs(fused - f64)) < 2e-6


def test_gqa_heads_per_kv_group(orc):
    """model.rs:10766-10829: 4 q heads / 2 kv heads; q heads 0,1 use kv head 0 and 2,3 kv head 1."""
    nh, nkv, hd, sl = 4, 2, 8, 5
    rng = np.random.default_rng(0)
    q = rng.standard_normal(nh * hd).astype(np.float32)
    k = rng.standard_normal(sl * nkv * hd).astype(np.float32)
    v = rng.standard_normal(sl * nkv * hd).astype(np.float32)
    out = orc.gqa_decode(q, k, v, nh, nkv, hd, sl)
    assert np.all(np.isfinite(out))
    # swap kv-head contents: heads 0,1 <-> 2,3 must swap when q is swapped alike
    k2 = k.reshape(sl, nkv, hd)[:, ::-1].copy()
    v2 = v.reshape(sl, nkv, hd)[:, ::-1].copy()
    q2 = q.reshape(nh, hd)[[2, 3, 0, 1]].copy()
    out2 = orc.gqa_decode(q2, k2, v2, nh, nkv, hd, sl).reshape(nh, hd)
    assert np.array_equal(out2[[2, 3, 0, 1]].reshape(-1), out)


def test_softcap_path(orc):
    """model.rs:10119-10212: tanh cap then 3-pass softmax, weights < 1e-8 skipped."""
    nh, nkv, hd, sl = 4, 2, 16, 33
    rng = np.random.default_rng(1)
    q = (rng.standard_normal(nh * hd) * 3).astype(np.float32)
    k = rng.standard_normal(sl * nkv * hd).astype(np.float32)
    v = rng.standard_normal(sl * nkv * hd).astype(np.float32)
    cap = 5.0
    out = orc.gqa_decode(q, k, v, nh, nkv, hd, sl, softcap=cap)
    qq, kk, vv = q.astype(np.float64).reshape(nh, hd), k.astype(np.float64).reshape(sl, nkv, hd), v.astype(np.float64).reshape(sl, nkv, hd)
    want = np.zeros((nh, hd))
    for h in range(nh):
        s = kk[:, h // 2] @ qq[h] / 4.0
        s = np.tanh(s / cap) * cap
        p = np.exp(s - s.max()); p /= p.sum()
        p[p < 1e-8] = 0
        want[h] = p @ vv[:, h // 2]
    assert np.max(np.abs(out - want.reshape(-1))) < 1e-5


def test_seq_len_zero_gives_zeros(orc):
    out = orc.gqa_decode(np.ones(8, np.float32), np.ones(8, np.float32), np.ones(8, np.float32), 2, 2, 4, 0)
    assert np.all(out == 0.0)


def test_prefill_equals_token_by_token(orc):
    """generate.rs:657-698 contract (batched prefill == sequential) and the wgpu-vs-CPU recipe of
    flare-gpu/src/backend.rs:6165-6212 (seq 4, 2 heads, hd 8)."""
    for (S, nh, nkv, hd) in [(4, 2, 2, 8), (9, 4, 2, 16), (1, 2, 1, 4)]:
        rng = np.random.default_rng(S)
        q = rng.standard_normal((S, nh * hd)).astype(np.float32)
        k = rng.standard_normal((S, nkv * hd)).astype(np.float32)
        v = rng.standard_normal((S, nkv * hd)).astype(np.float32)
        out = orc.prefill(q, k, v, S, nh, nkv, hd)
        for t in range(S):
            want = orc.gqa_decode(q[t], k[: t + 1], v[: t + 1], nh, nkv, hd, t + 1)
            assert np.array_equal(out[t], want)
        mt = orc.prefill(q, k, v, S, nh, nkv, hd, threads=4)
        assert np.array_equal(mt, out)


def test_prefill_window_and_row_subset(orc):
    S, nh, nkv, hd, W = 40, 4, 2, 8, 7
    rng = np.random.default_rng(5)
    q = rng.standard_normal((S, nh * hd)).astype(np.float32)
    k = rng.standard_normal((S, nkv * hd)).astype(np.float32)
    v = rng.standard_normal((S, nkv * hd)).astype(np.float32)
    out = orc.prefill(q, k, v, S, nh, nkv, hd, window=W, row_start=3, row_step=5)
    for t in range(S):
        if t >= 3 and (t - 3) % 5 == 0:
            lo = max(0, t - W + 1)
            assert np.array_equal(out[t], orc.gqa_decode(q[t], k[lo: t + 1], v[lo: t + 1], nh, nkv, hd, t + 1 - lo))
        else:
            assert np.all(np.isnan(out[t]))


def test_batched_verify_is_sequential_decode(orc):
    """generate.rs:258-303: verify of n drafts == n sequential decodes, query i sees L+i+1 slots."""
    B, n_q, nh, nkv, hd, slots = 3, 6, 8, 2, 16, 50
    rng = np.random.default_rng(9)
    q = rng.standard_normal((B, n_q, nh * hd)).astype(np.float32)
    k = rng.standard_normal((B, slots, nkv * hd)).astype(np.float32)
    v = rng.standard_normal((B, slots, nkv * hd)).astype(np.float32)
    attend = np.array([50, 31, 6], dtype=np.int32)
    out = orc.gqa_decode_batched(q, k, v, attend, nh, nkv, hd, n_q=n_q, threads=3)
    for b in range(B):
        for i in range(n_q):
            n = attend[b] - (n_q - 1 - i)
            assert np.array_equal(out[b, i], orc.gqa_decode(q[b, i], k[b], v[b], nh, nkv, hd, n))
    one = orc.gqa_decode_heads_mt(q[:, -1], k, v, attend, nh, nkv, hd, threads=4)
    assert np.array_equal(one, out[:, -1])


def test_partial_merge_equals_full(orc):
    nh, nkv, hd, sl = 8, 2, 32, 300
    rng = np.random.default_rng(2)
    q = rng.standard_normal(nh * hd).astype(np.float32)
    k = rng.standard_normal(sl * nkv * hd).astype(np.float32)
    v = rng.standard_normal(sl * nkv * hd).astype(np.float32)
    full = orc.gqa_decode(q, k, v, nh, nkv, hd, sl)
    cuts = [0, 1, 77, 77, 200, 300]   # includes an empty range
    parts = np.stack([orc.gqa_decode_partial(q, k, v, nh, nkv, hd, a, b) for a, b in zip(cuts[:-1], cuts[1:])])
    merged = orc.merge_partials(parts, nh, hd)
    assert np.max(np.abs(merged - full)) < 2e-6
    one = orc.merge_partials(orc.gqa_decode_partial(q, k, v, nh, nkv, hd, 0, sl)[None], nh, hd)
    assert np.max(np.abs(one - full)) < 1e-6


# ---------------------------------------------------------------- KvCache (kv_cache.rs:552-779)
def test_kv_cache_basic(orc):
    c = orc.KvCache(2, 4, 2, 4)
    assert c.len() == 0 and c.is_empty()
    c.write(0, np.full(8, 1.0), np.full(8, 2.0)); c.write(1, np.full(8, 1.0), np.full(8, 2.0)); c.advance()
    assert c.len() == 1 and c.position() == 1


def test_kv_cache_ring_buffer_and_wraparound_integrity(orc):
    c = orc.KvCache(1, 4, 1, 2)
    for i in range(6):
        c.write(0, np.full(2, i * 10.0), np.full(2, i * 100.0)); c.advance()
    assert c.len() == 4 and c.position() == 2
    k = c.keys(0)
    assert abs(k[0] - 40.0) < 1e-5 and abs(k[2] - 50.0) < 1e-5
    assert abs(c.values(0)[0] - 400.0) < 1e-5


def test_kv_cache_many_wraps_capacity_and_clear(orc):
    c = orc.KvCache(1, 4, 1, 1)
    for i in range(100):
        c.write(0, [float(i)], [0.0]); c.advance()
    assert c.position() == 0 and c.len() == 4
    c = orc.KvCache(1, 6, 1, 1)
    for i in range(6):
        c.write(0, [float(i)], [0.0]); c.advance()
    assert c.len() == 6 and c.position() == 0          # test_position_at_capacity
    c = orc.KvCache(1, 4, 1, 2)
    c.write(0, [99.0, 99.0], [99.0, 99.0]); c.advance(); c.clear()
    assert c.len() == 0 and c.position() == 0 and np.all(c.keys(0) == 0)
    c.write(0, [1.0, 2.0], [3.0, 4.0]); c.advance()
    assert c.len() == 1 and abs(c.keys(0)[0] - 1.0) < 1e-5   # test_clear_and_reuse


def test_kv_cache_multi_layer_minimal_and_dims(orc):
    c = orc.KvCache(2, 4, 1, 2)
    c.write(0, [1.0, 2.0], [10.0, 20.0]); c.write(1, [3.0, 4.0], [30.0, 40.0]); c.advance()
    assert c.keys(0)[0] == 1.0 and c.keys(1)[0] == 3.0 and c.values(0)[0] == 10.0 and c.values(1)[0] == 30.0
    c = orc.KvCache(1, 1, 1, 1)                          # test_minimal_cache_size_one
    c.write(0, [1.0], [10.0]); c.advance()
    assert c.len() == 1 and c.keys(0)[0] == 1.0
    c.write(0, [2.0], [20.0]); c.advance()
    assert c.len() == 1 and c.keys(0)[0] == 2.0
    c = orc.KvCache(1, 8, 1, 1)                          # test_head_dim_one
    for i in range(8):
        c.write(0, [float(i)], [i * 2.0]); c.advance()
    assert np.array_equal(c.keys(0), np.arange(8, dtype=np.float32))
    hd, nkv = 256, 4                                     # test_large_head_dim
    c = orc.KvCache(1, 2, nkv, hd)
    c.write(0, np.arange(nkv * hd, dtype=np.float32), np.full(nkv * hd, 0.5)); c.advance()
    assert c.keys(0)[0] == 0.0 and c.keys(0)[nkv * hd - 1] == nkv * hd - 1


def test_kv_truncate_only_before_wrap(orc):
    c = orc.KvCache(1, 4, 1, 1)
    for i in range(3):
        c.write(0, [float(i)], [0.0]); c.advance()
    c.truncate_to(1)
    assert c.len() == 1 and c.position() == 1
    for i in range(5):
        c.write(0, [float(i)], [0.0]); c.advance()
    assert c.len() == 4
    c.truncate_to(2)                                     # wrapped: ignored (kv_cache.rs:527-530)
    assert c.len() == 4


def test_attend_len_clamps_once_full(orc):
    c = orc.KvCache(1, 4, 1, 1)
    want = [1, 2, 3, 4, 4, 4]
    for i in range(6):
        c.write(0, [float(i)], [0.0])
        assert c.attend_len() == want[i]
        c.advance()


# ---------------------------------------------------------------- QuantizedKvCache (kv_cache.rs:781-921)
def test_quantized_basic_write_read(orc):
    c = orc.QuantizedKvCache(1, 64, 1, 4)
    key, val = [0.0, 1.0, 2.0, 3.0], [10.0, 20.0, 30.0, 40.0]
    c.write(0, key, val); c.advance()
    assert c.len() == 1 and c.position() == 1
    assert np.all(np.abs(c.dequant_keys(0)[:4] - key) < 1e-5)
    assert np.all(np.abs(c.dequant_values(0)[:4] - val) < 1e-5)


def test_quantized_packing_round_trip(orc):
    c = orc.QuantizedKvCache(1, 128, 1, 4)
    for t in range(32 + 10):
        c.write(0, [t, t + 0.5, t + 1.0, t + 1.5], [t * 10.0] * 4); c.advance()
    assert abs(c.dequant_values(0)[0] - 0.0) < 1.0


def test_quantized_clear_wrap_multilayer(orc):
    c = orc.QuantizedKvCache(1, 64, 1, 4)
    c.write(0, [1.0] * 4, [2.0] * 4); c.advance(); c.clear()
    assert c.len() == 0 and c.position() == 0 and c.is_empty()
    c = orc.QuantizedKvCache(1, 8, 1, 2)
    for i in range(12):
        c.write(0, [float(i)] * 2, [float(i)] * 2); c.advance()
    assert c.len() == 8 and c.position() == 12 % 8
    c = orc.QuantizedKvCache(2, 64, 1, 4)
    c.write(0, [1.0, 2.0, 3.0, 4.0], [10.0] * 4); c.write(1, [5.0, 6.0, 7.0, 8.0], [20.0] * 4); c.advance()
    assert abs(c.dequant_keys(0)[0] - 1.0) < 1e-5 and abs(c.dequant_keys(1)[0] - 5.0) < 1e-5


def test_quantized_value_accuracy_and_constant_no_nan(orc):
    c = orc.QuantizedKvCache(1, 64, 1, 4)
    val = [0.0, 1.0, 2.0, 3.0]
    c.write(0, [0.0] * 4, val); c.advance()
    assert np.all(np.abs(c.dequant_values(0)[:4] - val) < 1e-5)
    c = orc.QuantizedKvCache(1, 64, 1, 4)
    c.write(0, [42.0] * 4, [42.0] * 4); c.advance()
    for t in range(1, 34):
        c.write(0, [float(t)] * 4, [float(t)] * 4); c.advance()
    dv = c.dequant_values(0)
    assert not np.isnan(dv[0]) and dv[0] == 42.0     # scale 0 -> code 0 -> min


def test_quantized_quirks_are_reproduced(orc):
    """The behaviours listed for the reference's KIVI decode step: (b) during the step the
    current token's slot is not yet dequantised (zeros); (c) once length >= 32 the current
    token has overwritten the residual slot of logical token length-32."""
    kv = 8
    c = orc.QuantizedKvCache(1, 64, 2, 4)
    rng = np.random.default_rng(0)
    rows = rng.standard_normal((40, kv)).astype(np.float32)
    for t in range(36):
        c.write(0, rows[t], rows[t] * 2); c.advance()
    c.write(0, rows[36], rows[36] * 2)                 # the decode step: write, no advance yet
    dk = c.dequant_keys(0).reshape(64, kv)
    assert np.all(dk[36] == 0.0)                       # quirk (b)
    assert np.array_equal(dk[4], rows[36])             # quirk (c): logical token 36-32 reads the new token
    assert np.array_equal(dk[5], rows[5])
    # quirk (a): tokens outside the window decode with running per-channel stats
    mins, scales = rows[0].copy(), np.zeros(kv, np.float32)
    L = orc.lib()
    import ctypes as C
    for t in range(1, 37):
        L.orc_q2_update_per_channel_stats(rows[t].ctypes.data_as(C.POINTER(C.c_float)),
                                          mins.ctypes.data_as(C.POINTER(C.c_float)),
                                          scales.ctypes.data_as(C.POINTER(C.c_float)), kv, 0)
    packed, _, _ = orc.q2_quantize_to_packed(rows[2])
    assert np.array_equal(dk[2], orc.q2_dequant_per_channel(packed, mins, scales))


# ---------------------------------------------------------------- group-32 KIVI cache
def test_g32_cache_matches_direct_quantisation(orc):
    kv, ms = 64, 256
    rng = np.random.default_rng(4)
    n = 256 + 96 + 5      # wraps
    rows_k = rng.standard_normal((n, kv)).astype(np.float32)
    rows_v = rng.standard_normal((n, kv)).astype(np.float32)
    rows_k[:, 3] *= 8
    c = orc.G32Cache(ms, kv)
    for t in range(n):
        c.write_advance(rows_k[t], rows_v[t])
    assert c.attend_len() == ms
    k, v = c.dequant()
    k16 = orc.f16_to_f32(orc.f32_to_f16(rows_k))
    v16 = orc.f16_to_f32(orc.f32_to_f16(rows_v))
    last = n - 1
    for tok in range(n - ms, n):
        s = tok % ms
        if last - tok < 128:
            assert np.array_equal(k[s], k16[tok]) and np.array_equal(v[s], v16[tok])
        else:
            g0 = tok // 32 * 32
            col = k16[g0:g0 + 32]
            for ch in (0, 3, 63):
                packed, sc, mn = orc.q2_quantize_to_packed(col[:, ch])
                sc16 = orc.f16_to_f32(orc.f32_to_f16(sc))[0]
                mn16 = orc.f16_to_f32(orc.f32_to_f16(mn))[0]
                want = orc.q2_dequant_per_token(packed, sc16, mn16, 32)[tok - g0]
                assert k[s, ch] == want
            for g in range(kv // 32):
                packed, sc, mn = orc.q2_quantize_to_packed(v16[tok, g * 32:(g + 1) * 32])
                sc16 = orc.f16_to_f32(orc.f32_to_f16(sc))[0]
                mn16 = orc.f16_to_f32(orc.f32_to_f16(mn))[0]
                assert np.array_equal(v[s, g * 32:(g + 1) * 32], orc.q2_dequant_per_token(packed, sc16, mn16, 32))
    # error bound of 2-bit quantisation: half a step of the group range
    assert np.max(np.abs(v - v16[[(n - ms) + ((s - (n - ms)) % ms) for s in range(ms)]])) < 1.2


def test_g32_short_context_is_all_residual(orc):
    kv = 32
    c = orc.G32Cache(256, kv)
    rng = np.random.default_rng(8)
    rows = rng.standard_normal((100, kv)).astype(np.float32)
    for r in rows:
        c.write_advance(r, -r)
    k, v = c.dequant()
    r16 = orc.f16_to_f32(orc.f32_to_f16(rows))
    assert np.array_equal(k[:100], r16) and np.array_equal(v[:100], -r16)
    assert not k[100:].any()


# ------------------------------------------------------------------ rotary position embedding
def test_rope_reference_properties(orc):
    """flare-core/src/model.rs:10354-10364, 10934-11028 restated: magnitude is preserved, position 0 is the
    identity, the table path equals the inline path (bit for bit here: the same expression per entry), positions
    beyond the table fall back to the inline computation, the table is capped."""
    d = orc.apply_rope([1.0, 0.0, 0.0, 1.0], 1, 4, 5, 10000.0)
    assert abs(float(np.sum(d * d)) - 2.0) < 1e-4
    orig = np.arange(1, 9, dtype=np.float32)
    assert np.max(np.abs(orc.apply_rope(orig, 2, 4, 0, 10000.0) - orig)) < 1e-6
    cos, sin = orc.rope_table(8, 128, 10000.0)
    for pos in (0, 1, 5, 42, 127):
        orig = (np.arange(1, 25, dtype=np.float32) * np.float32(0.3))
        a = orc.apply_rope(orig, 3, 8, pos, 10000.0)
        b = orc.apply_rope_with_table(orig, 3, 8, pos, 10000.0, cos, sin)
        assert np.max(np.abs(a - b)) < 1e-6 and np.array_equal(a, b)
    cos16, sin16 = orc.rope_table(4, 16, 10000.0)
    orig = np.array([1, 2, 3, 4], np.float32)
    assert np.array_equal(orc.apply_rope(orig, 1, 4, 20, 10000.0), orc.apply_rope_with_table(orig, 1, 4, 20, 10000.0, cos16, sin16))
    capped, _ = orc.rope_table(4, 1_000_000, 10000.0)
    assert capped.shape[0] <= orc.ROPE_TABLE_MAX_SEQ_LEN
    cos64, sin64 = orc.rope_table(4, 64, 10000.0)
    d = orc.apply_rope_with_table([1.0, 0.0, 0.0, 1.0], 1, 4, 5, 10000.0, cos64, sin64)
    assert abs(float(np.sum(d * d)) - 2.0) < 1e-4
    # the half-split pairing and the sign convention, on numbers that can be checked by hand:
    # head_dim 2, position 1, theta anything: angle = 1 -> (x0 cos 1 - x1 sin 1, x0 sin 1 + x1 cos 1)
    d = orc.apply_rope([1.0, 2.0], 1, 2, 1, 10000.0)
    c, s = np.float32(np.cos(np.float32(1.0))), np.float32(np.sin(np.float32(1.0)))
    assert abs(d[0] - (c - 2 * s)) < 1e-6 and abs(d[1] - (s + 2 * c)) < 1e-6
