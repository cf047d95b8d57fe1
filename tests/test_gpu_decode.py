"""GPU parity: decode attention through the C ABI against the CPU oracle."""
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


# ------------------------------------------------------------------ the reference's own recipe
REF_SHAPES = [(2, 2, 2, 1), (2, 2, 2, 6), (4, 2, 4, 10), (32, 8, 64, 20), (8, 4, 64, 1), (1, 1, 3, 5)]


@pytest.mark.parametrize("nh,nkv,hd,sl", REF_SHAPES)
def test_reference_shapes_host_buffers(fb, orc, nh, nkv, hd, sl):
    """flare-core/src/model.rs:10427-10462 through ComputeBackend::grouped_query_attention."""
    from test_oracle_attention import ref_inputs
    q, k, v = ref_inputs(nh, nkv, hd, sl)
    be = fb.CudaBackend(0)
    got = be.grouped_query_attention(q, k, v, nh, nkv, hd, sl)
    want = orc.gqa_decode(q, k, v, nh, nkv, hd, sl)
    assert_close(got, want, f"ref shape {(nh, nkv, hd, sl)}")
    # the reference's own (tighter) tolerance holds as well
    assert np.all(np.abs(got - want) <= np.maximum(np.abs(want) * 1e-4, 1e-5) * 4)
    assert be.name() == "cuda"


def test_config1_smollm_shape_through_trait_hooks(fb, orc):
    """9 q / 3 kv heads, head_dim 64, 512 cached + 1 new token, seed 0, f32 cache."""
    nh, nkv, hd, L = 9, 3, 64, 512
    rng = np.random.default_rng(0)
    q = (rng.standard_normal(nh * hd, dtype=np.float32) * np.float32(0.125))
    k = (rng.standard_normal((L + 1, nkv * hd), dtype=np.float32) * np.float32(0.125))
    v = (rng.standard_normal((L + 1, nkv * hd), dtype=np.float32) * np.float32(0.125))
    be = fb.CudaBackend(0)
    assert not be.has_gpu_kv_cache()
    with pytest.raises(fb.FlareError) as e:
        be.grouped_query_attention_from_gpu_cache(q, 0, nh, nkv, hd, 1)
    assert e.value.status == fb.ERR_STATE
    be.init_gpu_kv_cache(2, 1024, nkv, hd)
    assert be.has_gpu_kv_cache()
    oc = orc.KvCache(2, 1024, nkv, hd)
    for t in range(L):
        for layer in range(2):
            be.gpu_kv_write(layer, t, nkv, hd, k[t] * (layer + 1), v[t])
            oc.write(layer, k[t] * (layer + 1), v[t])
        be.advance_kv(); oc.advance()
    for layer in range(2):
        be.gpu_kv_write(layer, L, nkv, hd, k[L] * (layer + 1), v[L])
        oc.write(layer, k[L] * (layer + 1), v[L])
    seq_len = oc.len() + 1
    assert seq_len == 513
    for layer in range(2):
        got = be.grouped_query_attention_from_gpu_cache(q, layer, nh, nkv, hd, seq_len)
        want = orc.gqa_decode(q, oc.keys(layer), oc.values(layer), nh, nkv, hd, seq_len)
        assert_close(got, want, f"config 1 layer {layer}")


def test_softcap_is_refused(fb):
    be = fb.CudaBackend(0)
    be.init_gpu_kv_cache(1, 8, 1, 64)
    with pytest.raises(fb.FlareError) as e:
        be.grouped_query_attention_from_gpu_cache(np.zeros(64, np.float32), 0, 1, 1, 64, 1, attn_softcap=30.0)
    assert e.value.status == fb.ERR_UNSUPPORTED


# ------------------------------------------------------------------ f32 cache, batch / ragged / wrap
@pytest.mark.parametrize("hd,nh,nkv", [(64, 8, 2), (128, 8, 8), (32, 6, 2), (256, 2, 1), (64, 16, 2), (64, 9, 3)])
def test_f32_batched_ragged(eng, fb, orc, hd, nh, nkv):
    B, ms = 3, 700
    kv = eng.kv_alloc(1, B, ms, nkv, hd, fb.KV_F32)
    k = normal(1, (B, ms, nkv * hd))
    v = normal(2, (B, ms, nkv * hd))
    q = normal(3, (B, 1, nh, hd), 0.3)
    for b in range(B):
        kv.append(0, b, k[b], v[b])
    attend = np.array([700, 1, 333], dtype=np.int32)
    got = eng.decode(kv, 0, nh, q, attend_len=attend)
    want = orc.gqa_decode_batched(q.reshape(B, 1, -1), k, v, attend, nh, nkv, hd)
    assert_close(got, want, "f32 ragged")
    # attend_len 0 -> zeros (cpu_grouped_query_attention_into leaves zeros)
    got0 = eng.decode(kv, 0, nh, q, attend_len=np.zeros(B, np.int32))
    assert not got0.any()
    kv.free()


def test_ring_wrap_f32_matches_oracle_cache(eng, fb, orc):
    """Ring of 64 slots, 64+20 tokens: position/length and slot contents follow KvCache
    (flare-core/src/kv_cache.rs:599-631); the full ring is attended once wrapped."""
    nh, nkv, hd, ms, n = 8, 2, 64, 64, 84
    kv = eng.kv_alloc(1, 1, ms, nkv, hd, fb.KV_F32)
    oc = orc.KvCache(1, ms, nkv, hd)
    k, v = normal(5, (n + 1, nkv * hd)), normal(6, (n + 1, nkv * hd))
    q = normal(7, (1, 1, nh, hd), 0.3)
    for t in range(n):
        kv.write(0, 0, t, k[t], v[t]); kv.advance()
        oc.write(0, k[t], v[t]); oc.advance()
        assert kv.state(0) == (oc.position(), oc.len())
    kv.write(0, 0, n, k[n], v[n]); oc.write(0, k[n], v[n])
    dk, dv = kv.export_dequant(0, 0)
    assert_bits_equal(dk.reshape(-1), oc.keys(0), "ring keys")
    assert_bits_equal(dv.reshape(-1), oc.values(0), "ring values")
    got = eng.decode(kv, 0, nh, q)            # attend_len from the ring state: min(len + 1, max)
    want = orc.gqa_decode(q, oc.keys(0), oc.values(0), nh, nkv, hd, oc.attend_len())
    assert oc.attend_len() == ms
    assert_close(got, want, "wrapped ring")
    kv.free()


def test_truncate_clear_and_state(eng, fb):
    kv = eng.kv_alloc(1, 2, 8, 1, 64, fb.KV_F32)
    row = np.ones(64, np.float32)
    for t in range(5):
        kv.write(0, 0, t, row * t, row); kv.advance(0)
    assert kv.state(0) == (5, 5) and kv.state(1) == (0, 0)
    kv.truncate(0, 3)
    assert kv.state(0) == (3, 3)
    for t in range(3, 12):
        kv.write(0, 0, t, row * t, row); kv.advance(0)
    assert kv.state(0) == (12 % 8, 8)
    kv.truncate(0, 2)                           # wrapped: ignored (kv_cache.rs:527-530)
    assert kv.state(0) == (4, 8)
    kv.clear()
    assert kv.state(0) == (0, 0)
    assert not kv.export_plane(0, 0, fb.PLANE_K, np.float32).any()
    kv.set_state(1, 3, 7)
    assert kv.state(1) == (3, 7)
    with pytest.raises(fb.FlareError):
        kv.set_state(1, 8, 0)
    kv.free()


# ------------------------------------------------------------------ Q8_0 cache (config 2 shape)
def _q8_setup(eng, fb, orc, B, ms, n_rows, nkv, hd, seed):
    kv = eng.kv_alloc(1, B, ms, nkv, hd, fb.KV_Q8_0)
    k = normal(seed, (B, n_rows, nkv * hd))
    v = normal(seed + 1, (B, n_rows, nkv * hd))
    for b in range(B):
        kv.append(0, b, k[b], v[b])
        kv.advance(b, n_rows)
    return kv, k, v


def test_q8_device_quantiser_is_bit_exact(eng, fb, orc):
    """On-device Q8_0 quantisation == flare-core/src/model.rs:5507-5527 + f16 RNE scale, and the
    dequantised view == flare-loader/src/quantize.rs:188-197, byte for byte."""
    nkv, hd, ms = 8, 64, 256
    kv, k, v = _q8_setup(eng, fb, orc, 2, ms, ms, nkv, hd, 11)
    k[1, 5, :32] = 0.0       # zero block (d == 0)
    k[1, 6, 7] = 1e4
    kv.clear(1); kv.append(0, 1, k[1], v[1]); kv.advance(1, ms)
    for b in range(2):
        kb, vb = kv.export_q8_0_blocks(0, b, 0, ms)
        assert_bits_equal(kb, orc.quantize_q8_0(k[b]), "K blocks")
        assert_bits_equal(vb, orc.quantize_q8_0(v[b]), "V blocks")
        dk, dv = kv.export_dequant(0, b)
        assert_bits_equal(dk, orc.dequant_q8_0(orc.quantize_q8_0(k[b])), "K dequant")
        assert_bits_equal(dv, orc.dequant_q8_0(orc.quantize_q8_0(v[b])), "V dequant")
    # block-stream import round trip, including a negative scale and -128 (quantize.rs:1259-1353)
    blocks = orc.quantize_q8_0(k[0]).reshape(ms, nkv * hd // 32, 34).copy()
    blocks[3, 0, :2] = [0x00, 0xC0]
    blocks[3, 0, 2] = 0x80
    kv.import_q8_0_blocks(0, 0, 0, blocks, blocks)
    kb, vb = kv.export_q8_0_blocks(0, 0, 0, ms)
    assert_bits_equal(kb, blocks, "imported blocks")
    dk, _ = kv.export_dequant(0, 0)
    assert dk[3, 0] == 256.0
    assert_bits_equal(dk, orc.dequant_q8_0(blocks.reshape(ms, -1)), "dequant of imported blocks")
    kv.free()


@pytest.mark.parametrize("B", [1, 8])
def test_q8_decode_llama1b_shape(eng, fb, orc, B):
    """32 q / 8 kv heads, head_dim 64, Q8_0 cache, context 4096."""
    nh, nkv, hd, ctx = 32, 8, 64, 4096
    kv, k, v = _q8_setup(eng, fb, orc, B, ctx, ctx - 1, nkv, hd, 21)
    q = normal(23, (B, 1, nh, hd), 0.125 * 4)
    knew, vnew = normal(24, (B, nkv * hd)), normal(25, (B, nkv * hd))
    for b in range(B):
        kv.write(0, b, ctx - 1, knew[b], vnew[b])
    got = eng.decode(kv, 0, nh, q)
    kd = np.stack([orc.dequant_q8_0(orc.quantize_q8_0(np.concatenate([k[b], knew[b:b + 1]]))) for b in range(B)])
    vd = np.stack([orc.dequant_q8_0(orc.quantize_q8_0(np.concatenate([v[b], vnew[b:b + 1]]))) for b in range(B)])
    want = orc.gqa_decode_batched(q.reshape(B, 1, -1), kd, vd, np.full(B, ctx, np.int32), nh, nkv, hd, threads=8)
    assert_close(got, want, f"Q8_0 batch {B}")
    kv.free()


@pytest.mark.parametrize("ctx,nh,nkv,hd", [(256, 8, 2, 64), (512, 32, 8, 64), (640, 16, 4, 64), (768, 8, 8, 64),
                                          (1024, 32, 8, 64), (1280, 8, 2, 128), (1024, 12, 3, 64),
                                          (1024, 64, 8, 64), (512, 12, 2, 64), (700, 16, 2, 128)])
def test_q8_split_counts_and_ragged_lengths(eng, fb, orc, ctx, nh, nkv, hd):
    """Contexts that give 2, 4, 5, 6, 8 and 10 slot ranges per sequence: with 2, 4 or 8 the ranges of a
    sequence merge inside the kernel (thread-block cluster), otherwise a second kernel merges.  The
    sequences of the batch have different lengths, one of them shorter than a tile.  The last three shapes
    have 8 and 6 query heads per KV head: two groups of up to 4 heads stream the cache separately."""
    B = 3
    lens = [ctx - 1, ctx // 3, 17]
    kv = eng.kv_alloc(1, B, ctx, nkv, hd, fb.KV_Q8_0)
    q = normal(61, (B, 1, nh, hd), 0.4)
    ks, vs = [], []
    for b in range(B):
        k, v = normal(62 + b, (lens[b] + 1, nkv * hd)), normal(72 + b, (lens[b] + 1, nkv * hd))
        ks.append(k); vs.append(v)
        kv.append(0, b, k[:lens[b]], v[:lens[b]]); kv.advance(b, lens[b])
        kv.write(0, b, lens[b], k[lens[b]], v[lens[b]])
    for _ in range(2):                      # twice: the second call follows one of the path's own kernels
        got = eng.decode(kv, 0, nh, q)
    for b in range(B):
        kd = orc.dequant_q8_0(orc.quantize_q8_0(ks[b]))
        vd = orc.dequant_q8_0(orc.quantize_q8_0(vs[b]))
        want = orc.gqa_decode(q[b].reshape(-1), kd, vd, nh, nkv, hd, lens[b] + 1)
        assert_close(got[b], want, f"ctx {ctx} seq {b}")
    kv.free()


def test_host_output_in_page_locked_memory(eng, fb, orc):
    """A page-locked output buffer is written by the kernels directly; a pageable one goes through a copy.
    Both must hold the same result when the call returns (Q8_0 fast path and the general f32 path)."""
    torch = pytest.importorskip("torch")
    nh, nkv, hd, ctx, B = 32, 8, 64, 1024, 2
    for dtype in (fb.KV_Q8_0, fb.KV_F32):
        kv = eng.kv_alloc(1, B, ctx, nkv, hd, dtype)
        for b in range(B):
            kv.append(0, b, normal(81 + b, (ctx - 1, nkv * hd)), normal(91 + b, (ctx - 1, nkv * hd)))
            kv.advance(b, ctx - 1)
            kv.write(0, b, ctx - 1, normal(85, nkv * hd), normal(86, nkv * hd))
        q = normal(99, (B, 1, nh, hd), 0.4)
        pageable = eng.decode(kv, 0, nh, q)
        q_pin = torch.from_numpy(q).pin_memory().numpy()
        out_pin = torch.zeros(B, 1, nh, hd).pin_memory().numpy()
        got = eng.decode(kv, 0, nh, q_pin, out=out_pin)
        assert got is out_pin
        assert_bits_equal(out_pin, pageable, "page-locked vs pageable output")
        kd, vd = kv.export_dequant(0, 0)
        assert_close(out_pin[0], orc.gqa_decode(q[0].reshape(-1), kd, vd, nh, nkv, hd, ctx), "page-locked output vs oracle")
        kv.free()


def test_q8_ring_wrap_4096_plus_256(eng, fb, orc):
    nh, nkv, hd, ms, n = 32, 8, 64, 4096, 4096 + 256
    kv = eng.kv_alloc(1, 1, ms, nkv, hd, fb.KV_Q8_0)
    k, v = normal(31, (n, nkv * hd)), normal(32, (n, nkv * hd))
    kv.append(0, 0, k[:3000], v[:3000]); kv.advance(0, 3000)
    kv.append(0, 0, k[3000:], v[3000:]); kv.advance(0, n - 3000)       # crosses the end of the ring
    assert kv.state(0) == (256, 4096)
    ring_k = np.concatenate([k[4096:], k[256:4096]])
    ring_v = np.concatenate([v[4096:], v[256:4096]])
    dk, dv = kv.export_dequant(0, 0)
    assert_bits_equal(dk, orc.dequant_q8_0(orc.quantize_q8_0(ring_k)), "wrapped K")
    q = normal(33, (1, 1, nh, hd), 0.5)
    knew, vnew = normal(34, nkv * hd), normal(35, nkv * hd)
    kv.write(0, 0, n, knew, vnew)                                      # overwrites slot 256
    ring_k[256], ring_v[256] = knew, vnew
    got = eng.decode(kv, 0, nh, q)                                     # min(4096 + 1, 4096) slots
    want = orc.gqa_decode(q, orc.dequant_q8_0(orc.quantize_q8_0(ring_k)), orc.dequant_q8_0(orc.quantize_q8_0(ring_v)),
                          nh, nkv, hd, ms)
    assert_close(got, want, "Q8_0 wrap")
    kv.free()


def test_q8_speculative_verify_six_queries(eng, fb, orc):
    """4090 cached rows + 6 draft rows; query i attends slots 0..=4090+i."""
    nh, nkv, hd, B, n_q, prior = 32, 8, 64, 2, 6, 4090
    kv, k, v = _q8_setup(eng, fb, orc, B, 4096, prior, nkv, hd, 41)
    dk_, dv_ = normal(43, (B, n_q, nkv * hd)), normal(44, (B, n_q, nkv * hd))
    for b in range(B):
        for i in range(n_q):
            kv.write(0, b, prior + i, dk_[b, i], dv_[b, i])
    q = normal(45, (B, n_q, nh, hd), 0.5)
    got = eng.decode(kv, 0, nh, q, n_q=n_q)                  # attend_len = min(len + n_q, max) = 4096
    kd = orc.dequant_q8_0(orc.quantize_q8_0(np.concatenate([k, dk_], axis=1)))
    vd = orc.dequant_q8_0(orc.quantize_q8_0(np.concatenate([v, dv_], axis=1)))
    want = orc.gqa_decode_batched(q.reshape(B, n_q, -1), kd, vd, np.full(B, prior + n_q, np.int32), nh, nkv, hd,
                                  n_q=n_q, threads=8)
    assert_close(got, want, "verify")
    # verify == sequential single-query decodes (flare-core/src/generate.rs:258-303)
    for i in range(n_q):
        one = eng.decode(kv, 0, nh, np.ascontiguousarray(q[:, i:i + 1]), attend_len=np.full(B, prior + i + 1, np.int32))
        assert_close(one, want[:, i], f"sequential step {i}")
    kv.free()


@pytest.mark.parametrize("nh,nkv,hd,n_q,prior", [
    (32, 8, 128, 5, 1000),        # head_dim 128, an odd number of queries: the last CTA carries one item only
    (16, 2, 64, 3, 777),          # 8 query heads per kv head: two head groups per query, 6 items in 3 CTAs
    (16, 2, 64, 1, 2000),         # the same heads, plain decode: the two head groups of one query share a CTA
])
def test_q8_two_items_per_warp(eng, fb, orc, nh, nkv, hd, n_q, prior):
    """Calls with several (query, group of 4 heads) items per sequence put two of them into one CTA: each query must
    see exactly its own causal range and each head its own rows, also when the items differ in range or are odd in
    number."""
    B = 3
    ms = 2048 if prior + n_q <= 2048 else 4096
    kv, k, v = _q8_setup(eng, fb, orc, B, ms, prior, nkv, hd, 71)
    dk_, dv_ = normal(73, (B, n_q, nkv * hd)), normal(74, (B, n_q, nkv * hd))
    for b in range(B):
        for i in range(n_q):
            kv.write(0, b, prior + i, dk_[b, i], dv_[b, i])
    q = normal(75, (B, n_q, nh, hd), 0.5)
    got = eng.decode(kv, 0, nh, q, n_q=n_q, attend_len=np.full(B, prior + n_q, np.int32))
    kd = orc.dequant_q8_0(orc.quantize_q8_0(np.concatenate([k, dk_], axis=1)))
    vd = orc.dequant_q8_0(orc.quantize_q8_0(np.concatenate([v, dv_], axis=1)))
    want = orc.gqa_decode_batched(q.reshape(B, n_q, -1), kd, vd, np.full(B, prior + n_q, np.int32), nh, nkv, hd,
                                  n_q=n_q, threads=8)
    assert_close(got, want, f"two items per warp, {nh}/{nkv} heads x {hd}, {n_q} queries")
    kv.free()


def test_q8_head_dim_128_long_context_and_partials(eng, fb, orc):
    """Llama-3-8B shape (32/8, head_dim 128), Q8_0; slot ranges merged by log-sum-exp."""
    nh, nkv, hd, n = 32, 8, 128, 8192
    kv, k, v = _q8_setup(eng, fb, orc, 1, n, n, nkv, hd, 51)
    q = normal(53, (1, 1, nh, hd), 0.4)
    kd, vd = orc.dequant_q8_0(orc.quantize_q8_0(k[0])), orc.dequant_q8_0(orc.quantize_q8_0(v[0]))
    want = orc.gqa_decode(q, kd, vd, nh, nkv, hd, n)
    got = eng.decode(kv, 0, nh, q, attend_len=[n])
    assert_close(got, want, "hd128 full")
    cuts = [0, 2048, 2048, 5000, 8192]
    parts = [eng.decode_partial(kv, 0, nh, q, a, b) for a, b in zip(cuts[:-1], cuts[1:])]
    for (a, b), p in zip(zip(cuts[:-1], cuts[1:]), parts):
        ref = orc.gqa_decode_partial(q, kd, vd, nh, nkv, hd, a, b)
        p = p.reshape(nh, hd + 2)
        if b > a:
            # a record is (reference max, sum, output) with any reference max at or near the true one:
            # the log-sum-exp m + ln(l) and the normalised output are what is invariant
            assert np.max(np.abs((p[:, 0] + np.log(p[:, 1])) - (ref[:, 0] + np.log(ref[:, 1])))) < 1e-3
            assert_close(p[:, 2:] / p[:, 1:2], ref[:, 2:] / ref[:, 1:2], f"partial {a}:{b}")
        else:
            assert np.all(p[:, 1] == 0)
    merged = eng.merge_partials(np.stack(parts), len(parts), nh, hd)
    assert_close(merged, want, "merged partials")
    assert_close(merged, orc.merge_partials(np.stack([orc.gqa_decode_partial(q, kd, vd, nh, nkv, hd, a, b)
                                                      for a, b in zip(cuts[:-1], cuts[1:])]), nh, hd), "oracle merge")
    kv.free()


@pytest.mark.parametrize("ms", [70, 173])
def test_q8_ring_size_not_a_tile_multiple_after_non_finite_scales(eng, fb, orc, ms):
    """A ring of 70 or 173 slots is not a multiple of the 32-slot tile and gives a CTA at most three tiles, so
    every stage is on its first use: the scale rows of the last tile that lie beyond the ring are never copied
    and that part of shared memory holds what the previous kernel left.  Here the previous kernel streamed a
    cache whose scales are Inf / NaN bit patterns on every SM; none of it may leak into the result."""
    nh, nkv, hd = 32, 8, 64
    poison = eng.kv_alloc(1, 300, 96, nkv, hd, fb.KV_Q8_0)
    blocks = np.zeros((96, nkv * hd // 32, 34), np.uint8)
    blocks[:, :, 0:2] = [0x00, 0x7E]                          # f16 NaN scale
    blocks[::2, :, 0:2] = [0x00, 0x7C]                        # f16 +Inf scale
    for b in range(300):
        poison.import_q8_0_blocks(0, b, 0, blocks, blocks)
    poison.advance(-1, 95)
    B = 8
    kv = eng.kv_alloc(1, B, ms, nkv, hd, fb.KV_Q8_0)
    k, v = normal(141, (B, ms, nkv * hd)), normal(142, (B, ms, nkv * hd))
    for b in range(B):
        kv.append(0, b, k[b, :-1], v[b, :-1]); kv.advance(b, ms - 1)
        kv.write(0, b, ms - 1, k[b, -1], v[b, -1])
    q = normal(143, (B, 1, nh, hd), 0.4)
    kd = orc.dequant_q8_0(orc.quantize_q8_0(k))
    vd = orc.dequant_q8_0(orc.quantize_q8_0(v))
    want = orc.gqa_decode_batched(q.reshape(B, 1, -1), kd, vd, np.full(B, ms, np.int32), nh, nkv, hd)
    for attempt in range(2):
        eng.decode(poison, 0, nh, np.zeros((300, 1, nh, hd), np.float32))     # leaves NaN / Inf scales in every stage
        got = eng.decode(kv, 0, nh, q)
        assert_close(got, want, f"ring of {ms} slots, attempt {attempt}")
    # two local shards as separate partial calls (the shape a rank of a split sequence sees), then the merge
    eng.decode(poison, 0, nh, np.zeros((300, 1, nh, hd), np.float32))
    cut = (ms // 2) // 32 * 32 + 32
    parts = np.stack([eng.decode_partial(kv, 0, nh, q, 0, cut), eng.decode_partial(kv, 0, nh, q, cut, ms)])
    merged = eng.merge_partials(parts.reshape(2, B * nh, hd + 2), 2, B * nh, hd)
    assert_close(merged, want, f"ring of {ms} slots, two partials merged")
    poison.free(); kv.free()


def test_stats_report_bytes_flops_and_time(eng, fb, orc):
    """flare_attn_get_stats: device time by CUDA events, algorithmic bytes and flops of the last call."""
    nh, nkv, hd, ctx, B = 32, 8, 64, 2048, 4
    kv = eng.kv_alloc(1, B, ctx, nkv, hd, fb.KV_Q8_0)
    for b in range(B):
        kv.append(0, b, normal(151 + b, (ctx - 1, nkv * hd)), normal(161 + b, (ctx - 1, nkv * hd)))
    kv.advance(-1, ctx - 1)
    q = normal(171, (B, 1, nh, hd), 0.4)
    eng.enable_stats(True)
    eng.set_peaks(6500.0, 1600.0)
    before = eng.stats().calls
    eng.decode(kv, 0, nh, q)
    eng.decode(kv, 0, nh, q, attend_len=[1000, 1, 0, 2048])
    st = eng.stats()
    assert st.calls == before + 2 and st.last_op == fb.OP_DECODE
    assert st.last_bytes == (1000 + 1 + 2048) * 2 * (nkv * hd + nkv * hd // 16)
    assert st.last_flops == 4.0 * nh * hd * (1000 + 1 + 2048)
    assert 0.5 < st.last_elapsed_us < 5000.0
    assert abs(st.last_gbs - st.last_bytes / (st.last_elapsed_us * 1e-6) / 1e9) < 1e-6 * st.last_gbs
    assert abs(st.last_frac_of_peak - st.last_gbs / 6500.0) < 1e-9
    eng.enable_stats(False)
    eng.decode(kv, 0, nh, q)
    assert eng.stats().calls == before + 2
    kv.free()


def test_bounded_wait_gives_up_and_context_survives(fb, orc):
    """A kernel wait that nothing satisfies runs out, the status reaches the host as ERR_TIMEOUT, and the
    same context then computes a correct attention (nothing hung, nothing poisoned)."""
    e = fb.Engine(0)
    assert e.selftest_wait_timeout() == fb.ERR_TIMEOUT
    assert e.selftest_wait_timeout() == fb.ERR_TIMEOUT      # the status word was cleared in between
    nh, nkv, hd, ctx = 8, 2, 64, 300
    kv = e.kv_alloc(1, 1, 512, nkv, hd, fb.KV_Q8_0)
    k, v = normal(5, (ctx, nkv * hd)), normal(6, (ctx, nkv * hd))
    kv.append(0, 0, k, v); kv.advance(0, ctx - 1)
    q = normal(7, (1, 1, nh, hd), 0.4)
    got = e.decode(kv, 0, nh, q)
    kd, vd = kv.export_dequant(0, 0)
    assert_close(got, orc.gqa_decode(q.reshape(-1), kd, vd, nh, nkv, hd, ctx), "after a timed-out wait")
    kv.free()
    e.close()


def test_bad_arguments_are_rejected(eng, fb):
    with pytest.raises(fb.FlareError):
        eng.kv_alloc(1, 1, 64, 2, 48, fb.KV_Q8_0)        # head_dim % 32
    with pytest.raises(fb.FlareError):
        eng.kv_alloc(1, 1, 100, 2, 64, fb.KV_KIVI_G32)   # max_seq_len % 128
    with pytest.raises(fb.FlareError):
        eng.kv_alloc(0, 1, 64, 2, 64, fb.KV_F32)
    kv = eng.kv_alloc(1, 1, 64, 2, 64, fb.KV_F32)
    q = np.zeros((1, 1, 3, 64), np.float32)
    with pytest.raises(fb.FlareError) as e:
        eng.decode(kv, 0, 3, q)                           # 3 heads over 2 kv heads
    assert e.value.status == fb.ERR_INVALID_ARG
    with pytest.raises(fb.FlareError):
        eng.decode(kv, 1, 4, np.zeros((1, 1, 4, 64), np.float32))     # layer out of range
    with pytest.raises(fb.FlareError):
        eng.decode(kv, 0, 4, np.zeros((1, 1, 4, 64), np.float32), attend_len=[65])
    with pytest.raises(fb.FlareError):
        kv.write(0, 3, 0, np.zeros(128, np.float32), np.zeros(128, np.float32))   # sequence out of range
    kv.free()
