"""GPU parity at the full sizes of the benchmark configurations, through the C ABI, against the CPU oracle.

  C2  32 q / 8 kv heads, head_dim 64, Q8_0, context 4096, batch 32, two layers
  C3  the same heads, 2-bit group-32 KIVI cache, context 32768, batch 16
  C4  32 / 8 heads, head_dim 128, bf16 prefill, S 4096 x batch 4, and window 4096 at S 8192
  C5  32 / 8 heads, head_dim 128, Q8_0, one sequence of 131072 slots: whole, and as four slot ranges merged
plus the trait hook's own contract for prefill: f32 inputs that are NOT representable in 16 bits, against the
f32 loop of flare-core/src/model.rs:336-368.
"""
import numpy as np
import pytest

from util import ABS_TOL, REL_TOL, assert_close, normal

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


def test_c2_q8_batch32_two_layers(eng, fb, orc):
    """Every sequence of both layers: the tensor maps address a sequence as layer * batch + sequence."""
    nh, nkv, hd, ctx, B, L = 32, 8, 64, 4096, 32, 2
    kv = eng.kv_alloc(L, B, ctx, nkv, hd, fb.KV_Q8_0)
    for layer in range(L):
        for b in range(B):
            seed = 1000 + 100 * layer + b
            kv.append(layer, b, normal(seed, (ctx - 1, nkv * hd)), normal(seed + 50, (ctx - 1, nkv * hd)))
    kv.advance(-1, ctx - 1)
    q = normal(7, (L, B, 1, nh, hd), 0.5)
    knew, vnew = normal(8, (L, B, nkv * hd)), normal(9, (L, B, nkv * hd))
    outs = []
    for layer in range(L):
        kv.write_step(layer, knew[layer], vnew[layer])
        outs.append(eng.decode(kv, layer, nh, q[layer]))
    worst = 0.0
    for layer in range(L):
        for b in range(B):
            kd, vd = kv.export_dequant(layer, b)
            want = orc.gqa_decode(q[layer, b].reshape(-1), kd, vd, nh, nkv, hd, ctx)
            worst = max(worst, assert_close(outs[layer][b], want, f"layer {layer} seq {b}"))
    # the fused step entry point gives the same answer as write + attend
    out_step = eng.decode_step(kv, 1, nh, knew[1], vnew[1], q[1])
    assert np.array_equal(out_step, outs[1])
    kv.free()


def _kivi_c3_cache(eng, fb, B, ctx, n_rows, nkv, hd, seed):
    kv = eng.kv_alloc(1, B, ctx, nkv, hd, fb.KV_KIVI_G32)
    rng = np.random.default_rng(seed)
    for b in range(B):
        k = rng.standard_normal((n_rows, nkv * hd), dtype=np.float32)
        v = rng.standard_normal((n_rows, nkv * hd), dtype=np.float32)
        k[:, rng.permutation(nkv * hd)[:6]] *= 8            # 1 % of the key channels are outliers
        kv.append(0, b, k, v)
        kv.advance(b, n_rows)
    return kv


def test_c3_kivi_ctx32768_batch16(eng, fb, orc):
    nh, nkv, hd, ctx, B = 32, 8, 64, 32768, 16
    kv = _kivi_c3_cache(eng, fb, B, ctx, ctx - 1, nkv, hd, 2)
    q = normal(21, (B, 1, nh, hd), 0.125)
    new = normal(22, (B, nkv * hd))
    kv.write_step(0, new, new)
    got = eng.decode(kv, 0, nh, q)                # write -> attend(len + 1) -> advance, as the model does
    assert np.all(np.isfinite(got))
    kv.advance(-1, 1)
    for b in (0, 7, B - 1):
        # after the advance the dequantised view is what the attention saw: the newest 128 tokens (the new
        # one included) from the f16 ring, every older one from its 2-bit codes
        kd, vd = kv.export_dequant(0, b)
        assert np.array_equal(kd[ctx - 1], orc.f16_to_f32(orc.f32_to_f16(new[b])))
        want = orc.gqa_decode(q[b].reshape(-1), kd, vd, nh, nkv, hd, ctx)
        assert_close(got[b], want, f"KIVI seq {b}")
    kv.free()


@pytest.mark.parametrize("S,W,B", [(4096, 0, 4), (8192, 4096, 4)])
def test_c4_prefill_bf16_full_size(eng, fb, orc, S, W, B):
    nh, nkv, hd = 32, 8, 128
    rng = np.random.default_rng(3)
    mk = lambda heads: orc.f32_to_bf16(rng.standard_normal((B, S, heads * hd), dtype=np.float32) * np.float32(0.5))
    qb, kb, vb = mk(nh), mk(nkv), mk(nkv)
    got = eng.prefill(qb, kb, vb, B, S, nh, nkv, hd, window=W, in_dtype=fb.DT_BF16, out_dtype=fb.DT_BF16)
    f32 = lambda u: (u.astype(np.uint32) << 16).view(np.float32)
    got32 = f32(got).reshape(B, S, nh * hd)
    for b in range(B):
        want = orc.prefill(f32(qb[b]), f32(kb[b]), f32(vb[b]), S, nh, nkv, hd, window=W, row_start=(17 * b + 5) % 251,
                           row_step=251, threads=orc.max_threads())
        rows = ~np.isnan(want[:, 0])
        assert rows.sum() >= S // 251
        err = np.abs(got32[b][rows] - want[rows])
        # the output itself is bf16: one more half-ulp (2^-9 relative) on top of the tolerance
        assert np.all(err <= ABS_TOL + (REL_TOL + 2.0 ** -8) * np.abs(want[rows])), (b, float(err.max()))


def test_c5_q8_131072_slots_whole_and_in_four_ranges(eng, fb, orc):
    """One CTA per SM and a 148-way split (merged by the second kernel) for the whole sequence; then the
    multi-GPU building blocks on one device: four slot ranges as partial records, merged by log-sum-exp."""
    nh, nkv, hd, n = 32, 8, 128, 131072
    kv = eng.kv_alloc(1, 1, n, nkv, hd, fb.KV_Q8_0)
    chunk = 16384
    for c in range(n // chunk):
        kv.append(0, 0, normal(400 + c, (chunk, nkv * hd)), normal(500 + c, (chunk, nkv * hd)))
        kv.advance(0, chunk)
    q = normal(4, (1, 1, nh, hd), 4.0 / np.sqrt(hd))
    kd, vd = kv.export_dequant(0, 0)
    att = np.full(1, n, np.int32)
    want = orc.gqa_decode_heads_mt(q.reshape(1, -1), kd[None], vd[None], att, nh, nkv, hd, orc.max_threads()).reshape(-1)
    got = eng.decode(kv, 0, nh, q, attend_len=[n])
    assert_close(got, want, "131072 slots, one call")
    cuts = [0, 32768, 65536, 98304, n]
    parts = np.stack([eng.decode_partial(kv, 0, nh, q, a, b) for a, b in zip(cuts[:-1], cuts[1:])])
    merged = eng.merge_partials(parts, 4, nh, hd)
    assert_close(merged, want, "131072 slots, four ranges merged")
    kv.free()


@pytest.mark.parametrize("hd,S,nh,nkv", [(128, 700, 8, 2), (64, 300, 4, 4)])
@pytest.mark.parametrize("recipe", ["normal", "outliers", "large_v", "tiny_q"])
def test_trait_hook_prefill_takes_f32_as_f32(fb, orc, hd, S, nh, nkv, recipe):
    """ComputeBackend::prefill_attention_gpu hands over f32 slices; the contract is flare-core's f32 loop
    within 2e-3 + 1e-3 |x|.  Inputs here use all 24 bits (nothing is pre-rounded), and row 0 — which attends
    one key and must return that key's value row — is part of the check."""
    rng = np.random.default_rng(S + hd)
    q = rng.standard_normal((S, nh * hd), dtype=np.float32) * np.float32(0.5)
    k = rng.standard_normal((S, nkv * hd), dtype=np.float32) * np.float32(0.5)
    v = rng.standard_normal((S, nkv * hd), dtype=np.float32) * np.float32(0.5)
    if recipe == "outliers":
        k[:, rng.permutation(nkv * hd)[:max(1, nkv * hd // 100)]] *= 8
    elif recipe == "large_v":
        v *= np.float32(3.0e5)                  # beyond the f16 range: the conversion must scale it
    elif recipe == "tiny_q":
        q *= np.float32(1.0e-6); k *= np.float32(1.0e6)      # below the f16 normal range and above 2^15
    be = fb.CudaBackend(0)
    got = be.prefill_attention_gpu(q, k, v, S, nh, nkv, hd).reshape(S, -1)
    want = orc.prefill(q, k, v, S, nh, nkv, hd, threads=8)
    assert np.all(np.isfinite(got))
    err = np.abs(got - want)
    bound = ABS_TOL * (3.0e5 if recipe == "large_v" else 1.0) + REL_TOL * np.abs(want)
    assert np.all(err <= bound), (recipe, float(err.max()), int(np.argmax(err)) // (nh * hd))
    # row 0 is v[0] per head group
    G = nh // nkv
    for h in range(nh):
        np.testing.assert_allclose(got[0, h * hd:(h + 1) * hd], v[0, (h // G) * hd:(h // G + 1) * hd], rtol=REL_TOL, atol=0)
