"""GPU parity for the two steps either side of attention that the library also takes over:

* rotary position embedding fused into the step write (flare-core/src/model.rs:2168-2206, 7256-7292): the
  rotated key row bit for bit, then the Q8_0 / 2-bit codes and statistics computed from it bit for bit;
* speculative verify as one n-query attention call per layer (flare-core/src/generate.rs:244-306): the same
  accepted tokens, the same cache state as the reference's one-forward-per-draft loop.
"""
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


def _rotated(orc, rows, nkv, hd, positions, theta, cos, sin):
    return np.stack([orc.apply_rope_with_table(rows[b], nkv, hd, int(positions[b]), theta, cos, sin) for b in range(len(rows))])


@pytest.mark.parametrize("hd,nkv", [(64, 8), (128, 2)])
def test_rope_fused_step_write_is_bit_exact(eng, fb, orc, hd, nkv):
    """Every cache type: what lands in the cache equals the CPU rotating the row with the same table and then
    writing it.  Positions include 0 (identity), the reference's table cap - 1 and one beyond it (a longer table)."""
    theta, B, ms = 10000.0, 5, 256
    cos, sin = orc.rope_table(hd, 9000, theta, cap=9000)
    positions = np.array([0, 1, 77, 8191, 8999], np.int64)
    k, v = normal(201, (B, nkv * hd)), normal(202, (B, nkv * hd))
    k[3, :32] = 0.0
    want_k = _rotated(orc, k, nkv, hd, positions, theta, cos, sin)
    # position 8999 lies beyond the reference's table: its inline fallback gives the same row
    assert np.array_equal(want_k[4], orc.apply_rope(k[4], nkv, hd, 8999, theta))
    assert np.array_equal(want_k[0], k[0])
    # f32: the rotated row itself
    kv = eng.kv_alloc(1, B, ms, nkv, hd, fb.KV_F32)
    kv.set_rope_table(cos, sin)
    kv.write_step_rope(0, k, v, positions)
    for b in range(B):
        assert_bits_equal(kv.export_plane(0, b, fb.PLANE_K, np.float32)[:nkv * hd], want_k[b], f"f32 rotated row {b}")
        assert_bits_equal(kv.export_plane(0, b, fb.PLANE_V, np.float32)[:nkv * hd], v[b], f"f32 value row {b}")
    # rows rotated in place (q): host and device forms
    q = normal(203, (B, 4 * nkv, hd))
    want_q = _rotated(orc, q.reshape(B, -1), 4 * nkv, hd, positions, theta, cos, sin)
    got_q = kv.rope_rows(q.copy(), 4 * nkv, positions)
    assert_bits_equal(got_q.reshape(B, -1), want_q, "q rotated in place")
    kv.free()
    # Q8_0: the quantiser of model.rs:5507-5527 on the rotated row
    kv = eng.kv_alloc(1, B, ms, nkv, hd, fb.KV_Q8_0)
    kv.set_rope_table(cos, sin)
    kv.write_step_rope(0, k, v, positions)
    for b in range(B):
        kb, vb = kv.export_q8_0_blocks(0, b, 0, 1)
        assert_bits_equal(kb, orc.quantize_q8_0(want_k[b]), f"Q8_0 blocks of the rotated row {b}")
        assert_bits_equal(vb, orc.quantize_q8_0(v[b]), f"Q8_0 value blocks {b}")
    with pytest.raises(fb.FlareError):
        kv.write_step_rope(0, k, v, np.full(B, 9000, np.int64))          # beyond the table
    kv.free()
    kv = eng.kv_alloc(1, B, ms, nkv, hd, fb.KV_Q8_0)
    with pytest.raises(fb.FlareError) as e:
        kv.write_step_rope(0, k, v, positions)                            # no table yet
    assert e.value.status == fb.ERR_STATE
    kv.free()


def test_rope_fused_step_write_two_bit_caches(eng, fb, orc):
    """The reference's QuantizedKvCache fed with rotated rows (kv_cache.rs:121-162 after model.rs:2168-2183):
    packed codes, running per-channel statistics, per-token scales and the residual window bit for bit, over
    several steps; and the group-32 cache the same way."""
    from test_gpu_kivi import G32_PLANES, REF_PLANES
    nkv, hd, ms, theta, steps = 2, 64, 128, 500000.0, 40
    cos, sin = orc.rope_table(hd, 4096, theta)
    kv = eng.kv_alloc(1, 1, ms, nkv, hd, fb.KV_KIVI_REF)
    kv.set_rope_table(cos, sin)
    oc = orc.QuantizedKvCache(1, ms, nkv, hd)
    k, v = normal(211, (steps, nkv * hd)), normal(212, (steps, nkv * hd))
    for t in range(steps):
        pos = 3000 + t
        kv.write_step_rope(0, k[t][None], v[t][None], [pos]); kv.advance()
        oc.write(0, orc.apply_rope_with_table(k[t], nkv, hd, pos, theta, cos, sin), v[t]); oc.advance()
    for oname, pname in REF_PLANES:
        assert_bits_equal(kv.export_plane(0, 0, getattr(fb, pname)), oc.plane(oname, 0), f"KIVI ref {oname}")
    kv.free()
    steps = 200
    kv = eng.kv_alloc(1, 1, 256, nkv, hd, fb.KV_KIVI_G32)
    kv.set_rope_table(cos, sin)
    og = orc.G32Cache(256, nkv * hd)
    k, v = normal(213, (steps, nkv * hd)), normal(214, (steps, nkv * hd))
    for t in range(steps):
        kv.write_step_rope(0, k[t][None], v[t][None], [t]); kv.advance()
        og.write_advance(orc.apply_rope_with_table(k[t], nkv, hd, t, theta, cos, sin), v[t])
    for oname, pname in G32_PLANES:
        assert_bits_equal(kv.export_plane(0, 0, getattr(fb, pname)), og.plane(oname), f"group-32 {oname}")
    kv.free()


class ToyModel:
    """A two-layer attention-only model small enough to run on the CPU with numpy, with every attention call
    going through `attend`: enough structure for the token at position p to depend on all tokens before it."""

    def __init__(self, seed, vocab=50, d=64, nh=8, nkv=2, hd=64, layers=2):
        rng = np.random.default_rng(seed)
        f = lambda *s: (rng.standard_normal(s) / np.sqrt(s[0])).astype(np.float32)
        self.vocab, self.d, self.num_heads, self.nkv, self.hd, self.num_layers = vocab, d, nh, nkv, hd, layers
        self.emb = rng.standard_normal((vocab, d)).astype(np.float32)
        self.wq = [f(d, nh * hd) * 3 for _ in range(layers)]
        self.wk = [f(d, nkv * hd) * 3 for _ in range(layers)]
        self.wv = [f(d, nkv * hd) for _ in range(layers)]
        self.wo = [f(nh * hd, d) for _ in range(layers)]
        self.head = f(d, vocab)

    def embed(self, tokens):
        return self.emb[np.asarray(tokens)]

    def qkv(self, layer, x):
        return x @ self.wq[layer], x @ self.wk[layer], x @ self.wv[layer]

    def post(self, layer, x, attn):
        return x + attn @ self.wo[layer]

    def greedy(self, x):
        return [int(t) for t in np.argmax(x @ self.head, axis=-1)]


def test_batched_verify_equals_the_sequential_loop(eng, fb, orc):
    """generate.rs:258-303 forwards one draft at a time and stops at the first mismatch; verify_drafts writes all
    draft rows, makes ONE n-query attention call per layer, accepts the matching prefix (plus the correcting
    token) and truncates the cache.  Both must accept the same tokens and leave the same cache length, for a
    draft that is all right, one that goes wrong in the middle, and one that is wrong at once."""
    model = ToyModel(7)
    nkv, hd, ms = model.nkv, model.hd, 512
    prompt = [3, 14, 15, 9, 26, 5, 35, 8, 9, 7, 9, 32, 38, 46, 26, 43]

    def fresh():
        kv = eng.kv_alloc(model.num_layers, 1, ms, nkv, hd, fb.KV_Q8_0)
        for t in prompt[:-1]:                                 # prefill token by token
            fb.forward_token(eng, kv, model, t)
        return kv

    # the true greedy continuation, one token at a time
    kv = fresh()
    truth, last = [], prompt[-1]
    for _ in range(8):
        last = fb.forward_token(eng, kv, model, last)
        truth.append(last)
    kv.free()
    for drafts in (truth[:6], truth[:3] + [(truth[3] + 1) % model.vocab] + truth[4:6], [(truth[0] + 1) % model.vocab] + truth[1:6]):
        kv_seq, kv_bat = fresh(), fresh()
        want = fb.verify_drafts_sequential(eng, kv_seq, model, prompt[-1], drafts)
        got = fb.verify_drafts(eng, kv_bat, model, prompt[-1], drafts)
        assert got == want, (drafts, got, want)
        n_match = 0
        while n_match < len(drafts) and drafts[n_match] == truth[n_match]:
            n_match += 1
        assert got == truth[:min(n_match + 1, len(drafts))]
        assert kv_bat.state(0) == kv_seq.state(0) == (len(prompt) - 1 + len(got), len(prompt) - 1 + len(got))
        # the cache rows that survive: layer 0 (computed from the embeddings alone) byte for byte; later layers saw
        # attention outputs that may differ in the last bits between the 1-query and the n-query call, so a code
        # may flip by one step here and there
        n = kv_bat.len(0)
        a, b = kv_bat.export_q8_0_blocks(0, 0, 0, n), kv_seq.export_q8_0_blocks(0, 0, 0, n)
        assert_bits_equal(a[0], b[0], "layer-0 K rows after verify"); assert_bits_equal(a[1], b[1], "layer-0 V rows after verify")
        for layer in range(1, model.num_layers):
            (ka, va), (kb, vb) = kv_bat.export_dequant(layer, 0), kv_seq.export_dequant(layer, 0)
            assert np.mean(np.abs(ka[:n] - kb[:n])) < 1e-3 and np.mean(np.abs(va[:n] - vb[:n])) < 1e-3
        kv_seq.free(); kv_bat.free()


@pytest.mark.parametrize("rows,cols,batch", [(2048, 2048, 1), (512, 2048, 32), (96, 4096, 5), (33, 64, 40), (2048, 2048, 32),
                                             (5000, 8192, 2), (37, 256, 1), (64, 96, 2)])
def test_q8_0_projection_is_bit_exact(eng, fb, orc, rows, cols, batch):
    """The Q / K / V and output projections (flare-core/src/model.rs:2016-2136, 2249-2291): matvec_q8_0_preq_into on
    quantize_input_q8_0, bit for bit — the integer dots are exact and the f32 sum over a row's blocks runs in the
    CPU's order.  Shapes: Llama-3.2-1B's q / kv projections at batch 1 and 32, a wide row (several 64-block
    chunks), a matrix smaller than a warp tile with a ragged batch."""
    rng = np.random.default_rng(rows + cols + batch)
    W = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.05)
    x = rng.standard_normal((batch, cols), dtype=np.float32)
    x[0, :32] = 0.0                                        # a zero block: d == 0, id == 0
    if batch > 1:
        x[1, 5] = 1.0e4                                    # a block dominated by one value
    blocks = orc.quantize_q8_0(W)
    w = eng.weight_upload_q8_0(blocks, rows, cols)
    got = eng.matvec_q8_0(w, x)
    want = np.stack([orc.matvec_q8_0(blocks, x[b], rows) for b in range(batch)])
    assert_bits_equal(got, want, f"Q8_0 projection {rows}x{cols}, batch {batch}")
    # device buffers in and out give the same bits
    import torch
    xd, od = torch.from_numpy(x).cuda(), torch.empty(batch, rows, device="cuda")
    eng.matvec_q8_0(w, xd.data_ptr(), out=(od.data_ptr(), batch))
    eng.sync()
    assert_bits_equal(od.cpu().numpy(), want, "device buffers")
    w.free()
