"""CPU-only: the oracle's restatements of the norm, the fused norm + quantiser, SiLU * up and the f32 product, pinned
by the known-answer tests flare-core holds for them (flare-core/src/model.rs:10219-10232, 10888-10903,
12302-12360), plus a plain numpy restatement of the same formulae as a second opinion, and the composed token."""
import numpy as np

import oracle


def test_rmsnorm_known_answers():
    # model.rs:10219-10232: rms of [1, 2, 3, 4] is sqrt(7.5 + eps)
    got = oracle.rmsnorm(np.array([1, 2, 3, 4], np.float32), np.ones(4, np.float32), 1e-5)
    rms = np.sqrt(np.float32(30.0) / np.float32(4.0) + np.float32(1e-5))
    assert np.all(np.abs(got - np.arange(1, 5, dtype=np.float32) / rms) < 1e-4)
    # model.rs:10888-10903: one element
    got = oracle.rmsnorm(np.array([2.0], np.float32), np.ones(1, np.float32), 1e-5)
    assert abs(float(got[0]) - 2.0 / np.sqrt(np.float32(4.0) + np.float32(1e-5))) < 1e-5


def test_fused_norm_quantiser_matches_the_two_steps():
    # model.rs:12302-12360, its inputs by formula: scales within 1e-6, codes within one step
    for dim in (32, 64, 128, 256, 512, 1024):
        i = np.arange(dim)
        x = (((i * 7 + 3) % 31) / 15.0 - 1.0).astype(np.float32)
        w = (((i * 11 + 5) % 23) / 11.5).astype(np.float32)
        s_two, q_two = oracle.quantize_input_q8_0(oracle.rmsnorm(x, w, 1e-5))
        s_fused, q_fused = oracle.rmsnorm_quantize_q8_0(x, w, 1e-5)
        assert np.all(np.abs(s_fused - s_two) < 1e-6), dim
        assert np.all(np.abs(q_fused.astype(np.int32) - q_two.astype(np.int32)) <= 1), dim


def test_fused_norm_quantiser_against_numpy():
    rng = np.random.default_rng(5)
    x = rng.standard_normal(256, dtype=np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    eps = np.float32(1e-5)
    sum_sq = np.float32(0.0)
    for v in x:                                   # left to right in f32, as the iterator sum does
        sum_sq = np.float32(sum_sq + np.float32(v * v))
    inv_rms = np.float32(1.0) / np.sqrt(np.float32(sum_sq / np.float32(256) + eps))
    n = (x * w).astype(np.float32) * inv_rms
    amax = np.abs(n.reshape(-1, 32)).max(axis=1)
    scale = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(scale != 0, np.float32(127.0) / amax, np.float32(0.0)).astype(np.float32)
    t = (n.reshape(-1, 32) * inv[:, None]).astype(np.float32)
    q = (np.sign(t) * np.floor(np.abs(t) + np.float32(0.5))).astype(np.int8)      # f32::round: half away from zero
    s_got, q_got = oracle.rmsnorm_quantize_q8_0(x, w, float(eps))
    assert np.array_equal(s_got, scale)
    assert np.array_equal(q_got.reshape(-1, 32), q)


def test_silu_mul_and_f32_product():
    rng = np.random.default_rng(6)
    g, u = rng.standard_normal(100, dtype=np.float32) * 3, rng.standard_normal(100, dtype=np.float32)
    want = (g.astype(np.float64) / (1.0 + np.exp(-g.astype(np.float64)))) * u
    assert np.allclose(oracle.silu_mul(g, u), want, rtol=1e-6, atol=1e-7)
    m, v = rng.standard_normal((7, 40), dtype=np.float32), rng.standard_normal(40, dtype=np.float32)
    assert np.allclose(oracle.matvec_f32(m, v, 7, 40), m.astype(np.float64) @ v, rtol=1e-5, atol=1e-5)


def test_one_token_of_the_q8_path_composes_its_pieces():
    """forward_token_q8 on one layer equals the steps written out by hand (the order of model.rs:2010-2548)."""
    rng = np.random.default_rng(7)
    dim, nh, nkv, hd, inter, vocab = 64, 2, 1, 32, 64, 50
    cfg = dict(hidden_dim=dim, num_heads=nh, num_kv_heads=nkv, head_dim=hd, intermediate_dim=inter, vocab_size=vocab,
               rms_norm_eps=1e-5)
    q8 = lambda r, c: oracle.quantize_q8_0((rng.standard_normal((r, c), dtype=np.float32) * np.float32(c ** -0.5)).reshape(-1)).reshape(-1)
    lw = dict(attn_norm=np.ones(dim, np.float32), qkv=q8((nh + 2 * nkv) * hd, dim), wo=q8(dim, nh * hd),
              ffn_norm=np.ones(dim, np.float32), gate_up=q8(2 * inter, dim), down=q8(dim, inter))
    out_norm, out_w = np.ones(dim, np.float32), q8(vocab, dim)
    cos, sin = oracle.rope_table(hd, 16, 10000.0)
    x = rng.standard_normal(dim, dtype=np.float32)
    kc, vc = [np.zeros((16, nkv * hd), np.float32)], [np.zeros((16, nkv * hd), np.float32)]
    got = oracle.forward_token_q8(cfg, [lw], out_norm, out_w, None, cos, sin, 10000.0, kc, vc, 0, x, 0)
    # by hand: with one cached slot the attention output is the value row itself
    s, qn = oracle.rmsnorm_quantize_q8_0(x, lw["attn_norm"], 1e-5)
    qkv = oracle.matvec_q8_0_preq(lw["qkv"], s, qn, (nh + 2 * nkv) * hd)
    v_row = qkv[(nh + nkv) * hd:]
    attn = np.concatenate([v_row[(h // (nh // nkv)) * hd:(h // (nh // nkv) + 1) * hd] for h in range(nh)])
    x1 = x + oracle.matvec_q8_0(lw["wo"], attn, dim)
    s, qn = oracle.rmsnorm_quantize_q8_0(x1, lw["ffn_norm"], 1e-5)
    gu = oracle.matvec_q8_0_preq(lw["gate_up"], s, qn, 2 * inter)
    x2 = x1 + oracle.matvec_q8_0(lw["down"], oracle.silu_mul(gu[:inter], gu[inter:]), dim)
    want = oracle.matvec_q8_0(out_w, oracle.rmsnorm(x2, out_norm, 1e-5), vocab)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)
    assert np.array_equal(vc[0][0], v_row)
