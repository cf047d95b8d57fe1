"""The device-resident single-token forward pass (flare_forward_token) against the CPU restatement of
Model::forward on the Q8_0 path (flare-core/src/model.rs:1740-1790, 2010-2548).

Integer dots, block sums, the rotation and every quantisation step are the reference's operation for operation;
the norm's sum of squares (a tree here, left to right on the CPU) and exp() are not, so an intermediate value can
land on the other side of a rounding boundary of the next quantisation.  Logits are therefore compared within a
tolerance scaled to their spread, and the greedy token must agree wherever the CPU's own top-2 margin is larger
than that tolerance."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _q8(orc, rng, rows, cols, scale):
    w = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(scale)
    return np.ascontiguousarray(orc.quantize_q8_0(w.reshape(-1))).reshape(-1)


def _make_model(orc, rng, cfg, n_layers, output_q8):
    dim, inter = cfg["hidden_dim"], cfg["intermediate_dim"]
    q_dim, kv_dim = cfg["num_heads"] * cfg["head_dim"], cfg["num_kv_heads"] * cfg["head_dim"]
    layers = []
    for _ in range(n_layers):
        layers.append(dict(
            attn_norm=(1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32),
            qkv=_q8(orc, rng, q_dim + 2 * kv_dim, dim, dim ** -0.5),
            wo=_q8(orc, rng, dim, q_dim, q_dim ** -0.5),
            ffn_norm=(1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32),
            gate_up=_q8(orc, rng, 2 * inter, dim, dim ** -0.5),
            down=_q8(orc, rng, dim, inter, inter ** -0.5)))
    output_norm = (1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    if output_q8:
        return layers, output_norm, _q8(orc, rng, cfg["vocab_size"], dim, dim ** -0.5), None
    return layers, output_norm, None, rng.standard_normal((cfg["vocab_size"], dim), dtype=np.float32) * np.float32(dim ** -0.5)


@pytest.mark.parametrize("kv_dtype,output_q8,batch,nh,nkv,hd,dim,inter,vocab", [
    ("f32", True, 1, 4, 2, 64, 256, 512, 1000),        # the f32 cache the reference's own forward keeps
    ("q8_0", False, 2, 8, 2, 64, 256, 512, 1000),      # quantised cache (tensor-core attention), f32 output matrix, two sequences
    ("f32", True, 1, 16, 4, 64, 1024, 2048, 4096),     # rows of 32 and 64 blocks: the 16-byte weight loads of the product
])
def test_forward_token_matches_the_cpu_path(orc, kv_dtype, output_q8, batch, nh, nkv, hd, dim, inter, vocab):
    import flarellm_b200 as fb
    rng = np.random.default_rng(11 + batch)
    cfg = dict(hidden_dim=dim, num_heads=nh, num_kv_heads=nkv, head_dim=hd, intermediate_dim=inter, vocab_size=vocab,
               rms_norm_eps=1e-5)
    n_layers, max_seq, theta, n_tokens = 2, 64, 10000.0, 6
    layers, output_norm, out_q8, out_f32 = _make_model(orc, rng, cfg, n_layers, output_q8)
    cos, sin = orc.rope_table(hd, max_seq, theta)
    eng = fb.Engine(0)
    kv = eng.kv_alloc(n_layers, batch, max_seq, nkv, hd, fb.KV_F32 if kv_dtype == "f32" else fb.KV_Q8_0)
    kv.set_rope_table(cos, sin)
    model = eng.model_create(num_layers=n_layers, **cfg)
    for li, lw in enumerate(layers):
        model.set_layer(li, **lw)
    model.set_output(output_norm, output_q8=out_q8, output_f32=out_f32)
    store = None if kv_dtype == "f32" else (lambda r: orc.dequant_q8_0(orc.quantize_q8_0(r)))
    caches = [([np.zeros((max_seq, nkv * hd), np.float32) for _ in range(n_layers)],
               [np.zeros((max_seq, nkv * hd), np.float32) for _ in range(n_layers)]) for _ in range(batch)]
    embed = rng.standard_normal((50, cfg["hidden_dim"]), dtype=np.float32)
    agree = 0
    for t in range(n_tokens):
        tokens = [(7 * t + 3 * b + 1) % 50 for b in range(batch)]
        x = embed[tokens]
        got = model.forward(kv, x, positions=[t] * batch)
        assert got.shape == (batch, cfg["vocab_size"]) and np.all(np.isfinite(got))
        for b in range(batch):
            want = orc.forward_token_q8(cfg, layers, output_norm, out_q8, out_f32, cos, sin, theta, caches[b][0], caches[b][1],
                                        t, x[b], t, store=store)
            tol = 2e-3 * float(np.abs(want).max()) + 1e-3 * np.abs(want)
            err = np.abs(got[b] - want)
            assert np.all(err <= tol), (t, b, float(err.max()), float(np.abs(want).max()))
            top2 = np.sort(want)[-2:]
            if top2[1] - top2[0] > 2 * float(tol.max()):
                assert int(np.argmax(got[b])) == int(np.argmax(want))
                agree += 1
        assert kv.state(0)[1] == t + 1            # the cache advanced by one, as Model::forward does
    assert agree >= 1
    model.free(); kv.free(); eng.close()


def test_forward_token_refuses_a_cache_of_another_shape(orc):
    import flarellm_b200 as fb
    eng = fb.Engine(0)
    model = eng.model_create(hidden_dim=64, num_heads=2, num_kv_heads=1, head_dim=32, intermediate_dim=64, vocab_size=10,
                             num_layers=1, rms_norm_eps=1e-5)
    kv = eng.kv_alloc(2, 1, 16, 1, 32, fb.KV_F32)
    with pytest.raises(fb.FlareError) as e:
        model.forward(kv, np.zeros((1, 64), np.float32), positions=[0])
    assert e.value.status in (fb.ERR_INVALID_ARG, fb.ERR_STATE)
    model.free(); kv.free(); eng.close()
