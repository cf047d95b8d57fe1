"""Generates the committed fixtures of this folder (`python tests/golden/make_golden.py`).

The reference is a Rust project and cannot be run where these fixtures are made, so the expected
values come from the CPU restatement under `oracle/` (which the CPU tests pin against the
reference's own known-answer tests).  The fixtures freeze those values: a later change of the
restatement or of a CUDA kernel is caught against bytes on disk, not against a moving target.

golden_v1.npz holds, all with seeded inputs:
  f16_*            f32 -> f16 -> f32 round trip of 4096 values incl. subnormals, halfway cases, inf, nan
  q8_*             Q8_0 quantisation of 64 blocks: the 34-byte block stream and its dequantised values
  dec_{i}_*        GQA decode attention (online softmax), the reference test's six shapes + 2 larger (GQA 4, head_dim 64 and 128)
  pre_*            causal prefill attention (S 70, 2 q / 1 kv heads, head_dim 64), plain and window 16
  kivi_ref_*       the reference's 2-bit KIVI cache (2 kv heads, head_dim 32) after 70 tokens: every plane, and its dequantised view
  g32_*            the group-32 KIVI cache (1 kv head, head_dim 64) after 200 tokens: every plane, and its dequantised view
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

DEC_SHAPES = [(2, 2, 2, 1), (2, 2, 2, 6), (4, 2, 4, 10), (32, 8, 64, 20), (8, 4, 64, 1), (1, 1, 3, 5),
              (8, 2, 64, 300), (4, 1, 128, 200)]      # (heads, kv heads, head_dim, seq_len)


KIVI_REF_PLANES = ["key_packed", "value_packed", "key_scales", "key_mins", "value_scales", "value_mins",
                   "residual_keys", "residual_values"]
G32_PLANES = ["k_codes", "k_meta", "v_codes", "v_meta", "res_k", "res_v"]


def normal(seed, shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


def build():
    import oracle as orc
    out = {}
    # ---- f16
    rng = np.random.default_rng(11)
    x = np.concatenate([
        normal(12, 3000, 10.0), (rng.standard_normal(500) * 1e-6).astype(np.float32),
        np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 65504.0, 65520.0, 65519.99, 5.9604645e-8, 2.9802322e-8, 6.1035156e-5],
                 dtype=np.float32),
        (np.arange(585, dtype=np.float32) + 0.5) * np.float32(2.0 ** -14)])[:4096]
    bits = orc.f32_to_f16(x)
    out["f16_in"], out["f16_bits"], out["f16_back"] = x, bits, orc.f16_to_f32(bits)
    # ---- Q8_0
    v = normal(21, 64 * 32, 3.0)
    v[32:64] = 0.0                                    # an all-zero block
    v[64:96] *= 1e-4
    blocks = orc.quantize_q8_0(v)
    out["q8_in"], out["q8_blocks"] = v, blocks
    out["q8_dequant"] = orc.dequant_q8_0(blocks)
    # ---- decode
    for i, (nh, nkv, hd, sl) in enumerate(DEC_SHAPES):
        q, k, v = normal(100 + i, nh * hd, 0.5), normal(200 + i, (sl, nkv * hd)), normal(300 + i, (sl, nkv * hd))
        out[f"dec_{i}_q"], out[f"dec_{i}_k"], out[f"dec_{i}_v"] = q, k, v
        out[f"dec_{i}_out"] = orc.gqa_decode(q, k, v, nh, nkv, hd, sl)
    # ---- prefill
    S, nh, nkv, hd = 70, 2, 1, 64
    # inputs rounded to bf16: head_dim 64/128 prefill computes on bf16 operands, the conversion is then exact
    q, k, v = (orc.bf16_round(a) for a in (normal(41, (S, nh * hd), 0.5), normal(42, (S, nkv * hd), 0.5), normal(43, (S, nkv * hd), 0.5)))
    out["pre_q"], out["pre_k"], out["pre_v"] = q, k, v
    out["pre_out"] = orc.prefill(q, k, v, S, nh, nkv, hd)
    out["pre_out_w16"] = orc.prefill(q, k, v, S, nh, nkv, hd, window=16)
    # ---- reference KIVI cache
    nkv, hd, ms, n = 2, 32, 128, 70
    kvd = nkv * hd
    k, v = normal(51, (n, kvd)), normal(52, (n, kvd))
    c = orc.QuantizedKvCache(1, ms, nkv, hd)
    for t in range(n):
        c.write(0, k[t], v[t]); c.advance()
    out["kivi_ref_k"], out["kivi_ref_v"] = k, v
    for name in KIVI_REF_PLANES:
        out[f"kivi_ref_plane_{name}"] = c.plane(name, 0)
    out["kivi_ref_dk"], out["kivi_ref_dv"] = c.dequant_keys(0), c.dequant_values(0)
    # ---- group-32 KIVI cache
    kvd, ms, n = 64, 256, 200
    k, v = normal(61, (n, kvd)), normal(62, (n, kvd))
    k[:, [3, 47]] *= 8
    g = orc.G32Cache(ms, kvd)
    for t in range(n):
        g.write_advance(k[t], v[t])
    out["g32_k"], out["g32_v"] = k, v
    for name in G32_PLANES:
        out[f"g32_plane_{name}"] = g.plane(name)
    dk, dv = g.dequant()
    out["g32_dk"], out["g32_dv"] = dk, dv
    return out


if __name__ == "__main__":
    data = build()
    path = os.path.join(HERE, "golden_v1.npz")
    np.savez_compressed(path, **data)
    print(path, os.path.getsize(path), "bytes,", len(data), "arrays")
