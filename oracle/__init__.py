"""ctypes front end of the CPU oracle (oracle/flare_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by
``bench.py``'s CPU-baseline legs.  The product package never imports it.

Each wrapper takes and returns numpy arrays; the arithmetic is entirely inside the
C file, whose functions cite the reference routine they restate.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libflare_oracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "flare_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _declare(_lib)
    return _lib


_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_u16p = C.POINTER(C.c_uint16)
_i32p = C.POINTER(C.c_int)
_sz = C.c_size_t


def _declare(L):
    L.orc_f16_to_f32_bits.restype = C.c_uint32
    L.orc_f16_to_f32_bits.argtypes = [C.c_uint16]
    L.orc_f16_to_f32.restype = C.c_float
    L.orc_f16_to_f32.argtypes = [C.c_uint16]
    L.orc_bf16_to_f32.restype = C.c_float
    L.orc_bf16_to_f32.argtypes = [C.c_uint16]
    L.orc_f32_to_f16.restype = C.c_uint16
    L.orc_f32_to_f16.argtypes = [C.c_float]
    L.orc_f32_to_bf16.restype = C.c_uint16
    L.orc_f32_to_bf16.argtypes = [C.c_float]
    L.orc_f32_to_f16_n.argtypes = [_f32p, _sz, _u16p]
    L.orc_f16_to_f32_n.argtypes = [_u16p, _sz, _f32p]
    L.orc_f32_to_bf16_n.argtypes = [_f32p, _sz, _u16p]
    L.orc_dequant_q8_0_block.argtypes = [_u8p, _sz, _f32p]
    L.orc_quantize_q8_0.argtypes = [_f32p, _sz, _u8p]
    L.orc_dequant_q8_0.argtypes = [_u8p, _sz, _f32p]
    L.orc_dequant_q8_0_mt.argtypes = [_u8p, _sz, _f32p, C.c_int]
    L.orc_q2_quantize_to_packed.argtypes = [_f32p, _sz, _u8p, _f32p, _f32p]
    L.orc_q2_dequant_per_channel.argtypes = [_u8p, _f32p, _f32p, _f32p, _sz]
    L.orc_q2_dequant_per_token.argtypes = [_u8p, C.c_float, C.c_float, _f32p, _sz]
    L.orc_q2_update_per_channel_stats.argtypes = [_f32p, _f32p, _f32p, _sz, C.c_int]
    L.orc_gqa_decode.argtypes = [_f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, C.c_float, _f32p]
    L.orc_gqa_decode_three_pass.argtypes = [_f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, _f32p]
    L.orc_gqa_decode_batched.argtypes = [_f32p, _f32p, _f32p, _sz, _sz, _sz, _i32p, _sz, _sz, _sz,
                                         C.c_float, _f32p, C.c_int]
    L.orc_gqa_decode_heads_mt.argtypes = [_f32p, _f32p, _f32p, _sz, _sz, _i32p, _sz, _sz, _sz, _f32p, C.c_int]
    L.orc_prefill.argtypes = [_f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, C.c_float, _sz, _sz, _sz, _f32p, C.c_int]
    L.orc_gqa_decode_partial.argtypes = [_f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, _sz, _f32p]
    L.orc_merge_partials.argtypes = [_f32p, _sz, _sz, _sz, _f32p]
    for name in ("orc_kv_new", "orc_qkv_new"):
        getattr(L, name).restype = C.c_void_p
        getattr(L, name).argtypes = [_sz, _sz, _sz, _sz]
    for pre in ("orc_kv", "orc_qkv"):
        getattr(L, pre + "_free").argtypes = [C.c_void_p]
        getattr(L, pre + "_write").argtypes = [C.c_void_p, _sz, _f32p, _f32p]
        getattr(L, pre + "_advance").argtypes = [C.c_void_p]
        getattr(L, pre + "_len").restype = _sz
        getattr(L, pre + "_len").argtypes = [C.c_void_p]
        getattr(L, pre + "_position").restype = _sz
        getattr(L, pre + "_position").argtypes = [C.c_void_p]
        getattr(L, pre + "_truncate_to").argtypes = [C.c_void_p, _sz]
        getattr(L, pre + "_clear").argtypes = [C.c_void_p]
    L.orc_kv_keys.restype = _f32p
    L.orc_kv_keys.argtypes = [C.c_void_p, _sz]
    L.orc_kv_values.restype = _f32p
    L.orc_kv_values.argtypes = [C.c_void_p, _sz]
    L.orc_kv_attend_len.restype = _sz
    L.orc_kv_attend_len.argtypes = [C.c_void_p]
    L.orc_qkv_dequant.argtypes = [C.c_void_p, _sz, C.c_int, _f32p]
    for name, rt in (("key_packed", _u8p), ("value_packed", _u8p), ("key_scales", _f32p),
                     ("key_mins", _f32p), ("value_scales", _f32p), ("value_mins", _f32p),
                     ("residual_keys", _f32p), ("residual_values", _f32p)):
        f = getattr(L, "orc_qkv_" + name)
        f.restype = rt
        f.argtypes = [C.c_void_p, _sz]
    L.orc_g32_quant_key_group.argtypes = [_f32p, _sz, _u8p, _u16p]
    L.orc_g32_quant_value_row.argtypes = [_f32p, _sz, _u8p, _u16p]
    L.orc_g32_dequant_key_group.argtypes = [_u8p, _u16p, _sz, _f32p]
    L.orc_g32_dequant_value_row.argtypes = [_u8p, _u16p, _sz, _f32p]
    L.orc_g32_new.restype = C.c_void_p
    L.orc_g32_new.argtypes = [_sz, _sz]
    L.orc_g32_free.argtypes = [C.c_void_p]
    L.orc_g32_write_advance.argtypes = [C.c_void_p, _f32p, _f32p]
    L.orc_g32_dequant.argtypes = [C.c_void_p, _f32p, _f32p]
    for name, rt in (("k_codes", _u8p), ("v_codes", _u8p), ("k_meta", _u16p), ("v_meta", _u16p),
                     ("res_k", _u16p), ("res_v", _u16p)):
        f = getattr(L, "orc_g32_" + name)
        f.restype = rt
        f.argtypes = [C.c_void_p]
    L.orc_g32_written.restype = _sz
    L.orc_g32_written.argtypes = [C.c_void_p]
    L.orc_max_threads.restype = C.c_int


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def _u8(a):
    a = np.ascontiguousarray(a, dtype=np.uint8)
    return a, a.ctypes.data_as(_u8p)


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ---------------------------------------------------------------- codecs
def f16_to_f32(bits) -> np.ndarray:
    bits = np.ascontiguousarray(np.atleast_1d(bits), dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().orc_f16_to_f32_n(bits.ctypes.data_as(_u16p), bits.size, out.ctypes.data_as(_f32p))
    return out


def f32_to_f16(x) -> np.ndarray:
    x = np.ascontiguousarray(np.atleast_1d(x), dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_f16_n(x.ctypes.data_as(_f32p), x.size, out.ctypes.data_as(_u16p))
    return out


def f32_to_bf16(x) -> np.ndarray:
    x = np.ascontiguousarray(np.atleast_1d(x), dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16_n(x.ctypes.data_as(_f32p), x.size, out.ctypes.data_as(_u16p))
    return out


def bf16_round(x) -> np.ndarray:
    """f32 -> nearest bf16 (RNE) -> f32."""
    return (f32_to_bf16(x).astype(np.uint32) << 16).view(np.float32)


def dequant_q8_0_block(block: bytes, out32: np.ndarray) -> None:
    b, bp = _u8(np.frombuffer(bytes(block), dtype=np.uint8)) if len(block) else (None, None)
    assert out32.dtype == np.float32 and out32.size == 32
    lib().orc_dequant_q8_0_block(bp, len(block), out32.ctypes.data_as(_f32p))


def quantize_q8_0(x) -> np.ndarray:
    """f32 [..., n] (n % 32 == 0) -> uint8 [..., n/32*34] Q8_0 block stream."""
    x, xp = _f(x)
    assert x.shape[-1] % 32 == 0
    out = np.empty(x.shape[:-1] + (x.shape[-1] // 32 * 34,), dtype=np.uint8)
    lib().orc_quantize_q8_0(xp, x.size, out.ctypes.data_as(_u8p))
    return out


def dequant_q8_0(blocks) -> np.ndarray:
    b, bp = _u8(blocks)
    assert b.shape[-1] % 34 == 0
    out = np.empty(b.shape[:-1] + (b.shape[-1] // 34 * 32,), dtype=np.float32)
    lib().orc_dequant_q8_0(bp, out.size, out.ctypes.data_as(_f32p))
    return out


def dequant_q8_0_mt(blocks, threads) -> np.ndarray:
    """dequant_q8_0 spread over host threads (same arithmetic per block)."""
    b, bp = _u8(blocks)
    assert b.shape[-1] % 34 == 0
    out = np.empty(b.shape[:-1] + (b.shape[-1] // 34 * 32,), dtype=np.float32)
    lib().orc_dequant_q8_0_mt(bp, out.size, out.ctypes.data_as(_f32p), int(threads))
    return out


def q2_quantize_to_packed(values):
    v, vp = _f(values)
    packed = np.zeros((v.size + 3) // 4, dtype=np.uint8)
    s, m = C.c_float(), C.c_float()
    lib().orc_q2_quantize_to_packed(vp, v.size, packed.ctypes.data_as(_u8p), C.byref(s), C.byref(m))
    return packed, np.float32(s.value), np.float32(m.value)


def q2_dequant_per_token(packed, scale, min_val, n):
    p, pp = _u8(packed)
    out = np.empty(n, dtype=np.float32)
    lib().orc_q2_dequant_per_token(pp, float(scale), float(min_val), out.ctypes.data_as(_f32p), n)
    return out


def q2_dequant_per_channel(packed, mins, scales):
    p, pp = _u8(packed)
    mn, mnp = _f(mins)
    sc, scp = _f(scales)
    out = np.empty(mn.size, dtype=np.float32)
    lib().orc_q2_dequant_per_channel(pp, mnp, scp, out.ctypes.data_as(_f32p), mn.size)
    return out


# ---------------------------------------------------------------- attention
def gqa_decode(q, k, v, nh, nkv, hd, seq_len, softcap=0.0) -> np.ndarray:
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    out = np.empty(nh * hd, dtype=np.float32)
    lib().orc_gqa_decode(qp, kp, vp, nh, nkv, hd, seq_len, softcap, out.ctypes.data_as(_f32p))
    return out


def gqa_decode_three_pass(q, k, v, nh, nkv, hd, seq_len) -> np.ndarray:
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    out = np.empty(nh * hd, dtype=np.float32)
    lib().orc_gqa_decode_three_pass(qp, kp, vp, nh, nkv, hd, seq_len, out.ctypes.data_as(_f32p))
    return out


def gqa_decode_batched(q, k, v, attend_len, nh, nkv, hd, n_q=1, softcap=0.0, threads=1) -> np.ndarray:
    """q [batch][n_q][nh*hd]; k, v [batch][slots][nkv*hd]; attend_len [batch] (of the LAST query)."""
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    batch = k.shape[0]
    al = np.ascontiguousarray(attend_len, dtype=np.int32)
    out = np.empty((batch, n_q, nh * hd), dtype=np.float32)
    seq_stride = k[0].size
    lib().orc_gqa_decode_batched(qp, kp, vp, batch, n_q, seq_stride, al.ctypes.data_as(_i32p), nh, nkv, hd,
                                 softcap, out.ctypes.data_as(_f32p), threads)
    return out


def gqa_decode_heads_mt(q, k, v, attend_len, nh, nkv, hd, threads) -> np.ndarray:
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    batch = k.shape[0]
    al = np.ascontiguousarray(attend_len, dtype=np.int32)
    out = np.empty((batch, nh * hd), dtype=np.float32)
    lib().orc_gqa_decode_heads_mt(qp, kp, vp, batch, k[0].size, al.ctypes.data_as(_i32p), nh, nkv, hd,
                                  out.ctypes.data_as(_f32p), threads)
    return out


def prefill(q, k, v, seq_len, nh, nkv, hd, softcap=0.0, window=0, row_start=0, row_step=1, threads=1):
    """One sequence.  q [S][nh*hd], k,v [S][nkv*hd] -> out [S][nh*hd]; rows that are not
    selected by (row_start, row_step) are NaN."""
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    out = np.full((seq_len, nh * hd), np.nan, dtype=np.float32)
    lib().orc_prefill(qp, kp, vp, seq_len, nh, nkv, hd, softcap, window, row_start, row_step,
                      out.ctypes.data_as(_f32p), threads)
    return out


def gqa_decode_partial(q, k, v, nh, nkv, hd, slot_begin, slot_end) -> np.ndarray:
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    out = np.empty((nh, hd + 2), dtype=np.float32)
    lib().orc_gqa_decode_partial(qp, kp, vp, nh, nkv, hd, slot_begin, slot_end, out.ctypes.data_as(_f32p))
    return out


def merge_partials(partials, nh, hd) -> np.ndarray:
    p, pp = _f(partials)
    n_parts = p.size // (nh * (hd + 2))
    out = np.empty(nh * hd, dtype=np.float32)
    lib().orc_merge_partials(pp, n_parts, nh, hd, out.ctypes.data_as(_f32p))
    return out


# ---------------------------------------------------------------- rotary position embedding
ROPE_TABLE_MAX_SEQ_LEN = 8192      # flare-core/src/model.rs:7171


def rope_table(head_dim, max_seq_len, theta, cap=ROPE_TABLE_MAX_SEQ_LEN):
    """RopeTable::new: (cos, sin), each [min(max_seq_len, cap)][head_dim // 2]."""
    n, half = min(max_seq_len, cap), head_dim // 2
    cos, sin = np.empty((n, half), np.float32), np.empty((n, half), np.float32)
    L = lib()
    L.orc_rope_table.restype = _sz
    L.orc_rope_table.argtypes = [_sz, _sz, C.c_float, _sz, _f32p, _f32p]
    got = L.orc_rope_table(head_dim, max_seq_len, theta, cap, cos.ctypes.data_as(_f32p), sin.ctypes.data_as(_f32p))
    assert got == n
    return cos, sin


def apply_rope(data, num_heads, head_dim, pos, theta) -> np.ndarray:
    d = np.array(data, dtype=np.float32).reshape(-1).copy()
    L = lib()
    L.orc_apply_rope.argtypes = [_f32p, _sz, _sz, _sz, C.c_float]
    L.orc_apply_rope(d.ctypes.data_as(_f32p), num_heads, head_dim, pos, theta)
    return d


def apply_rope_with_table(data, num_heads, head_dim, pos, theta, cos, sin) -> np.ndarray:
    d = np.array(data, dtype=np.float32).reshape(-1).copy()
    cos, cp = _f(cos)
    sin, sp = _f(sin)
    L = lib()
    L.orc_apply_rope_with_table.argtypes = [_f32p, _sz, _sz, _sz, C.c_float, _f32p, _f32p, _sz, _sz]
    L.orc_apply_rope_with_table(d.ctypes.data_as(_f32p), num_heads, head_dim, pos, theta, cp, sp, cos.shape[0], cos.shape[1] * 2)
    return d


# ---------------------------------------------------------------- Q8_0-weight matrix-vector product
def quantize_input_q8_0(x):
    """quantize_input_q8_0: f32 [n] -> (f32 scales [n/32], i8 quants [n])."""
    x, xp = _f(x)
    n = x.size
    assert n % 32 == 0
    scales, quants = np.empty(n // 32, np.float32), np.empty(n, np.int8)
    L = lib()
    L.orc_quantize_input_q8_0.argtypes = [_f32p, _sz, _f32p, C.POINTER(C.c_int8)]
    L.orc_quantize_input_q8_0(xp, n, scales.ctypes.data_as(_f32p), quants.ctypes.data_as(C.POINTER(C.c_int8)))
    return scales, quants


def matvec_q8_0(weight_blocks, x, rows) -> np.ndarray:
    """matvec_q8_0_preq_into on quantize_input_q8_0(x): weight_blocks is the Q8_0 block stream [rows][cols/32 x 34]."""
    w, wp = _u8(weight_blocks)
    scales, quants = quantize_input_q8_0(x)
    out = np.empty(rows, np.float32)
    L = lib()
    L.orc_matvec_q8_0_preq.argtypes = [_u8p, _f32p, C.POINTER(C.c_int8), _sz, _sz, _f32p]
    L.orc_matvec_q8_0_preq(wp, scales.ctypes.data_as(_f32p), quants.ctypes.data_as(C.POINTER(C.c_int8)), rows, scales.size,
                           out.ctypes.data_as(_f32p))
    return out


def matvec_q8_0_preq(weight_blocks, scales, quants, rows) -> np.ndarray:
    """matvec_q8_0_preq_into on an input that is already quantised."""
    w, wp = _u8(weight_blocks)
    scales = np.ascontiguousarray(scales, np.float32)
    quants = np.ascontiguousarray(quants, np.int8)
    out = np.empty(rows, np.float32)
    L = lib()
    L.orc_matvec_q8_0_preq.argtypes = [_u8p, _f32p, C.POINTER(C.c_int8), _sz, _sz, _f32p]
    L.orc_matvec_q8_0_preq(wp, scales.ctypes.data_as(_f32p), quants.ctypes.data_as(C.POINTER(C.c_int8)), rows, scales.size,
                           out.ctypes.data_as(_f32p))
    return out


# ---------------------------------------------------------------- the rest of a token's forward pass
def rmsnorm_quantize_q8_0(x, weight, eps):
    """rmsnorm_quantize_q8_0_into (model.rs:5581-5641): (f32 scales [n/32], i8 quants [n])."""
    x, xp = _f(x)
    weight, wp = _f(weight)
    n = x.size
    scales, quants = np.empty(n // 32, np.float32), np.empty(n, np.int8)
    L = lib()
    L.orc_rmsnorm_quantize_q8_0.argtypes = [_f32p, _f32p, C.c_float, _sz, _f32p, C.POINTER(C.c_int8)]
    L.orc_rmsnorm_quantize_q8_0(xp, wp, eps, n, scales.ctypes.data_as(_f32p), quants.ctypes.data_as(C.POINTER(C.c_int8)))
    return scales, quants


def rmsnorm(x, weight, eps) -> np.ndarray:
    """rmsnorm_into (model.rs:7456-7478)."""
    x, xp = _f(x)
    weight, wp = _f(weight)
    out = np.empty(x.size, np.float32)
    L = lib()
    L.orc_rmsnorm_into.argtypes = [_f32p, _f32p, C.c_float, _sz, _f32p]
    L.orc_rmsnorm_into(xp, wp, eps, x.size, out.ctypes.data_as(_f32p))
    return out


def silu_mul(gate, up) -> np.ndarray:
    """silu_mul_cpu (model.rs:7078-7099)."""
    gate, gp = _f(gate)
    up, up_p = _f(up)
    out = np.empty(gate.size, np.float32)
    L = lib()
    L.orc_silu_mul.argtypes = [_f32p, _f32p, _sz, _f32p]
    L.orc_silu_mul(gp, up_p, gate.size, out.ctypes.data_as(_f32p))
    return out


def matvec_f32(mat, vec, rows, cols) -> np.ndarray:
    mat, mp = _f(mat)
    vec, vp = _f(vec)
    out = np.empty(rows, np.float32)
    L = lib()
    L.orc_matvec_f32.argtypes = [_f32p, _f32p, _sz, _sz, _f32p]
    L.orc_matvec_f32(mp, vp, rows, cols, out.ctypes.data_as(_f32p))
    return out


def forward_token_q8(cfg, layers, output_norm, output_q8, output_f32, cos, sin, theta, k_cache, v_cache, length, x, pos,
                     store=None):
    """One token of Model::forward on the Q8_0 path (model.rs:1740-1790, 2010-2548) for one sequence.

    cfg: dict(hidden_dim, num_heads, num_kv_heads, head_dim, intermediate_dim, vocab_size, rms_norm_eps);
    layers: list of dict(attn_norm, qkv, wo, ffn_norm, gate_up, down) with Q8_0 block streams (uint8);
    k_cache / v_cache: per layer f32 arrays [max_seq][kv_dim], written at slot `length` (no ring wrap here);
    store: what the cache does to a row before attention reads it back (None: kept as f32; a Q8_0 cache:
    lambda r: dequant_q8_0(quantize_q8_0(r)));
    x: the token's embedding row.  Returns the logits; the caller advances `length`."""
    store = store or (lambda r: r)
    dim, nh, nkv, hd = cfg["hidden_dim"], cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    inter, eps = cfg["intermediate_dim"], cfg["rms_norm_eps"]
    q_dim, kv_dim = nh * hd, nkv * hd
    x = np.array(x, np.float32).copy()
    for li, lw in enumerate(layers):
        s, qn = rmsnorm_quantize_q8_0(x, lw["attn_norm"], eps)
        qkv = matvec_q8_0_preq(lw["qkv"], s, qn, q_dim + 2 * kv_dim)
        q = apply_rope_with_table(qkv[:q_dim], nh, hd, pos, theta, cos, sin)
        k = apply_rope_with_table(qkv[q_dim:q_dim + kv_dim], nkv, hd, pos, theta, cos, sin)
        k_cache[li][length] = store(k)
        v_cache[li][length] = store(qkv[q_dim + kv_dim:])
        attn = gqa_decode(q, k_cache[li], v_cache[li], nh, nkv, hd, length + 1)
        x = x + matvec_q8_0(lw["wo"], attn, dim)
        s, qn = rmsnorm_quantize_q8_0(x, lw["ffn_norm"], eps)
        gu = matvec_q8_0_preq(lw["gate_up"], s, qn, 2 * inter)
        hidden = silu_mul(gu[:inter], gu[inter:])
        x = x + matvec_q8_0(lw["down"], hidden, dim)
    normed = rmsnorm(x, output_norm, eps)
    if output_q8 is not None:
        return matvec_q8_0(output_q8, normed, cfg["vocab_size"])
    return matvec_f32(output_f32, normed, cfg["vocab_size"], dim)


# ---------------------------------------------------------------- caches
class KvCache:
    """flare-core/src/kv_cache.rs:431-546."""

    def __init__(self, num_layers, max_seq_len, num_kv_heads, head_dim):
        self.L = lib()
        self.h = C.c_void_p(self.L.orc_kv_new(num_layers, max_seq_len, num_kv_heads, head_dim))
        self.num_layers, self.max_seq_len = num_layers, max_seq_len
        self.num_kv_heads, self.head_dim = num_kv_heads, head_dim

    def __del__(self):
        if getattr(self, "h", None):
            self.L.orc_kv_free(self.h)
            self.h = None

    def write(self, layer, key, value):
        k, kp = _f(key)
        v, vp = _f(value)
        assert k.size == v.size == self.num_kv_heads * self.head_dim
        self.L.orc_kv_write(self.h, layer, kp, vp)

    def advance(self):
        self.L.orc_kv_advance(self.h)

    def len(self):
        return int(self.L.orc_kv_len(self.h))

    def is_empty(self):
        return self.len() == 0

    def position(self):
        return int(self.L.orc_kv_position(self.h))

    def attend_len(self):
        return int(self.L.orc_kv_attend_len(self.h))

    def truncate_to(self, n):
        self.L.orc_kv_truncate_to(self.h, n)

    def clear(self):
        self.L.orc_kv_clear(self.h)

    def _view(self, ptr):
        n = self.max_seq_len * self.num_kv_heads * self.head_dim
        return np.ctypeslib.as_array(ptr, shape=(n,))

    def keys(self, layer):
        return self._view(self.L.orc_kv_keys(self.h, layer))

    def values(self, layer):
        return self._view(self.L.orc_kv_values(self.h, layer))


class QuantizedKvCache:
    """flare-core/src/kv_cache.rs:35-323 (the reference's KIVI-style cache, quirks included)."""

    def __init__(self, num_layers, max_seq_len, num_kv_heads, head_dim):
        self.L = lib()
        self.h = C.c_void_p(self.L.orc_qkv_new(num_layers, max_seq_len, num_kv_heads, head_dim))
        self.num_layers, self.max_seq_len = num_layers, max_seq_len
        self.num_kv_heads, self.head_dim = num_kv_heads, head_dim
        self.kv = num_kv_heads * head_dim
        self.residual_len = min(32, max_seq_len)

    def __del__(self):
        if getattr(self, "h", None):
            self.L.orc_qkv_free(self.h)
            self.h = None

    def write(self, layer, key, value):
        k, kp = _f(key)
        v, vp = _f(value)
        assert k.size == v.size == self.kv
        self.L.orc_qkv_write(self.h, layer, kp, vp)

    def advance(self):
        self.L.orc_qkv_advance(self.h)

    def len(self):
        return int(self.L.orc_qkv_len(self.h))

    def is_empty(self):
        return self.len() == 0

    def position(self):
        return int(self.L.orc_qkv_position(self.h))

    def truncate_to(self, n):
        self.L.orc_qkv_truncate_to(self.h, n)

    def clear(self):
        self.L.orc_qkv_clear(self.h)

    def _dq(self, layer, want_values):
        out = np.empty(self.max_seq_len * self.kv, dtype=np.float32)
        self.L.orc_qkv_dequant(self.h, layer, want_values, out.ctypes.data_as(_f32p))
        return out

    def dequant_keys(self, layer):
        return self._dq(layer, 0)

    def dequant_values(self, layer):
        return self._dq(layer, 1)

    def plane(self, name, layer):
        ppt = (self.kv + 3) // 4
        shapes = {"key_packed": self.max_seq_len * ppt, "value_packed": self.max_seq_len * ppt,
                  "key_scales": self.kv, "key_mins": self.kv, "value_scales": self.max_seq_len,
                  "value_mins": self.max_seq_len, "residual_keys": self.residual_len * self.kv,
                  "residual_values": self.residual_len * self.kv}
        ptr = getattr(self.L, "orc_qkv_" + name)(self.h, layer)
        return np.ctypeslib.as_array(ptr, shape=(shapes[name],)).copy()


class G32Cache:
    """Group-32 KIVI cache of one layer of one sequence (no counterpart in the reference)."""

    def __init__(self, max_seq_len, kv_dim):
        assert max_seq_len % 32 == 0 and kv_dim % 32 == 0
        self.L = lib()
        self.h = C.c_void_p(self.L.orc_g32_new(max_seq_len, kv_dim))
        self.max_seq_len, self.kv = max_seq_len, kv_dim

    def __del__(self):
        if getattr(self, "h", None):
            self.L.orc_g32_free(self.h)
            self.h = None

    def write_advance(self, key, value):
        k, kp = _f(key)
        v, vp = _f(value)
        self.L.orc_g32_write_advance(self.h, kp, vp)

    def written(self):
        return int(self.L.orc_g32_written(self.h))

    def attend_len(self):
        return min(self.written(), self.max_seq_len)

    def dequant(self):
        k = np.empty((self.max_seq_len, self.kv), dtype=np.float32)
        v = np.empty((self.max_seq_len, self.kv), dtype=np.float32)
        self.L.orc_g32_dequant(self.h, k.ctypes.data_as(_f32p), v.ctypes.data_as(_f32p))
        return k, v

    def plane(self, name):
        ms, kv = self.max_seq_len, self.kv
        shapes = {"k_codes": ms * kv // 4, "v_codes": ms * kv // 4, "k_meta": ms // 32 * kv * 2,
                  "v_meta": ms * kv // 32 * 2, "res_k": 128 * kv, "res_v": 128 * kv}
        ptr = getattr(self.L, "orc_g32_" + name)(self.h)
        return np.ctypeslib.as_array(ptr, shape=(shapes[name],)).copy()
