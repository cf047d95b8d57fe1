"""flarellm_b200 — B200 attention engine for Flare, host side.

Everything here is a thin ctypes layer over ``libflare_attn.so`` (the C ABI declared in
``include/flare_attn.h``).  There is no CPU path: a missing library or a missing CUDA
device raises.

* ``Engine`` / ``KvCache``  — the rich interface (batch, quantised caches, verify, partials)
* ``CudaBackend``           — the attention hooks of flare-core's ``ComputeBackend`` trait
  (flare-core/src/model.rs:246-368), same names and argument meaning, batch 1, host f32.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# FLARE_ATTN_LIB selects another build of the same library (e.g. a variant under test)
LIB_PATH = os.environ.get("FLARE_ATTN_LIB") or os.path.join(_HERE, "libflare_attn.so")

(OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_OOM, ERR_CUDA, ERR_TIMEOUT, ERR_STATE, ERR_NCCL,
 ERR_BOUNDS) = range(9)
KV_F32, KV_Q8_0, KV_KIVI_REF, KV_KIVI_G32 = range(4)
DT_F32, DT_BF16 = 0, 1
(PLANE_K, PLANE_V, PLANE_K_Q, PLANE_V_Q, PLANE_K_SCALE, PLANE_V_SCALE, PLANE_K_MIN, PLANE_V_MIN,
 PLANE_K_RES, PLANE_V_RES) = range(10)

_STATUS_NAMES = {0: "OK", 1: "INVALID_ARG", 2: "UNSUPPORTED", 3: "OOM", 4: "CUDA", 5: "TIMEOUT", 6: "STATE", 7: "NCCL",
                 8: "BOUNDS"}
OP_NONE, OP_DECODE, OP_PREFILL = range(3)
PATH_NONE, PATH_GENERAL, PATH_Q8_TENSOR, PATH_KIVI_TENSOR, PATH_PREFILL_TENSOR = range(5)


class Stats(C.Structure):
    """flare_attn_stats of include/flare_attn.h."""
    _fields_ = [("calls", C.c_uint64), ("last_op", C.c_int32), ("last_path", C.c_int32),
                ("last_elapsed_us", C.c_double), ("last_bytes", C.c_double), ("last_flops", C.c_double),
                ("last_gbs", C.c_double), ("last_tflops", C.c_double), ("last_frac_of_peak", C.c_double),
                ("total_elapsed_us", C.c_double), ("total_bytes", C.c_double), ("total_flops", C.c_double)]


# every symbol include/flare_attn.h declares: (name, restype, argtypes)
_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t
_ip = C.POINTER(C.c_int)
_i64p = C.POINTER(C.c_int64)
SYMBOLS = [
    ("flare_attn_create", _i, [_i, C.POINTER(_vp)]),
    ("flare_attn_destroy", _i, [_vp]),
    ("flare_attn_set_stream", _i, [_vp, _vp]),
    ("flare_attn_sync", _i, [_vp]),
    ("flare_attn_last_error", C.c_char_p, [_vp]),
    ("flare_attn_launch_count", C.c_uint64, [_vp]),
    ("flare_attn_backend_name", C.c_char_p, []),
    ("flare_attn_selftest_wait_timeout", _i, [_vp]),
    ("flare_attn_enable_stats", _i, [_vp, _i]),
    ("flare_attn_set_peaks", _i, [_vp, C.c_double, C.c_double]),
    ("flare_attn_get_stats", _i, [_vp, C.POINTER(Stats)]),
    ("flare_kv_alloc", _i, [_vp, _i, _i, _i, _i, _i, _i, C.POINTER(_vp)]),
    ("flare_kv_free", _i, [_vp]),
    ("flare_kv_write_f32", _i, [_vp, _i, _i, _i64, _vp, _vp, _i]),
    ("flare_kv_append_f32", _i, [_vp, _i, _i, _i, _vp, _vp, _i]),
    ("flare_kv_write_step_f32", _i, [_vp, _i, _vp, _vp, _i]),
    ("flare_kv_set_rope_table", _i, [_vp, _vp, _vp, _i]),
    ("flare_kv_write_step_rope_f32", _i, [_vp, _i, _vp, _vp, _i64p, _i]),
    ("flare_rope_rows_f32", _i, [_vp, _vp, _i, _i, _i64p, _i]),
    ("flare_kv_advance", _i, [_vp, _i, _i]),
    ("flare_kv_get_state", _i, [_vp, _i, _i64p, _i64p]),
    ("flare_kv_set_state", _i, [_vp, _i, _i64, _i64]),
    ("flare_kv_truncate", _i, [_vp, _i, _i64]),
    ("flare_kv_clear", _i, [_vp, _i]),
    ("flare_kv_plane_bytes", _sz, [_vp, _i]),
    ("flare_kv_export_plane", _i, [_vp, _i, _i, _i, _vp, _sz, _i]),
    ("flare_kv_import_plane", _i, [_vp, _i, _i, _i, _vp, _sz, _i]),
    ("flare_kv_import_q8_0_blocks", _i, [_vp, _i, _i, _i, _i, _vp, _vp, _i]),
    ("flare_kv_export_q8_0_blocks", _i, [_vp, _i, _i, _i, _i, _vp, _vp, _i]),
    ("flare_kv_export_dequant", _i, [_vp, _i, _i, _vp, _vp, _i]),
    ("flare_decode_attn", _i, [_vp, _vp, _i, _i, _vp, _i, _ip, _f, _vp, _i]),
    ("flare_decode_step", _i, [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _i]),
    ("flare_decode_attn_noalloc", _i, [_vp, _vp, _i, _i, _vp, _i, _ip, _vp]),
    ("flare_decode_attn_noalloc_scratch_bytes", _sz, []),
    ("flare_decode_attn_partial", _i, [_vp, _vp, _i, _i, _vp, _i, _i, _i, _vp, _i]),
    ("flare_merge_partials", _i, [_vp, _vp, _i, _i, _i, _vp, _i]),
    ("flare_weight_upload_q8_0", _i, [_vp, _vp, _i, _i, C.POINTER(_vp)]),
    ("flare_weight_free", _i, [_vp]),
    ("flare_matvec_q8_0", _i, [_vp, _vp, _vp, _i, _vp, _i]),
    ("flare_model_create", _i, [_vp, _vp, _vp]),
    ("flare_model_set_layer", _i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    ("flare_model_set_output", _i, [_vp, _vp, _vp, _vp]),
    ("flare_model_free", _i, [_vp]),
    ("flare_forward_token", _i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    ("flare_attn_comm_unique_id", _i, [_vp]),
    ("flare_attn_comm_init", _i, [_vp, _vp, _i, _i]),
    ("flare_attn_comm_enable_direct", _i, [_vp, _i, _i]),
    ("flare_attn_comm_set_wait_ms", _i, [_vp, C.c_uint]),
    ("flare_attn_comm_info", _i, [_vp, _ip, _ip, _ip]),
    ("flare_attn_comm_probe_us", C.c_double, [_vp]),
    ("flare_attn_comm_destroy", _i, [_vp]),
    ("flare_decode_attn_splitkv_multi", _i, [_vp, _vp, _i, _i, _vp, _i, _vp, _i]),
    ("flare_attn_comm_selftest_missing_peer", _i, [_vp]),
    ("flare_gqa_attention_host", _i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp]),
    ("flare_prefill_attn", _i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _i, _i]),
    ("flare_backend_init_gpu_kv_cache", _i, [_vp, _i, _i, _i, _i]),
    ("flare_backend_init_gpu_kv_cache_dtype", _i, [_vp, _i, _i, _i, _i, _i]),
    ("flare_backend_gpu_kv_write", _i, [_vp, _i, _i64, _i, _i, _vp, _vp]),
    ("flare_backend_has_gpu_kv_cache", _i, [_vp]),
    ("flare_backend_gqa_from_gpu_cache", _i, [_vp, _vp, _i, _i, _i, _i, _i, _f, _vp]),
    ("flare_backend_kv", _vp, [_vp]),
]

_lib = None


class FlareError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"flare_attn status {status} ({_STATUS_NAMES.get(status, '?')}): {message}")
        self.status = status


def lib() -> C.CDLL:
    """Load libflare_attn.so and declare every entry point.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m flarellm_b200.build` "
                "(there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        for name, res, args in SYMBOLS:
            fn = getattr(L, name)          # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _ptr(a):
    """numpy array -> host pointer; int -> device pointer."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data
    return int(a)


class Engine:
    """One CUDA device + stream (flare_attn_ctx)."""

    def __init__(self, device: int = 0):
        self.L = lib()
        h = _vp()
        st = self.L.flare_attn_create(device, C.byref(h))
        if st != OK:
            raise FlareError(st, "flare_attn_create failed (is a CUDA device present?)")
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.L.flare_attn_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, st):
        if st != OK:
            raise FlareError(st, self.L.flare_attn_last_error(self.h).decode())

    def set_stream(self, cuda_stream):
        """Run on a caller-owned stream.  A handle of 0 is CUDA's legacy default stream (what
        ``torch.cuda.current_stream().cuda_stream`` is unless a side stream is current); the C ABI
        reserves NULL for "back to the context's own stream", so 0 is passed as cudaStreamLegacy."""
        CUDA_STREAM_LEGACY = 1
        self.check(self.L.flare_attn_set_stream(self.h, cuda_stream if cuda_stream else CUDA_STREAM_LEGACY))

    def use_own_stream(self):
        self.check(self.L.flare_attn_set_stream(self.h, None))

    def sync(self):
        self.check(self.L.flare_attn_sync(self.h))

    def launch_count(self) -> int:
        return int(self.L.flare_attn_launch_count(self.h))

    def selftest_wait_timeout(self) -> int:
        """Runs the kernels' give-up path once (a bounded wait that nothing satisfies); returns the status,
        ``ERR_TIMEOUT`` when the path works."""
        return int(self.L.flare_attn_selftest_wait_timeout(self.h))

    def enable_stats(self, on=True):
        self.check(self.L.flare_attn_enable_stats(self.h, int(bool(on))))

    def set_peaks(self, hbm_gbs, tensor_tflops):
        self.check(self.L.flare_attn_set_peaks(self.h, float(hbm_gbs), float(tensor_tflops)))

    def stats(self) -> Stats:
        """Measurements of the attention calls made while stats were enabled (waits for the last one)."""
        st = Stats()
        self.check(self.L.flare_attn_get_stats(self.h, C.byref(st)))
        return st

    def last_path(self) -> int:
        """Which kernel family served the most recent attention call (PATH_*)."""
        return int(self.stats().last_path)

    def kv_alloc(self, num_layers, batch, max_seq_len, num_kv_heads, head_dim, dtype=KV_F32) -> "KvCache":
        return KvCache(self, num_layers, batch, max_seq_len, num_kv_heads, head_dim, dtype)

    # ---- attention -------------------------------------------------------------------------
    def decode(self, kv: "KvCache", layer, num_heads, q, n_q=1, attend_len=None, softcap=0.0, out=None):
        """q: host ndarray [batch][n_q][num_heads][head_dim] f32, or a device pointer (int) with
        ``out`` a device pointer as well."""
        on_device = not isinstance(q, np.ndarray)
        if not on_device:
            q = np.ascontiguousarray(q, dtype=np.float32)
            assert q.size == kv.batch * n_q * num_heads * kv.head_dim
            if out is None:
                out = np.empty((kv.batch, n_q, num_heads, kv.head_dim), dtype=np.float32)
        al = None
        if attend_len is not None:
            al_arr = np.ascontiguousarray(attend_len, dtype=np.int32)
            assert al_arr.size == kv.batch
            al = al_arr.ctypes.data_as(_ip)
        self.check(self.L.flare_decode_attn(self.h, kv.h, layer, num_heads, _ptr(q), n_q, al, softcap, _ptr(out),
                                            int(on_device)))
        return out

    def decode_step(self, kv: "KvCache", layer, num_heads, key, value, q, out=None, on_device=None):
        """flare_decode_step: store the new K/V row of every sequence, then attend.  Host ndarrays
        (``out`` optional), device pointers (``out`` required), or — with ``on_device=False`` — plain host addresses
        (ints) of buffers the caller keeps alive, resolved once outside a loop the way a Rust caller's slices are:
        converting four ndarrays to pointers costs about 5 us per call in Python."""
        if on_device is not None and not isinstance(q, np.ndarray):
            rc = self.L.flare_decode_step(self.h, kv.h, layer, num_heads, key, value, q, out, 1 if on_device else 0)
            if rc:
                self.check(rc)
            return out
        on_device = not isinstance(q, np.ndarray)
        if not on_device:
            key, value, q = (a if (a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]) else
                             np.ascontiguousarray(a, dtype=np.float32) for a in (key, value, q))
            if out is None:
                out = np.empty((kv.batch, 1, num_heads, kv.head_dim), dtype=np.float32)
        self.check(self.L.flare_decode_step(self.h, kv.h, layer, num_heads, _ptr(key), _ptr(value), _ptr(q), _ptr(out),
                                            int(on_device)))
        return out

    def decode_noalloc(self, kv: "KvCache", layer, num_heads, q_dev: int, out_dev: int, n_q=1, attend_len=None):
        """flare_decode_attn_noalloc: device pointers in and out, workspace inside the library,
        no device allocation during the call."""
        al = None
        if attend_len is not None:
            al_arr = np.ascontiguousarray(attend_len, dtype=np.int32)
            assert al_arr.size == kv.batch
            al = al_arr.ctypes.data_as(_ip)
        self.check(self.L.flare_decode_attn_noalloc(self.h, kv.h, layer, num_heads, int(q_dev), n_q, al, int(out_dev)))

    def decode_partial(self, kv, layer, num_heads, q, slot_begin, slot_end, n_q=1, out=None):
        on_device = not isinstance(q, np.ndarray)
        if not on_device:
            q = np.ascontiguousarray(q, dtype=np.float32)
            if out is None:
                out = np.empty((kv.batch, n_q, num_heads, kv.head_dim + 2), dtype=np.float32)
        self.check(self.L.flare_decode_attn_partial(self.h, kv.h, layer, num_heads, _ptr(q), n_q, slot_begin,
                                                    slot_end, _ptr(out), int(on_device)))
        return out

    def merge_partials(self, partials, n_parts, rows, head_dim, out=None):
        on_device = not isinstance(partials, np.ndarray)
        if not on_device:
            partials = np.ascontiguousarray(partials, dtype=np.float32)
            assert partials.size == n_parts * rows * (head_dim + 2)
            if out is None:
                out = np.empty((rows, head_dim), dtype=np.float32)
        self.check(self.L.flare_merge_partials(self.h, _ptr(partials), n_parts, rows, head_dim, _ptr(out),
                                               int(on_device)))
        return out

    # ---- Q8_0-weight projections -----------------------------------------------------------------
    def model_create(self, hidden_dim, num_heads, num_kv_heads, head_dim, intermediate_dim, vocab_size, num_layers,
                     rms_norm_eps) -> "ResidentModel":
        return ResidentModel(self, hidden_dim, num_heads, num_kv_heads, head_dim, intermediate_dim, vocab_size, num_layers,
                             rms_norm_eps)

    def weight_upload_q8_0(self, blocks, rows: int, cols: int) -> "Q8Weight":
        return Q8Weight(self, blocks, rows, cols)

    def matvec_q8_0(self, w: "Q8Weight", x, out=None):
        """out[b][r] = row r of w . x[b], bit-identical to flare-core's matvec_q8_0_preq_into.  x: host ndarray
        [batch][cols] or a device pointer (then `batch` is taken from ``out`` = (pointer, batch))."""
        on_device = not isinstance(x, np.ndarray)
        if on_device:
            out_ptr, batch = out
        else:
            x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, w.cols)
            batch = x.shape[0]
            if out is None:
                out = np.empty((batch, w.rows), dtype=np.float32)
            out_ptr = _ptr(out)
        self.check(self.L.flare_matvec_q8_0(self.h, w.h, _ptr(x), batch, out_ptr, int(on_device)))
        return out

    # ---- one sequence over several GPUs ------------------------------------------------------
    @staticmethod
    def comm_unique_id() -> bytes:
        """128 bytes that rank 0 hands to the other ranks (flare_attn_comm_unique_id)."""
        buf = C.create_string_buffer(128)
        st = lib().flare_attn_comm_unique_id(buf)
        if st != OK:
            raise FlareError(st, "flare_attn_comm_unique_id failed (is libnccl.so.2 loadable?)")
        return buf.raw

    def comm_init(self, uid, rank: int, world: int):
        self.check(self.L.flare_attn_comm_init(self.h, C.c_char_p(uid) if uid else None, rank, world))

    def comm_enable_direct(self, max_rows: int, head_dim: int):
        self.check(self.L.flare_attn_comm_enable_direct(self.h, max_rows, head_dim))

    def comm_info(self):
        """(rank, world, direct) of the context's communicator."""
        r, w, d = C.c_int(), C.c_int(), C.c_int()
        self.check(self.L.flare_attn_comm_info(self.h, C.byref(r), C.byref(w), C.byref(d)))
        return int(r.value), int(w.value), bool(d.value)

    def comm_probe_us(self) -> float:
        return float(self.L.flare_attn_comm_probe_us(self.h))

    def comm_set_wait_ms(self, ms: int):
        self.check(self.L.flare_attn_comm_set_wait_ms(self.h, ms))

    def comm_destroy(self):
        self.check(self.L.flare_attn_comm_destroy(self.h))

    def comm_selftest_missing_peer(self) -> int:
        return int(self.L.flare_attn_comm_selftest_missing_peer(self.h))

    def decode_splitkv_multi(self, kv: "KvCache", layer, num_heads, q, n_local_slots, out=None):
        """flare_decode_attn_splitkv_multi: this rank's slots 0..n_local_slots-1, merged with every other rank's."""
        on_device = not isinstance(q, np.ndarray)
        if not on_device:
            q = np.ascontiguousarray(q, dtype=np.float32)
            if out is None:
                out = np.empty((kv.batch, 1, num_heads, kv.head_dim), dtype=np.float32)
        self.check(self.L.flare_decode_attn_splitkv_multi(self.h, kv.h, layer, num_heads, _ptr(q), n_local_slots,
                                                          _ptr(out), int(on_device)))
        return out

    def gqa_attention_host(self, q, k_cache, v_cache, num_heads, num_kv_heads, head_dim, seq_len, softcap=0.0):
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k_cache, dtype=np.float32)
        v = np.ascontiguousarray(v_cache, dtype=np.float32)
        out = np.empty(num_heads * head_dim, dtype=np.float32)
        self.check(self.L.flare_gqa_attention_host(self.h, _ptr(q), _ptr(k), _ptr(v), num_heads, num_kv_heads,
                                                   head_dim, seq_len, softcap, _ptr(out)))
        return out

    def prefill(self, q, k, v, batch, seq_len, num_heads, num_kv_heads, head_dim, window=0, softcap=0.0,
                in_dtype=DT_F32, out_dtype=DT_F32, out=None):
        """Host: q/k/v ndarrays (float32, or uint16 holding bf16 bits).  Device: pointers (int)."""
        on_device = not isinstance(q, np.ndarray)
        if not on_device:
            want = np.float32 if in_dtype == DT_F32 else np.uint16
            q, k, v = (np.ascontiguousarray(a, dtype=want) for a in (q, k, v))
            if out is None:
                out = np.empty((batch, seq_len, num_heads, head_dim),
                               dtype=np.float32 if out_dtype == DT_F32 else np.uint16)
        self.check(self.L.flare_prefill_attn(self.h, _ptr(q), _ptr(k), _ptr(v), in_dtype, batch, seq_len, num_heads,
                                             num_kv_heads, head_dim, window, softcap, _ptr(out), out_dtype,
                                             int(on_device)))
        return out


class Q8Weight:
    """A Q8_0 weight matrix on the device (flare_weight)."""

    def __init__(self, eng: Engine, blocks, rows: int, cols: int):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        assert blocks.size == rows * (cols // 32) * 34
        self.eng, self.L, self.rows, self.cols = eng, eng.L, rows, cols
        h = _vp()
        eng.check(self.L.flare_weight_upload_q8_0(eng.h, _ptr(blocks), rows, cols, C.byref(h)))
        self.h = h

    def free(self):
        if getattr(self, "h", None) and getattr(self.eng, "h", None):
            self.L.flare_weight_free(self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class ModelConfig(C.Structure):
    _fields_ = [("hidden_dim", C.c_int), ("num_heads", C.c_int), ("num_kv_heads", C.c_int), ("head_dim", C.c_int),
                ("intermediate_dim", C.c_int), ("vocab_size", C.c_int), ("num_layers", C.c_int), ("rms_norm_eps", C.c_float)]


class ResidentModel:
    """Weights of a Llama-style model with Q8_0 matrices on the device (flare_model), and the single-token forward
    pass that stays there: the counterpart of WebGpuBackend::upload_weights_to_gpu + forward_single_token_gpu
    (flare-gpu/src/backend.rs:4010-4375), computing what Model::forward computes on its Q8_0 path."""

    def __init__(self, eng: Engine, hidden_dim, num_heads, num_kv_heads, head_dim, intermediate_dim, vocab_size, num_layers,
                 rms_norm_eps):
        self.eng, self.L = eng, eng.L
        self.cfg = ModelConfig(hidden_dim, num_heads, num_kv_heads, head_dim, intermediate_dim, vocab_size, num_layers,
                               rms_norm_eps)
        h = _vp()
        eng.check(self.L.flare_model_create(eng.h, C.byref(self.cfg), C.byref(h)))
        self.h = h

    def set_layer(self, layer, attn_norm, qkv, wo, ffn_norm, gate_up, down):
        """Norms: f32 [hidden_dim]; matrices: Q8_0 block streams (uint8), qkv = wq, wk, wv stacked by rows, gate_up =
        w_gate, w_up stacked by rows."""
        c = self.cfg
        q_dim, kv_dim = c.num_heads * c.head_dim, c.num_kv_heads * c.head_dim
        f = lambda a: np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
        u = lambda a, rows, cols: self._blocks(a, rows, cols)
        an, fn = f(attn_norm), f(ffn_norm)
        assert an.size == c.hidden_dim and fn.size == c.hidden_dim
        mats = [u(qkv, q_dim + 2 * kv_dim, c.hidden_dim), u(wo, c.hidden_dim, q_dim),
                u(gate_up, 2 * c.intermediate_dim, c.hidden_dim), u(down, c.hidden_dim, c.intermediate_dim)]
        self.eng.check(self.L.flare_model_set_layer(self.h, layer, _ptr(an), _ptr(mats[0]), _ptr(mats[1]), _ptr(fn),
                                                    _ptr(mats[2]), _ptr(mats[3])))

    @staticmethod
    def _blocks(a, rows, cols):
        a = np.ascontiguousarray(a, dtype=np.uint8).reshape(-1)
        assert a.size == rows * (cols // 32) * 34, (a.size, rows, cols)
        return a

    def set_output(self, output_norm, output_q8=None, output_f32=None):
        c = self.cfg
        on = np.ascontiguousarray(output_norm, dtype=np.float32).reshape(-1)
        assert on.size == c.hidden_dim and (output_q8 is None) != (output_f32 is None)
        q8 = None if output_q8 is None else self._blocks(output_q8, c.vocab_size, c.hidden_dim)
        f32 = None if output_f32 is None else np.ascontiguousarray(output_f32, dtype=np.float32).reshape(-1)
        assert f32 is None or f32.size == c.vocab_size * c.hidden_dim
        self.eng.check(self.L.flare_model_set_output(self.h, _ptr(on), None if q8 is None else _ptr(q8),
                                                     None if f32 is None else _ptr(f32)))

    def forward(self, kv: "KvCache", token_embed, positions) -> np.ndarray:
        """One token per sequence of ``kv``: token_embed [batch][hidden_dim], positions [batch] -> logits
        [batch][vocab_size].  Writes every layer's K/V row and advances the cache by one (Model::forward)."""
        x = np.ascontiguousarray(token_embed, dtype=np.float32).reshape(-1, self.cfg.hidden_dim)
        pos = np.ascontiguousarray(positions, dtype=np.int64).reshape(-1)
        assert x.shape[0] == kv.batch == pos.size
        logits = np.empty((kv.batch, self.cfg.vocab_size), dtype=np.float32)
        self.eng.check(self.L.flare_forward_token(self.eng.h, self.h, kv.h, _ptr(x), _ptr(pos), _ptr(logits)))
        return logits

    def free(self):
        if getattr(self, "h", None) and getattr(self.eng, "h", None):
            self.L.flare_model_free(self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class KvCache:
    """Device ring-buffer KV cache for ``batch`` sequences (flare_kv)."""

    def __init__(self, eng: Engine, num_layers, batch, max_seq_len, num_kv_heads, head_dim, dtype):
        self.eng, self.L = eng, eng.L
        h = _vp()
        eng.check(self.L.flare_kv_alloc(eng.h, num_layers, batch, max_seq_len, num_kv_heads, head_dim, dtype,
                                        C.byref(h)))
        self.h = h
        self.num_layers, self.batch, self.max_seq_len = num_layers, batch, max_seq_len
        self.num_kv_heads, self.head_dim, self.dtype = num_kv_heads, head_dim, dtype
        self.kv_dim = num_kv_heads * head_dim
        self._owned = True

    def free(self):
        if getattr(self, "h", None) and self._owned and getattr(self.eng, "h", None):
            self.L.flare_kv_free(self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def write(self, layer, seq, abs_position, key, value):
        on_device = not isinstance(key, np.ndarray)
        if not on_device:
            key = np.ascontiguousarray(key, dtype=np.float32)
            value = np.ascontiguousarray(value, dtype=np.float32)
            assert key.size == value.size == self.kv_dim
        self.eng.check(self.L.flare_kv_write_f32(self.h, layer, seq, abs_position, _ptr(key), _ptr(value),
                                                 int(on_device)))

    def append(self, layer, seq, key, value, n_rows=None):
        on_device = not isinstance(key, np.ndarray)
        if not on_device:
            key = np.ascontiguousarray(key, dtype=np.float32)
            value = np.ascontiguousarray(value, dtype=np.float32)
            n_rows = key.size // self.kv_dim
            assert key.size == value.size == n_rows * self.kv_dim
        self.eng.check(self.L.flare_kv_append_f32(self.h, layer, seq, n_rows, _ptr(key), _ptr(value), int(on_device)))

    def write_step(self, layer, key, value):
        """Row b of key/value [batch][kv_dim] -> the current ring position of sequence b."""
        on_device = not isinstance(key, np.ndarray)
        if not on_device:
            key = np.ascontiguousarray(key, dtype=np.float32)
            value = np.ascontiguousarray(value, dtype=np.float32)
            assert key.size == value.size == self.batch * self.kv_dim
        self.eng.check(self.L.flare_kv_write_step_f32(self.h, layer, _ptr(key), _ptr(value), int(on_device)))

    def set_rope_table(self, cos, sin):
        """The caller's RopeTable: cos, sin [table_len][head_dim // 2] f32."""
        cos = np.ascontiguousarray(cos, dtype=np.float32)
        sin = np.ascontiguousarray(sin, dtype=np.float32)
        assert cos.shape == sin.shape and cos.shape[1] == self.head_dim // 2
        self.eng.check(self.L.flare_kv_set_rope_table(self.h, _ptr(cos), _ptr(sin), cos.shape[0]))

    def write_step_rope(self, layer, key, value, positions):
        """write_step on key rows that are still to be rotated for ``positions`` [batch]."""
        on_device = not isinstance(key, np.ndarray)
        if not on_device:
            key = np.ascontiguousarray(key, dtype=np.float32)
            value = np.ascontiguousarray(value, dtype=np.float32)
            assert key.size == value.size == self.batch * self.kv_dim
        pos = np.ascontiguousarray(positions, dtype=np.int64)
        assert pos.size == self.batch
        self.eng.check(self.L.flare_kv_write_step_rope_f32(self.h, layer, _ptr(key), _ptr(value),
                                                           pos.ctypes.data_as(_i64p), int(on_device)))

    def rope_rows(self, rows, num_heads, positions):
        """Rotate [n_rows][num_heads][head_dim] in place (host ndarray, or a device pointer)."""
        pos = np.ascontiguousarray(positions, dtype=np.int64)
        on_device = not isinstance(rows, np.ndarray)
        if not on_device:
            assert rows.dtype == np.float32 and rows.flags["C_CONTIGUOUS"] and rows.size == pos.size * num_heads * self.head_dim
        self.eng.check(self.L.flare_rope_rows_f32(self.h, _ptr(rows), pos.size, num_heads, pos.ctypes.data_as(_i64p),
                                                  int(on_device)))
        return rows

    def advance(self, seq=-1, n=1):
        self.eng.check(self.L.flare_kv_advance(self.h, seq, n))

    def state(self, seq=0):
        p, l = C.c_int64(), C.c_int64()
        self.eng.check(self.L.flare_kv_get_state(self.h, seq, C.byref(p), C.byref(l)))
        return int(p.value), int(l.value)

    def set_state(self, seq, position, length):
        self.eng.check(self.L.flare_kv_set_state(self.h, seq, position, length))

    def len(self, seq=0):
        return self.state(seq)[1]

    def position(self, seq=0):
        return self.state(seq)[0]

    def truncate(self, seq, target_len):
        self.eng.check(self.L.flare_kv_truncate(self.h, seq, target_len))

    def clear(self, seq=-1):
        self.eng.check(self.L.flare_kv_clear(self.h, seq))

    def plane_bytes(self, plane) -> int:
        return int(self.L.flare_kv_plane_bytes(self.h, plane))

    def export_plane(self, layer, seq, plane, dtype=np.uint8) -> np.ndarray:
        n = self.plane_bytes(plane)
        out = np.empty(n, dtype=np.uint8)
        self.eng.check(self.L.flare_kv_export_plane(self.h, layer, seq, plane, _ptr(out), n, 0))
        return out.view(dtype)

    def import_plane(self, layer, seq, plane, data):
        on_device = not isinstance(data, np.ndarray)
        if on_device:
            n = self.plane_bytes(plane)
        else:
            data = np.ascontiguousarray(data)
            n = data.nbytes
        self.eng.check(self.L.flare_kv_import_plane(self.h, layer, seq, plane, _ptr(data), n, int(on_device)))

    def import_q8_0_blocks(self, layer, seq, first_slot, k_blocks, v_blocks):
        k_blocks = np.ascontiguousarray(k_blocks, dtype=np.uint8)
        v_blocks = np.ascontiguousarray(v_blocks, dtype=np.uint8)
        n_slots = k_blocks.size // (self.kv_dim // 32 * 34)
        self.eng.check(self.L.flare_kv_import_q8_0_blocks(self.h, layer, seq, first_slot, n_slots, _ptr(k_blocks),
                                                          _ptr(v_blocks), 0))

    def export_q8_0_blocks(self, layer, seq, first_slot, n_slots):
        n = n_slots * (self.kv_dim // 32 * 34)
        kb, vb = np.empty(n, dtype=np.uint8), np.empty(n, dtype=np.uint8)
        self.eng.check(self.L.flare_kv_export_q8_0_blocks(self.h, layer, seq, first_slot, n_slots, _ptr(kb), _ptr(vb), 0))
        return kb, vb

    def export_dequant(self, layer, seq):
        k = np.empty((self.max_seq_len, self.kv_dim), dtype=np.float32)
        v = np.empty((self.max_seq_len, self.kv_dim), dtype=np.float32)
        self.eng.check(self.L.flare_kv_export_dequant(self.h, layer, seq, _ptr(k), _ptr(v), 0))
        return k, v


class CudaBackend:
    """The attention hooks of flare-core's ``ComputeBackend`` (flare-core/src/model.rs:246-368),
    as a Rust ``impl ComputeBackend for CudaBackend`` would forward them.  The trait's only
    error channel is a panic; here a non-zero status raises ``FlareError``."""

    def __init__(self, device: int = 0):
        self.eng = Engine(device)
        self.L = self.eng.L

    def name(self) -> str:
        return self.L.flare_attn_backend_name().decode()

    def init_gpu_kv_cache(self, num_layers, max_seq_len, num_kv_heads, head_dim, kv_dtype=KV_F32):
        self.eng.check(self.L.flare_backend_init_gpu_kv_cache_dtype(self.eng.h, num_layers, max_seq_len, num_kv_heads,
                                                                    head_dim, kv_dtype))

    def gpu_kv_write(self, layer, position, num_kv_heads, head_dim, key, value):
        key = np.ascontiguousarray(key, dtype=np.float32)
        value = np.ascontiguousarray(value, dtype=np.float32)
        self.eng.check(self.L.flare_backend_gpu_kv_write(self.eng.h, layer, position, num_kv_heads, head_dim,
                                                         _ptr(key), _ptr(value)))

    def has_gpu_kv_cache(self) -> bool:
        return bool(self.L.flare_backend_has_gpu_kv_cache(self.eng.h))

    def grouped_query_attention_from_gpu_cache(self, q, layer, num_heads, num_kv_heads, head_dim, seq_len,
                                               attn_softcap=0.0) -> np.ndarray:
        q = np.ascontiguousarray(q, dtype=np.float32)
        out = np.empty(num_heads * head_dim, dtype=np.float32)
        self.eng.check(self.L.flare_backend_gqa_from_gpu_cache(self.eng.h, _ptr(q), layer, num_heads, num_kv_heads,
                                                               head_dim, seq_len, attn_softcap, _ptr(out)))
        return out

    def grouped_query_attention(self, q, k_cache, v_cache, num_heads, num_kv_heads, head_dim, seq_len,
                                attn_softcap=0.0) -> np.ndarray:
        return self.eng.gqa_attention_host(q, k_cache, v_cache, num_heads, num_kv_heads, head_dim, seq_len,
                                           attn_softcap)

    def prefill_attention_gpu(self, q, k, v, seq_len, num_heads, num_kv_heads, head_dim, attn_softcap=0.0):
        out = self.eng.prefill(q, k, v, 1, seq_len, num_heads, num_kv_heads, head_dim, softcap=attn_softcap)
        return out.reshape(-1)

    def advance_kv(self, n=1):
        """KvCache::advance for the context-owned cache (the Rust side calls flare_kv_advance on
        flare_backend_kv() where Model advances its CPU cache, flare-core/src/model.rs:2547)."""
        self.eng.check(self.L.flare_kv_advance(self.L.flare_backend_kv(self.eng.h), 0, n))


# ---------------------------------------------------------------------------------------------
# Speculative verify, the host-side loop (flare-core/src/generate.rs:244-306, 314-405).
#
# `model` is whatever runs the layers around attention for the caller; it provides
#   num_layers, num_heads
#   embed(tokens) -> x [n][d]              qkv(layer, x) -> (q [n][nh*hd], k [n][kv_dim], v [n][kv_dim])  (post-RoPE)
#   post(layer, x, attn [n][nh*hd]) -> x   greedy(x) -> n token ids
# The cache holds one sequence (the reference's Generator is single-sequence).
# ---------------------------------------------------------------------------------------------
def forward_token(eng: Engine, kv: KvCache, model, token: int) -> int:
    """One decode step the way Model::forward orders it (flare-core/src/model.rs:2186-2247, 2547): per layer
    write the token's K/V row at the current position, attend over length + 1 slots; then advance.  Returns the
    greedy next token (forward_greedy)."""
    pos = kv.len(0)
    x = np.asarray(model.embed([token]), dtype=np.float32)
    for layer in range(model.num_layers):
        q, k, v = model.qkv(layer, x)
        kv.write(layer, 0, pos, k[0], v[0])
        attn = eng.decode(kv, layer, model.num_heads, np.ascontiguousarray(q, dtype=np.float32).reshape(1, 1, model.num_heads, kv.head_dim))
        x = model.post(layer, x, attn.reshape(1, -1))
    kv.advance(0, 1)
    return int(model.greedy(x)[0])


def verify_drafts_sequential(eng: Engine, kv: KvCache, model, last_token: int, drafts) -> list:
    """The reference's loop as it stands (generate.rs:258-303): one full forward per draft token, accept while the
    verified token equals the draft, accept the correcting token at the first mismatch and stop."""
    accepted, last = [], last_token
    for draft in drafts:
        verified = forward_token(eng, kv, model, last)
        accepted.append(verified)
        last = verified
        if verified != draft:
            break
    return accepted


def verify_drafts(eng: Engine, kv: KvCache, model, last_token: int, drafts) -> list:
    """The same verification with ONE attention call per layer: the K/V rows of all n forward inputs (the last
    accepted token and the first n - 1 drafts) are written at the next n positions, a single n-query call attends
    them causally (query i sees length + i + 1 slots), the matching prefix plus the correcting token is accepted
    and the cache is rolled back to what the sequential loop would have kept (Model::truncate_kv_cache,
    flare-core/src/model.rs:4835-4840)."""
    drafts = list(drafts)
    n = len(drafts)
    if n == 0:
        return []
    base = kv.len(0)
    if base + n > kv.max_seq_len:
        raise ValueError("the drafts do not fit in the ring: verify them one by one")
    x = np.asarray(model.embed([last_token] + drafts[:-1]), dtype=np.float32)
    for layer in range(model.num_layers):
        q, k, v = model.qkv(layer, x)
        for i in range(n):
            kv.write(layer, 0, base + i, k[i], v[i])
        attn = eng.decode(kv, layer, model.num_heads,
                          np.ascontiguousarray(q, dtype=np.float32).reshape(1, n, model.num_heads, kv.head_dim), n_q=n)
        x = model.post(layer, x, attn.reshape(n, -1))
    verified = [int(t) for t in model.greedy(x)]
    accepted = []
    for i in range(n):
        accepted.append(verified[i])
        if verified[i] != drafts[i]:
            break
    kv.advance(0, n)
    kv.truncate(0, base + len(accepted))
    return accepted
