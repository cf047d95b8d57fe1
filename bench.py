#!/usr/bin/env python
"""Attention benchmark: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--case NAME]

Headline workload (N GPUs, one process per GPU, weak scaling, no collective): the Llama-3.2-1B-shaped
Q8_0 decode of BASELINE.json configs[1] at batch 32 on every GPU — 32 query / 8 KV heads, head_dim 64,
context 4096, 16 layers.  One step = one new token for every sequence = 16 attention calls (one per
layer), each streaming that layer's whole K/V cache once.

  value     tokens/s of the whole job (all ranks), inputs resident in HBM, CUDA-event timed: the median of
            `repeats.n` timed regions of exactly K steps each (every region bracketed by a barrier and a
            device synchronisation, the maximum over ranks taken per region); min and max beside it
  e2e       the same through the host-buffer C-ABI call a batched ComputeBackend makes per layer
            (flare_decode_step: new K/V rows and q host -> device, store, attend, output device -> host),
            page-locked host buffers
  roofline  algorithmic KV bytes of one layer call / its average device time, against the measured HBM
            copy bandwidth; `traffic` = DRAM bytes of one launch from the ncu capture recorded in
            profiles/ncu_traffic.json (null when that file has no entry for the kernel)
  cpu_baseline  the CPU oracle (a restatement of flare-core's scalar attention) on a bounded sample
  cases     the other configurations of BASELINE.json, each with its own value, roofline, clocks and a
            parity check against the oracle: prefill (S 4096 x batch 4, bf16), prefill_window (S 8192,
            window 4096), kivi (2-bit group-32, ctx 32768 x batch 16), longctx (one sequence of 131072 slots,
            the slot range split over the N ranks and merged through the library's multi-GPU call), f32
            (the reference's own CPU-runnable shape: latency)

`--case NAME` runs that case alone and prints its record (used for profiler captures of one kernel).
Synthetic data: seeded N(0,1) K/V quantised on the device, q ~ N(0,1)/8.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NH, NKV, HD, CTX, LAYERS, BATCH = 32, 8, 64, 4096, 16, 32
KV_DIM = NKV * HD
ROW_BYTES = KV_DIM + KV_DIM // 32 * 2                 # 544: the Q8_0 bytes of one K (or V) row
LAYER_BYTES = BATCH * CTX * 2 * ROW_BYTES             # algorithmic bytes of one layer call
WORKLOAD = "llama-3.2-1b-shaped Q8_0 decode attention: 32q/8kv heads, head_dim 64, ctx 4096, batch 32/GPU, 16 layers"
DTYPE = "q8_0 kv; s8 (scores) and f16 (output) mma; s32 / f32 accumulate"


def workload_config(world, layers=LAYERS, batch=BATCH):
    """The `config` object, the same for this arm and the reference arm."""
    w = WORKLOAD if (layers, batch) == (LAYERS, BATCH) else f"{WORKLOAD} [reduced: batch {batch}, {layers} layers]"
    return {"workload": w, "kv_cache": "Q8_0 (int8 + f16 scale per 32)",
            "l2": "inputs larger than L2: %.2f GB of KV per step" % (layers * batch * CTX * 2 * ROW_BYTES / 1e9),
            "parallelism": f"{world} x independent batch-{batch} shards, no collective"}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def ncu_traffic(key):
    """DRAM bytes per launch of a kernel from the committed ncu summary data, or (None, reason)."""
    p = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        rec = json.load(open(p)).get(key)
    except Exception:
        rec = None
    if not rec:
        return None, f"no ncu capture recorded for '{key}' in profiles/ncu_traffic.json"
    return float(rec["dram_bytes_per_launch"]), rec.get("source", "profiles/ncu_traffic.json")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.marks = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def window(self, t0, t1):
        """Summary of the samples taken between two time.perf_counter() readings."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, r in list(self.rows):
            if t < t0 or t > t1 + 0.06:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()


# --------------------------------------------------------------------------------------------
# the reference arm: flare-core's CPU attention for this path on the host cores
# --------------------------------------------------------------------------------------------
def cpu_attention_sample(threads: int, seqs: int, repeats: int):
    """Time the CPU oracle on `seqs` sequences of one layer (Q8_0 rows dequantised to f32, then the scalar
    online-softmax loop, which is how flare-core would run a quantised cache: dequantise, then
    cpu_grouped_query_attention_into).  Returns (tokens/s of the 16-layer step, seconds per repeat)."""
    import oracle
    rng = np.random.default_rng(1)
    k = rng.standard_normal((seqs, CTX, KV_DIM), dtype=np.float32)
    v = rng.standard_normal((seqs, CTX, KV_DIM), dtype=np.float32)
    q = rng.standard_normal((seqs, NH * HD), dtype=np.float32) * np.float32(0.125)
    kb, vb = oracle.quantize_q8_0(k), oracle.quantize_q8_0(v)
    att = np.full(seqs, CTX, np.int32)
    oracle.gqa_decode_heads_mt(q[:1], k[:1], v[:1], att[:1], NH, NKV, HD, threads)   # warm
    t0 = time.perf_counter()
    for _ in range(repeats):
        kd, vd = oracle.dequant_q8_0_mt(kb, threads), oracle.dequant_q8_0_mt(vb, threads)
        oracle.gqa_decode_heads_mt(q, kd, vd, att, NH, NKV, HD, threads)
    dt = (time.perf_counter() - t0) / repeats          # seconds for `seqs` sequences, one layer
    return seqs / (dt * LAYERS), dt


def run_reference(args):
    """The reference's CPU attention for this path (its Rust cannot be built here: no cargo/rustc), restated
    in oracle/flare_oracle.c, on all host threads.  A step is a bounded sample of the workload: 8 of the 32
    sequences of 1 of the 16 layers; tokens/s is scaled linearly from it, ms_per_step is the sample's own time."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    threads = oracle.max_threads()
    seqs = 8
    for _ in range(min(args.warmup, 2)):
        cpu_attention_sample(threads, seqs, 1)
    vals, dts = [], []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok_s, dt = cpu_attention_sample(threads, seqs, 1)
        vals.append(tok_s); dts.append(dt)
    wall = time.perf_counter() - t0
    v = float(np.mean(vals))
    sample = (f"each step = {seqs} of {BATCH} sequences x 1 of {LAYERS} layers (dequantise + attend, all on "
              f"{threads} threads); tok/s scaled linearly to the whole workload, ms_per_step is the sample's own time")
    print(json.dumps({
        "impl": "reference", "metric": "decode_attn_tokens_per_s", "value": v, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * float(np.mean(dts)), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "full_step_ms_extrapolated": 1000.0 * BATCH / v, "wall_s": wall}))


# --------------------------------------------------------------------------------------------
# shared set-up and timing
# --------------------------------------------------------------------------------------------
class Run:
    def __init__(self, args):
        import torch
        import flarellm_b200 as fb
        self.torch, self.fb, self.args = torch, fb, args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist
        self.eng = fb.Engine(self.local)
        # a side stream shared by torch and the library: the CUDA events are recorded on the very stream the
        # kernels are launched on
        self.stream = torch.cuda.Stream()
        torch.cuda.set_stream(self.stream)
        self.eng.set_stream(self.stream.cuda_stream)
        self.sampler = ClockSampler(self.local).start() if self.rank == 0 else None
        self.peaks, self.peak_kind = measured_peaks()

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def timed(self, fn, steps, warmup, min_repeats=25, min_seconds=0.5, max_repeats=400):
        """`warmup` untimed calls, then regions of exactly `steps` calls each: every region sits between two
        (barrier + synchronise) pairs and is timed with CUDA events on the launching stream; per region the
        maximum over ranks is taken.  Returns a dict with the median / min / max ms per step and the clocks
        sampled while the regions ran."""
        torch = self.torch
        if self.args.quick:
            min_repeats, min_seconds = 1, 0.0
        for _ in range(warmup):
            fn()
        times = []
        t_start = time.perf_counter()
        n0 = self.eng.launch_count()
        launches = None
        while True:
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(steps):
                fn()
            e1.record(self.stream)
            self.barrier()
            times.append(e0.elapsed_time(e1) / steps)
            if launches is None:
                launches = self.eng.launch_count() - n0
            done = len(times) >= min_repeats and (time.perf_counter() - t_start) >= min_seconds
            if self.dist is not None:        # every rank must take the same number of regions
                flag = torch.tensor([1 if done else 0], device="cuda")
                self.dist.all_reduce(flag, op=self.dist.ReduceOp.MIN)
                done = bool(flag.item())
            if done or len(times) >= max_repeats:
                break
        t_end = time.perf_counter()
        t = torch.tensor(times, device="cuda", dtype=torch.float64)
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        t = t.cpu().numpy()
        return {"ms": float(np.median(t)), "ms_min": float(t.min()), "ms_max": float(t.max()), "ms_first": float(t[0]),
                "n": int(t.size), "launches_per_region": int(launches),
                "clocks": self.sampler.window(t_start, t_end) if self.sampler else None}

    def roofline(self, bound, achieved, traffic_key=None, per_launch=None):
        peak = self.peaks["hbm_gbs"] if bound == "hbm" else self.peaks["bf16_tflops"]
        r = {"bound": bound, "achieved": achieved, "peak": peak, "unit": "GB/s" if bound == "hbm" else "TFLOP/s",
             "frac": achieved / peak, "peak_source": self.peak_kind}
        if traffic_key is not None:
            r["traffic"], r["traffic_source"] = ncu_traffic(traffic_key)
        else:
            r["traffic"] = None
        if per_launch:
            r["per_launch"] = per_launch
        return r

    def close(self):
        if self.sampler:
            self.sampler.stop()
        self.eng.close()
        if self.dist is not None:
            self.dist.destroy_process_group()


def _repeat_info(t):
    return {"n": t["n"], "ms_median": t["ms"], "ms_min": t["ms_min"], "ms_max": t["ms_max"], "ms_first_region": t["ms_first"]}


# --------------------------------------------------------------------------------------------
# the other configurations of BASELINE.json
# --------------------------------------------------------------------------------------------
def case_prefill(R: Run, window=0, batch=4, steps=None):
    """configs[3]: Llama-3-8B-shaped causal prefill, bf16, S 4096, batch 4 per GPU (window 4096: the sliding-window
    variant at S 8192).  Tensor-bound: flops over the attended (query, key) pairs."""
    torch, fb, eng, args = R.torch, R.fb, R.eng, R.args
    B, nh, nkv, hd, W = batch, 32, 8, 128, window
    S = 8192 if W else 4096
    gen = torch.Generator(device="cuda").manual_seed(3 + R.rank)
    q = (torch.randn(B, S, nh, hd, device="cuda", generator=gen) * 0.5).bfloat16()
    k = (torch.randn(B, S, nkv, hd, device="cuda", generator=gen) * 0.5).bfloat16()
    v = (torch.randn(B, S, nkv, hd, device="cuda", generator=gen) * 0.5).bfloat16()
    o = torch.empty(B, S, nh, hd, device="cuda", dtype=torch.bfloat16)
    fn = lambda: eng.prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), B, S, nh, nkv, hd, window=W,
                             in_dtype=fb.DT_BF16, out_dtype=fb.DT_BF16, out=o.data_ptr())
    t = R.timed(fn, steps or 5, 3, min_repeats=15)
    pairs = sum(min(i + 1, W) for i in range(S)) if W else S * (S + 1) // 2
    flops = 4 * B * nh * hd * pairs
    tf = flops / (t["ms"] * 1e-3) / 1e12
    check = None
    if R.rank == 0 and not args.no_cpu:
        import oracle
        worst, ok, n_rows = 0.0, True, 0
        for b in sorted({0, B - 1}):
            f32 = lambda x: x[b].float().cpu().numpy().reshape(S, -1)
            want = oracle.prefill(f32(q), f32(k), f32(v), S, nh, nkv, hd, window=W, row_start=5 + 17 * b, row_step=251,
                                  threads=oracle.max_threads())
            rows = ~np.isnan(want[:, 0])
            err = np.abs(f32(o)[rows] - want[rows])
            worst = max(worst, float(err.max())); n_rows += int(rows.sum())
            # the output is bf16: one more half-ulp (2^-9 relative) on top of the tolerance
            ok = ok and bool(np.all(err <= 2e-3 + (1e-3 + 2.0 ** -8) * np.abs(want[rows])))
        check = {"rows_checked": n_rows, "max_abs_err": worst, "within_tolerance": ok}
    return {"metric": "prefill_attn_tflops", "value": R.world * tf, "unit": "TFLOP/s", "ms": t["ms"], "repeats": _repeat_info(t),
            "dtype": "bf16 operands, f32 accumulate", "scaling": "weak",
            "workload": f"llama-3-8b-shaped causal prefill attention: 32q/8kv heads, head_dim 128, S {S}, batch {B}/GPU"
                        + (f", sliding window {W}" if W else ""),
            "flops_per_call": flops, "tokens_per_s": R.world * B * S / (t["ms"] * 1e-3),
            "roofline": R.roofline("tensor", tf, "prefill_pp_kernel<128>|llama8b_s4096" if not W else None,
                                   "4 * batch * heads * head_dim * attended (q, k) pairs / call time"),
            "clocks": t["clocks"], "parity_check": check}


def case_kivi(R: Run, steps=None):
    """configs[2]: 2-bit group-32 KIVI cache, context 32768, batch 16; two identical layers read alternately so that
    a call never finds its cache in L2."""
    torch, fb, eng, args = R.torch, R.fb, R.eng, R.args
    nh, nkv, hd, ctx, B, L = 32, 8, 64, 32768, 16, 2
    kv = eng.kv_alloc(L, B, ctx, nkv, hd, fb.KV_KIVI_G32)
    gen = torch.Generator(device="cuda").manual_seed(2 + R.rank)
    for b in range(B):
        k = torch.randn(ctx - 1, nkv * hd, device="cuda", generator=gen)
        v = torch.randn(ctx - 1, nkv * hd, device="cuda", generator=gen)
        outl = torch.randperm(nkv * hd, device="cuda", generator=gen)[:6]      # 1 % of key channels x8
        k[:, outl] *= 8
        for layer in range(L):
            kv.append(layer, b, k.data_ptr(), v.data_ptr(), n_rows=ctx - 1)
        kv.advance(b, ctx - 1)
    q = torch.randn(B, 1, nh, hd, device="cuda", generator=gen) * 0.125
    knew = torch.randn(B, nkv * hd, device="cuda", generator=gen)
    o = torch.empty(L, B, 1, nh, hd, device="cuda")
    for layer in range(L):
        kv.write_step(layer, knew.data_ptr(), knew.data_ptr())
    state = {"i": 0}

    def fn():
        layer = state["i"] & 1
        state["i"] += 1
        eng.decode(kv, layer, nh, q.data_ptr(), out=o[layer].data_ptr())
    t = R.timed(fn, steps or 20, 4)
    got = o.cpu().numpy()
    check = None
    if R.rank == 0 and not args.no_cpu:
        import oracle
        kv.advance(-1, 1)                          # the dequantised view now is what the attention saw
        worst, ok = 0.0, True
        for layer, b in ((0, 0), (1, B - 1)):
            kd, vd = kv.export_dequant(layer, b)
            want = oracle.gqa_decode(q[b].cpu().numpy().reshape(-1), kd, vd, nh, nkv, hd, ctx)
            err = np.abs(got[layer, b].reshape(-1) - want)
            worst = max(worst, float(err.max()))
            ok = ok and bool(np.all(err <= 2e-3 + 1e-3 * np.abs(want)))
        check = {"sequences_checked": 2, "max_abs_err": worst, "within_tolerance": ok}
    per_seq = (ctx - 128) * 384 + 128 * nkv * hd * 2 * 2
    nbytes = B * per_seq
    ach = nbytes / (t["ms"] * 1e-3) / 1e9
    kv.free()
    return {"metric": "kivi_decode_attn_tokens_per_s", "value": R.world * B / (t["ms"] * 1e-3), "unit": "tok/s (one layer)",
            "ms": t["ms"], "repeats": _repeat_info(t), "dtype": "2-bit codes, f16 scale/zero; f16 mma, f32 accumulate", "scaling": "weak",
            "workload": "KIVI 2-bit (group 32, f16 scale+zero, 128-token f16 residual) decode attention, 32q/8kv, head_dim 64, "
                        "ctx 32768, batch 16/GPU, 1 layer per call (2 cache copies alternate: 410 MB > L2)",
            "roofline": R.roofline("hbm", ach, "decode_g32_kernel|c3_ctx32768",
                                   f"{nbytes} algorithmic bytes (384 B per quantised token + the f16 ring rows) / call time"),
            "gpu_launches_per_call": t["launches_per_region"] / (steps or 20), "clocks": t["clocks"], "parity_check": check}


def case_verify(R: Run, steps=None, n_q=6):
    """Speculative verify (flare-core/src/generate.rs:258-303 done in one call per layer): n_q causally ordered
    queries per sequence over the Q8_0 cache of the headline case (batch 32, context 4096); query i sees
    n_q - 1 - i slots fewer than the last one.  Two identical layers are read alternately."""
    torch, fb, eng, args = R.torch, R.fb, R.eng, R.args
    nh, nkv, hd, ctx, B, L = NH, NKV, HD, CTX, 32, 2
    kv = eng.kv_alloc(L, B, ctx, nkv, hd, fb.KV_Q8_0)
    gen = torch.Generator(device="cuda").manual_seed(6 + R.rank)
    for b in range(B):
        k = torch.randn(ctx, nkv * hd, device="cuda", generator=gen)
        v = torch.randn(ctx, nkv * hd, device="cuda", generator=gen)
        for layer in range(L):
            kv.append(layer, b, k.data_ptr(), v.data_ptr(), n_rows=ctx)
        kv.advance(b, ctx)
    q = torch.randn(B, n_q, nh, hd, device="cuda", generator=gen) * 0.125
    o = torch.empty(L, B, n_q, nh, hd, device="cuda")
    att = [ctx] * B
    state = {"i": 0}

    def fn():
        layer = state["i"] & 1
        state["i"] += 1
        eng.decode(kv, layer, nh, q.data_ptr(), n_q=n_q, attend_len=att, out=o[layer].data_ptr())
    t = R.timed(fn, steps or 10, 3, min_repeats=10, min_seconds=0.3)
    check = None
    if R.rank == 0 and not args.no_cpu:
        import oracle
        got = o.cpu().numpy()
        worst, ok = 0.0, True
        for layer, b in ((0, 0), (1, B - 1)):
            kd, vd = kv.export_dequant(layer, b)
            want = oracle.gqa_decode_batched(q[b].cpu().numpy().reshape(1, n_q, -1), kd[None], vd[None], np.full(1, ctx, np.int32),
                                             nh, nkv, hd, n_q=n_q).reshape(n_q, -1)
            err = np.abs(got[layer, b].reshape(n_q, -1) - want)
            worst = max(worst, float(err.max()))
            ok = ok and bool(np.all(err <= 2e-3 + 1e-3 * np.abs(want)))
        check = {"sequences_checked": 2, "queries": n_q, "max_abs_err": worst, "within_tolerance": ok}
    nbytes = B * ctx * 2 * ROW_BYTES
    kv.free()
    return {"metric": "verify_attn_us_per_layer_call", "value": t["ms"] * 1e3, "unit": "us per layer call", "higher_is_better": False,
            "ms": t["ms"], "repeats": _repeat_info(t), "dtype": DTYPE, "scaling": "weak",
            "workload": f"speculative verify: {n_q} causally ordered queries per sequence, Q8_0, 32q/8kv heads, head_dim 64, "
                        f"ctx {ctx}, batch {B}/GPU, 1 layer per call (2 cache copies alternate)",
            "roofline": R.roofline("hbm", nbytes / (t["ms"] * 1e-3) / 1e9,
                                   per_launch=f"{nbytes} algorithmic KV bytes (the cache read once for all {n_q} queries) / call time; the "
                                              "kernel reads the cache once per query, mostly out of L2"),
            "clocks": t["clocks"], "parity_check": check}


def case_f32(R: Run, steps=None):
    """configs[0]: SmolLM2-135M-shaped f32 decode, 512 cached + 1, batch 1: a latency case (788 KB of K+V)."""
    torch, fb, eng, args = R.torch, R.fb, R.eng, R.args
    nh, nkv, hd, L = 9, 3, 64, 512
    rng = np.random.default_rng(0)
    q = rng.standard_normal(nh * hd, dtype=np.float32) * np.float32(0.125)
    k = rng.standard_normal((L + 1, nkv * hd), dtype=np.float32) * np.float32(0.125)
    v = rng.standard_normal((L + 1, nkv * hd), dtype=np.float32) * np.float32(0.125)
    kv = eng.kv_alloc(1, 1, 1024, nkv, hd, fb.KV_F32)
    kv.append(0, 0, k[:L], v[:L]); kv.advance(0, L); kv.write(0, 0, L, k[L], v[L])
    qd = torch.from_numpy(q).cuda()
    od = torch.empty(nh * hd, device="cuda")
    fn = lambda: eng.decode(kv, 0, nh, qd.data_ptr(), out=od.data_ptr())
    t = R.timed(fn, steps or 200, 10, min_repeats=10, min_seconds=0.2)
    t0 = time.perf_counter()
    for _ in range(200):
        host = eng.decode(kv, 0, nh, q.reshape(1, 1, nh, hd))
    ms_host = (time.perf_counter() - t0) / 200 * 1e3
    rec = {"metric": "f32_decode_attn_latency_us", "value": t["ms"] * 1e3, "unit": "us per call (device, stream-pipelined)",
           "higher_is_better": False, "ms": t["ms"], "repeats": _repeat_info(t), "dtype": "f32", "scaling": "replicas",
           "workload": "smollm2-135m-shaped f32 decode attention: 9q/3kv heads, head_dim 64, 512 cached + 1, batch 1, 1 layer",
           "host_call_us": ms_host * 1e3,
           "roofline": dict(R.roofline("hbm", 2 * (L + 1) * nkv * hd * 4 / (t["ms"] * 1e-3) / 1e9),
                            note="787,968 B of K+V, resident in L2 between calls: a latency case, the fraction is not a bandwidth claim"),
           "clocks": t["clocks"], "parity_check": None}
    if R.rank == 0 and not args.no_cpu:
        import oracle
        want = oracle.gqa_decode(q, k, v, nh, nkv, hd, L + 1)
        t0 = time.perf_counter()
        for _ in range(100):
            oracle.gqa_decode(q, k, v, nh, nkv, hd, L + 1)
        rec["cpu_oracle_us"] = (time.perf_counter() - t0) / 100 * 1e6
        err = np.abs(host.reshape(-1) - want)
        dev = np.abs(od.cpu().numpy() - want)
        rec["parity_check"] = {"max_abs_err": float(max(err.max(), dev.max())),
                               "within_tolerance": bool(np.all(err <= 2e-3 + 1e-3 * np.abs(want)) and
                                                        np.all(dev <= 2e-3 + 1e-3 * np.abs(want)))}
    kv.free()
    return rec


def case_longctx(R: Run, steps=None, total=131072):
    """configs[4]: one sequence, 131072 cached positions, Q8_0, Llama-3-8B shape; the slot range is split evenly
    over the ranks, every rank attends its range, the per-rank (m, l, o) records are exchanged and merged
    (strong scaling: the work of one call is fixed).  Two cache copies alternate so that no call finds its
    range in L2."""
    torch, fb, eng, args = R.torch, R.fb, R.eng, R.args
    from flarellm_b200.splitkv import make_split_decoder, shard_slots
    nh, nkv, hd, L = 32, 8, 128, 2
    lo, hi = shard_slots(total, R.world, R.rank)
    n_local = hi - lo
    kv = eng.kv_alloc(L, 1, max(n_local, 32), nkv, hd, fb.KV_Q8_0)
    want_check = R.rank == 0 and not args.no_cpu
    kv_full = eng.kv_alloc(1, 1, total, nkv, hd, fb.KV_Q8_0) if (want_check and R.world > 1) else None
    gen = torch.Generator(device="cuda").manual_seed(4)          # every rank draws the whole sequence's stream
    chunk = 8192
    for c0 in range(0, total, chunk):
        k = torch.randn(chunk, nkv * hd, device="cuda", generator=gen)
        v = torch.randn(chunk, nkv * hd, device="cuda", generator=gen)
        a, b_ = max(c0, lo), min(c0 + chunk, hi)
        if b_ > a:
            ks, vs = k[a - c0:b_ - c0].contiguous(), v[a - c0:b_ - c0].contiguous()
            for layer in range(L):
                kv.append(layer, 0, ks.data_ptr(), vs.data_ptr(), n_rows=b_ - a)
            kv.advance(0, b_ - a)
        if kv_full is not None:
            kv_full.append(0, 0, k.data_ptr(), v.data_ptr(), n_rows=chunk)
            kv_full.advance(0, chunk)
    q = torch.randn(1, 1, nh, hd, device="cuda", generator=gen) / (hd ** 0.5) * 4
    dec = make_split_decoder(eng, kv, nh, n_local, R.dist)
    state = {"i": 0, "out": None}

    def fn():
        layer = state["i"] & 1
        state["i"] += 1
        state["out"] = dec.decode(layer, q)

    def fn_kernel_only():
        layer = state["i"] & 1
        state["i"] += 1
        dec.partial_only(layer, q)
    for _ in range(3):
        fn()
    status = dec.status()
    if status != "ok":          # a rank is missing or out of step: do not queue hundreds of calls that each wait for it
        raise RuntimeError("long-context exchange failed during warm-up: " + status)
    t = R.timed(fn, steps or 20, 4)
    tk = R.timed(fn_kernel_only, steps or 20, 3, min_repeats=10, min_seconds=0.2)
    got = state["out"].cpu().numpy().reshape(-1)
    status = dec.status()
    check = None
    if want_check:
        import oracle
        src = kv_full if kv_full is not None else kv
        kd, vd = src.export_dequant(0, 0)
        att = np.full(1, total, np.int32)
        want = oracle.gqa_decode_heads_mt(q.cpu().numpy().reshape(1, -1), kd[None, :total], vd[None, :total], att, nh, nkv, hd,
                                          oracle.max_threads()).reshape(-1)
        err = np.abs(got - want)
        check = {"slots": total, "ranks": R.world, "max_abs_err": float(err.max()),
                 "within_tolerance": bool(np.all(err <= 2e-3 + 1e-3 * np.abs(want)))}
    row_bytes = nkv * hd + nkv * hd // 32 * 2
    layer_bytes = total * 2 * row_bytes
    ach = layer_bytes / R.world / (tk["ms"] * 1e-3) / 1e9
    rec = {"metric": "longctx_decode_attn_tokens_per_s", "value": 1.0 / (t["ms"] * 1e-3), "unit": "tok/s (one layer)",
           "ms": t["ms"], "repeats": _repeat_info(t), "kernel_only_ms": tk["ms"], "dtype": DTYPE, "scaling": "strong",
           "workload": f"llama-3-8b-shaped single-sequence decode attention, Q8_0, {total} slots, 1 layer per call "
                       "(2 cache copies alternate: 570 MB > L2)",
           "parallelism": f"slot range split over {R.world} GPU(s); exchange of {nh * (hd + 2) * 4} B per rank + merge: {dec.how}",
           "hbm_gbs_whole_call": layer_bytes / (t["ms"] * 1e-3) / 1e9,
           "roofline": R.roofline("hbm", ach, "decode_q8_kernel<128>|c5_131072" if R.world == 1 else None,
                                  f"{layer_bytes // R.world} algorithmic KV bytes per rank / time of the attention kernels alone (no exchange)"),
           "exchange_status": status, "clocks": t["clocks"], "parity_check": check}
    dec.close()
    if kv_full is not None:
        kv_full.free()
    kv.free()
    return rec


def _random_q8_0(rng, rows, cols):
    """A Q8_0 block stream with random int8 weights and one scale for all blocks, sized so that a unit-variance
    input gives a unit-variance output."""
    nb = rows * (cols // 32)
    blocks = np.empty((nb, 34), dtype=np.uint8)
    blocks[:, 2:] = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
    blocks[:, :2] = np.array([np.float16(1.0 / (73.0 * cols ** 0.5))]).view(np.uint8)
    return blocks.reshape(-1)


def case_forward(R: Run, steps=None, layers=16, vocab=128256):
    """The device-resident single-token forward pass (flare_forward_token) at Llama-3.2-1B shapes with Q8_0
    matrices: hidden 2048, 32 q / 8 kv heads x 64, intermediate 8192, 16 layers, vocabulary 128256, Q8_0 cache
    holding 1024 earlier tokens.  One call = one token per sequence: embedding row up, logits down."""
    torch, fb, eng, args = R.torch, R.fb, R.eng, R.args
    cfg = dict(hidden_dim=2048, num_heads=32, num_kv_heads=8, head_dim=64, intermediate_dim=8192, vocab_size=vocab,
               rms_norm_eps=1e-5)
    dim, inter, q_dim, kv_dim = 2048, 8192, 2048, 512
    rng = np.random.default_rng(5)
    lw = dict(attn_norm=np.ones(dim, np.float32), ffn_norm=np.ones(dim, np.float32),
              qkv=_random_q8_0(rng, q_dim + 2 * kv_dim, dim), wo=_random_q8_0(rng, dim, q_dim),
              gate_up=_random_q8_0(rng, 2 * inter, dim), down=_random_q8_0(rng, dim, inter))
    out_w = _random_q8_0(rng, vocab, dim)
    model = eng.model_create(num_layers=layers, **cfg)
    for li in range(layers):
        model.set_layer(li, **lw)          # every layer its own copy on the device (the same random draw)
    model.set_output(np.ones(dim, np.float32), output_q8=out_w)
    half = np.arange(32, dtype=np.float64)
    ang = np.arange(4096, dtype=np.float64)[:, None] * (10000.0 ** (-2.0 * half / 64.0))[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    weight_bytes = layers * sum(lw[k].size for k in ("qkv", "wo", "gate_up", "down")) + out_w.size
    results = {}
    for batch in (1, 8):
        kv = eng.kv_alloc(layers, batch, 4096, 8, 64, fb.KV_Q8_0)
        kv.set_rope_table(cos, sin)
        x = rng.standard_normal((batch, dim), dtype=np.float32)
        state = {"t": 0}

        def fn():
            # every timed token sees 1024 cached tokens: the ring state is put back before each call
            for b in range(batch):
                kv.set_state(b, 1024, 1024)
            state["logits"] = model.forward(kv, x, positions=[1024] * batch)
        t = R.timed(fn, steps or 10, 3, min_repeats=5, min_seconds=0.3, max_repeats=50)
        kv_bytes = layers * batch * 1025 * 2 * (kv_dim // 32 * 34)
        results[batch] = (t, kv_bytes)
        assert np.all(np.isfinite(state["logits"]))
        kv.free()
    t1, kvb1 = results[1]
    t8, kvb8 = results[8]
    rec = {"metric": "resident_forward_tokens_per_s", "value": 1e3 / t1["ms"], "unit": "tok/s (batch 1)", "ms": t1["ms"],
           "repeats": _repeat_info(t1), "batch8_tokens_per_s": 8e3 / t8["ms"], "batch8_ms": t8["ms"],
           "dtype": "q8_0 weights and inputs (dp4a, s32), f32 block sums; q8_0 kv", "scaling": "replicas",
           "workload": f"llama-3.2-1b-shaped forward, Q8_0 matrices ({weight_bytes / 1e9:.2f} GB read per token), {layers} layers, "
                       f"vocabulary {vocab}, 1024 cached tokens, host embedding row in, host logits out",
           "gpu_launches_per_token": t1["launches_per_region"] / (steps or 10),
           "roofline": R.roofline("hbm", (weight_bytes + kvb1) / (t1["ms"] * 1e-3) / 1e9,
                                  per_launch="Q8_0 weight bytes + attended KV bytes of one token / time of the whole call "
                                             "(about 180 launches; the call is launch- and latency-bound at batch 1)"),
           "clocks": t1["clocks"], "parity_check": None}
    if R.rank == 0 and not args.no_cpu:
        import oracle
        # two tokens from an empty cache on a two-layer cut of the same model against the CPU restatement
        small = eng.model_create(num_layers=2, **cfg)
        for li in range(2):
            small.set_layer(li, **lw)
        small.set_output(np.ones(dim, np.float32), output_q8=out_w)
        kv = eng.kv_alloc(2, 1, 64, 8, 64, fb.KV_Q8_0)
        kv.set_rope_table(cos[:64], sin[:64])
        kc = [np.zeros((64, kv_dim), np.float32) for _ in range(2)]
        vc = [np.zeros((64, kv_dim), np.float32) for _ in range(2)]
        store = lambda r: oracle.dequant_q8_0(oracle.quantize_q8_0(r))
        worst, rel, ok = 0.0, 0.0, True
        for tkn in range(2):
            xe = rng.standard_normal(dim, dtype=np.float32)
            got = small.forward(kv, xe[None], positions=[tkn])[0]
            want = oracle.forward_token_q8(cfg, [lw, lw], np.ones(dim, np.float32), out_w, None, cos[:64], sin[:64], 10000.0,
                                           kc, vc, tkn, xe, tkn, store=store)
            err = np.abs(got - want)
            # The attention output of a Q8_0 cache carries the 2e-3 + 1e-3 |x| contract of the attention path (its
            # weights are rounded to f16); the next step quantises that output to 8 bits, so a few codes per hundred
            # land one step away and the logits of 128256 rows move by up to about 1 % of their spread.  (With an f32
            # cache the same pass agrees to 2e-3 of the spread: tests/test_gpu_forward.py.)
            worst = max(worst, float(err.max()))
            rel = max(rel, float(np.linalg.norm(got - want) / np.linalg.norm(want)))
            ok = ok and float(err.max()) <= 2e-2 * float(np.abs(want).max()) and int(np.argmax(got)) == int(np.argmax(want))
        rec["parity_check"] = {"tokens": 2, "layers": 2, "max_abs_err": worst, "rel_l2_err": rel,
                               "tolerance": "max |err| <= 2 % of max |logit|, same arg max", "within_tolerance": ok}
        small.free(); kv.free()
    model.free()
    return rec


def _prefill_batch(R):
    return R.args.batch if R.args.batch != BATCH else 4          # --batch: a smaller case for profiler captures


CASES = {"prefill": lambda R, **kw: case_prefill(R, 0, _prefill_batch(R), **kw),
         "prefill_window": lambda R, **kw: case_prefill(R, 4096, _prefill_batch(R), **kw),
         "kivi": case_kivi, "longctx": case_longctx, "f32": case_f32, "forward": case_forward, "verify": case_verify}


def case_decode(R: Run):
    """The headline line."""
    torch, fb, eng, args = R.torch, R.fb, R.eng, R.args
    layers, batch = args.layers, args.batch
    layer_bytes = batch * CTX * 2 * ROW_BYTES
    kv = eng.kv_alloc(layers, batch, CTX, NKV, HD, fb.KV_Q8_0)
    gen = torch.Generator(device="cuda").manual_seed(1 + R.rank)
    for layer in range(layers):
        for b in range(batch):
            k = torch.randn(CTX - 1, KV_DIM, device="cuda", generator=gen)
            v = torch.randn(CTX - 1, KV_DIM, device="cuda", generator=gen)
            kv.append(layer, b, k.data_ptr(), v.data_ptr(), n_rows=CTX - 1)
        torch.cuda.synchronize()
    kv.advance(-1, CTX - 1)                       # 4095 cached tokens; each step adds the 4096th
    q_dev = torch.randn(layers, batch, 1, NH, HD, device="cuda", generator=gen) * 0.125
    knew = torch.randn(layers, batch, KV_DIM, device="cuda", generator=gen)
    vnew = torch.randn(layers, batch, KV_DIM, device="cuda", generator=gen)
    out_dev = torch.empty(layers, batch, 1, NH, HD, device="cuda")
    for layer in range(layers):
        kv.write_step(layer, knew[layer].data_ptr(), vnew[layer].data_ptr())
    torch.cuda.synchronize()

    def step_device():
        for layer in range(layers):
            eng.decode(kv, layer, NH, q_dev[layer].data_ptr(), out=out_dev[layer].data_ptr())

    # host-side buffers of the end-to-end arm: page-locked, one allocation per layer laid out [K rows][V rows][q]
    # (what a host does that keeps its per-layer forward buffers together: the step then needs one transfer)
    row_fl, q_fl = batch * KV_DIM, batch * NH * HD
    pack = torch.empty(layers, 2 * row_fl + q_fl).pin_memory()
    pack[:, :row_fl] = knew.cpu().reshape(layers, -1)
    pack[:, row_fl:2 * row_fl] = vnew.cpu().reshape(layers, -1)
    pack[:, 2 * row_fl:] = q_dev.cpu().reshape(layers, -1)
    pack_np = pack.numpy()
    q_host = q_dev.cpu().numpy()
    out_host = torch.zeros(layers, batch, 1, NH, HD).pin_memory().numpy()
    k_l = [pack_np[i, :row_fl] for i in range(layers)]
    v_l = [pack_np[i, row_fl:2 * row_fl] for i in range(layers)]
    q_l = [pack_np[i, 2 * row_fl:] for i in range(layers)]
    o_l = [out_host[i] for i in range(layers)]

    # host addresses resolved once, as a Rust caller's slices are (the ndarrays above stay alive)
    k_a, v_a, q_a, o_a = ([int(x.ctypes.data) for x in xs] for xs in (k_l, v_l, q_l, o_l))

    def step_e2e():
        for layer in range(layers):
            eng.decode_step(kv, layer, NH, k_a[layer], v_a[layer], q_a[layer], out=o_a[layer], on_device=False)

    t = R.timed(step_device, args.steps, max(3, args.warmup))
    te = R.timed(step_e2e, max(3, min(args.steps, 20)), 3, min_repeats=10, min_seconds=0.3)

    # parity of what was just timed: a few (layer, sequence) pairs against the oracle, device and host arms
    check = None
    if R.rank == 0 and not args.no_cpu:
        import oracle
        worst, ok = 0.0, True
        out_np = out_dev.cpu().numpy()
        pairs = sorted({(0, 0), (layers - 1, batch - 1), (layers // 2, batch // 3), (1 % layers, batch - 1)})
        for layer, b in pairs:
            kd, vd = kv.export_dequant(layer, b)
            want = oracle.gqa_decode(q_host[layer, b].reshape(-1), kd, vd, NH, NKV, HD, CTX)
            for got in (out_np[layer, b], out_host[layer, b]):
                err = np.abs(got.reshape(-1) - want)
                worst = max(worst, float(err.max()))
                ok = ok and bool(np.all(err <= 2e-3 + 1e-3 * np.abs(want)))
        check = {"pairs_checked": len(pairs), "arms": "device-resident and host-buffer (e2e)", "max_abs_err": worst,
                 "within_tolerance": ok}
    kv.free()

    ms_step = t["ms"]
    tok_s = R.world * batch / (ms_step * 1e-3)
    achieved = layer_bytes / (ms_step * 1e-3 / layers) / 1e9
    full = (layers, batch) == (LAYERS, BATCH)
    out = {
        "metric": "decode_attn_tokens_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": R.world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": workload_config(R.world, layers, batch),
        "repeats": _repeat_info(t),
        "hbm_gbs_total": R.world * achieved,
        "roofline": R.roofline("hbm", achieved, "decode_q8_kernel<64>|c2_batch32" if full else None,
                               f"{layer_bytes} algorithmic KV bytes per layer call / (step time / {layers} layers)"),
        "e2e": {"value": R.world * batch / (te["ms"] * 1e-3), "unit": "tok/s", "ms_per_step": te["ms"],
                "ms_min": te["ms_min"], "ms_max": te["ms_max"], "regions": te["n"],
                "h2d_bytes_per_step": int(layers * (batch * NH * HD * 4 + 2 * batch * KV_DIM * 4)),
                "d2h_bytes_per_step": int(layers * batch * NH * HD * 4),
                "call": "flare_decode_step per layer: K/V rows + q host->device in one transfer (page-locked, contiguous), "
                        "store, attend, output written to the caller's page-locked buffer; one synchronisation per layer"},
        "gpu_launches": int(t["launches_per_region"]), "clocks": t["clocks"], "parity_check": check,
    }
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", choices=["all", "decode"] + sorted(CASES))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=LAYERS, help=argparse.SUPPRESS)      # smaller cases for profiler captures
    ap.add_argument("--batch", type=int, default=BATCH, help=argparse.SUPPRESS)
    ap.add_argument("--case-steps", type=int, default=0, help=argparse.SUPPRESS)
    ap.add_argument("--no-cpu", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--quick", action="store_true", help=argparse.SUPPRESS)             # one timed region: profiler captures
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    R = Run(args)
    kw = {"steps": args.case_steps} if args.case_steps else {}
    if args.case in CASES:
        rec = CASES[args.case](R, **kw)
        if R.rank == 0:
            rec.setdefault("n_gpus", R.world)
            print(json.dumps(rec))
        return R.close()

    out = case_decode(R)
    if args.case == "all":
        cases = {}
        for name in ("prefill", "prefill_window", "kivi", "longctx", "f32", "forward", "verify"):
            try:
                cases[name] = CASES[name](R)
            except Exception as e:                     # a failing side case must not take the headline line with it
                cases[name] = {"error": f"{type(e).__name__}: {e}"}
                if R.dist is not None:
                    raise
        out["cases"] = cases
    if R.rank == 0:
        if not args.no_cpu:
            tok_cpu, dt = cpu_attention_sample(1, 8, 2)
            out["cpu_baseline"] = {"value": tok_cpu, "unit": "tok/s", "cores": 1, "kind": "port",
                                   "sample": "8 of 32 sequences x 1 of 16 layers, 2 repeats, scaled linearly; "
                                             "single thread because flare-core's attention is single-threaded"}
        print(json.dumps(out))
    R.close()


if __name__ == "__main__":
    main()
