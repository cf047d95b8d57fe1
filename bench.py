#!/usr/bin/env python
"""Decode-attention benchmark: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N GPUs, one process per GPU, weak scaling, no collective): the Llama-3.2-1B-shaped
Q8_0 decode of BASELINE.json configs[1] at batch 32 on every GPU — 32 query / 8 KV heads,
head_dim 64, context 4096, 16 layers.  One step = one new token for every sequence = 16
attention calls (one per layer), each streaming that layer's whole K/V cache once.

  value     tokens/s of the whole job (all ranks), inputs resident in HBM, CUDA-event timed
  e2e       the same through the host-buffer C-ABI calls a ComputeBackend makes per layer:
            new K/V rows H2D (flare_kv_write_step_f32), q H2D + attention + output D2H
            (flare_decode_attn with host pointers), pinned host buffers
  roofline  algorithmic KV bytes of one layer call / its average device time, against the
            measured HBM copy bandwidth
  cpu_baseline  the CPU oracle (a restatement of flare-core's scalar attention) on a bounded
            sample, on this box's host cores

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


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_attention_sample(threads: int, seqs: int, repeats: int):
    """Time the CPU oracle on `seqs` sequences of one layer (Q8_0 rows dequantised to f32, then
    the scalar online-softmax loop, which is how flare-core would run a quantised cache:
    dequantise, then cpu_grouped_query_attention_into).  Returns tokens/s for the 16-layer step."""
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
        kd, vd = oracle.dequant_q8_0(kb), oracle.dequant_q8_0(vb)
        oracle.gqa_decode_heads_mt(q, kd, vd, att, NH, NKV, HD, threads)
    dt = (time.perf_counter() - t0) / repeats          # seconds for `seqs` sequences, one layer
    tok_s = seqs / (dt * LAYERS)
    return tok_s, dt


def run_reference(args):
    """The reference's CPU attention for this path (its Rust cannot be built here: no cargo/rustc),
    restated in oracle/flare_oracle.c, on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    threads = oracle.max_threads()
    seqs = 8
    vals = []
    for _ in range(args.warmup):
        cpu_attention_sample(threads, seqs, 1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok_s, _ = cpu_attention_sample(threads, seqs, 1)
        vals.append(tok_s)
    wall = time.perf_counter() - t0
    v = float(np.mean(vals))
    sample = f"{seqs} of {BATCH} sequences x 1 of {LAYERS} layers per step, scaled linearly"
    print(json.dumps({
        "impl": "reference", "metric": "decode_attn_tokens_per_s", "value": v, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * BATCH / v, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": wall}))


# --------------------------------------------------------------------------------------------
# the other configurations of BASELINE.json (selected with --case; the default line is `decode`)
# --------------------------------------------------------------------------------------------
def _setup(args):
    import torch
    import flarellm_b200 as fb
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    eng = fb.Engine(local)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    eng.set_stream(stream.cuda_stream)
    return torch, fb, dist, eng, stream, rank, world, local


def _timed(torch, dist, stream, fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def case_prefill(args):
    """BASELINE.json configs[3]: Llama-3-8B-shaped causal prefill, bf16, S 4096, batch 4 per GPU
    (--window 4096: the sliding-window variant at S 8192).  Tensor-bound: flops over causal pairs."""
    torch, fb, dist, eng, stream, rank, world, local = _setup(args)
    B, nh, nkv, hd = (args.batch if args.batch != BATCH else 4), 32, 8, 128     # --batch: smaller case for ncu
    W = args.window
    S = 8192 if W else 4096
    gen = torch.Generator(device="cuda").manual_seed(3 + rank)
    q = (torch.randn(B, S, nh, hd, device="cuda", generator=gen) * 0.5).bfloat16()
    k = (torch.randn(B, S, nkv, hd, device="cuda", generator=gen) * 0.5).bfloat16()
    v = (torch.randn(B, S, nkv, hd, device="cuda", generator=gen) * 0.5).bfloat16()
    o = torch.empty(B, S, nh, hd, device="cuda", dtype=torch.bfloat16)
    fn = lambda: eng.prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), B, S, nh, nkv, hd, window=W,
                             in_dtype=fb.DT_BF16, out_dtype=fb.DT_BF16, out=o.data_ptr())
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms = _timed(torch, dist, stream, fn, args.steps, max(3, args.warmup))
    clocks = sampler.stop() if sampler else None
    pairs = sum(min(t + 1, W) for t in range(S)) if W else S * (S + 1) // 2
    flops = 4 * B * nh * hd * pairs
    if rank == 0:
        peaks, kind = measured_peaks()
        tf = flops / (ms * 1e-3) / 1e12
        check = None
        if not args.no_cpu:
            import oracle
            f32 = lambda t: t[0].float().cpu().numpy().reshape(S, -1)
            want = oracle.prefill(f32(q), f32(k), f32(v), S, nh, nkv, hd, window=W, row_start=5, row_step=251,
                                  threads=oracle.max_threads())
            rows = ~np.isnan(want[:, 0])
            err = np.abs(f32(o)[rows] - want[rows])
            check = {"rows_checked": int(rows.sum()), "max_abs_err": float(err.max()),
                     "within_tolerance": bool(np.all(err <= 2e-3 + (1e-3 + 2.0 ** -8) * np.abs(want[rows])))}
        print(json.dumps({
            "metric": "prefill_attn_tflops", "value": world * tf, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"llama-3-8b-shaped causal prefill attention: 32q/8kv heads, head_dim 128, S {S}, batch {B}/GPU"
                                   + (f", sliding window {W}" if W else ""), "flops": "4*B*heads*head_dim*attended (q,k) pairs"},
            "tokens_per_s": world * B * S / (ms * 1e-3),
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16_tflops"], "traffic": None, "peak_source": kind},
            "clocks": clocks, "parity_check": check}))
    eng.close()
    if dist is not None:
        dist.destroy_process_group()


def case_longctx(args):
    """BASELINE.json configs[4]: one sequence, 131072 cached positions, Q8_0, Llama-3-8B shape, the slot
    range split evenly over the ranks; per-rank (m, l, o) records all-gathered (NCCL) and merged."""
    torch, fb, dist, eng, stream, rank, world, local = _setup(args)
    from flarellm_b200.splitkv import SplitKvDecoder, shard_slots
    nh, nkv, hd, total = 32, 8, 128, 131072
    lo, hi = shard_slots(total, world, rank)
    n_local = hi - lo
    kv = eng.kv_alloc(1, 1, max(n_local, 32), nkv, hd, fb.KV_Q8_0)
    gen = torch.Generator(device="cuda").manual_seed(4)          # every rank draws the whole sequence's stream
    chunk = 8192
    for c0 in range(0, total, chunk):
        k = torch.randn(chunk, nkv * hd, device="cuda", generator=gen)
        v = torch.randn(chunk, nkv * hd, device="cuda", generator=gen)
        a, b_ = max(c0, lo), min(c0 + chunk, hi)
        if b_ > a:
            kv.append(0, 0, k[a - c0:b_ - c0].contiguous().data_ptr(), v[a - c0:b_ - c0].contiguous().data_ptr(), n_rows=b_ - a)
            kv.advance(0, b_ - a)
    q = torch.randn(1, 1, nh, hd, device="cuda", generator=gen) / (hd ** 0.5) * 4
    dec = SplitKvDecoder(eng, kv, nh, n_local)
    out = None

    def fn():
        nonlocal out
        out = dec.decode(0, q)

    def fn_kernel_only():
        dec.partial_fn(0, q)
    ms = _timed(torch, dist, stream, fn, args.steps, max(3, args.warmup))
    ms_k = _timed(torch, dist, stream, fn_kernel_only, args.steps, 3)
    row_bytes = nkv * hd + nkv * hd // 32 * 2
    layer_bytes = total * 2 * row_bytes
    if rank == 0:
        peaks, kind = measured_peaks()
        ach = layer_bytes / world / (ms_k * 1e-3) / 1e9
        print(json.dumps({
            "metric": "longctx_decode_attn_tokens_per_s", "value": 1.0 / (ms * 1e-3), "unit": "tok/s (one layer)", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "llama-3-8b-shaped single-sequence decode attention, Q8_0, 131072 slots, 1 layer",
                       "parallelism": f"slot range split over {world} GPU(s); all-gather of {nh * (hd + 2) * 4} B per rank + merge"},
            "kernel_only_ms": ms_k, "hbm_gbs_total": layer_bytes / (ms * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                         "traffic": None, "peak_source": kind,
                         "per_launch": f"{layer_bytes // world} algorithmic KV bytes per rank / partial-kernel time (no collective)"}}))
    kv.free()
    eng.close()
    if dist is not None:
        dist.destroy_process_group()


def case_kivi(args):
    """BASELINE.json configs[2]: 2-bit group-32 KIVI cache, context 32768, batch 16, one layer."""
    torch, fb, dist, eng, stream, rank, world, local = _setup(args)
    nh, nkv, hd, ctx, B = 32, 8, 64, 32768, 16
    kv = eng.kv_alloc(1, B, ctx, nkv, hd, fb.KV_KIVI_G32)
    gen = torch.Generator(device="cuda").manual_seed(2 + rank)
    for b in range(B):
        k = torch.randn(ctx - 1, nkv * hd, device="cuda", generator=gen)
        v = torch.randn(ctx - 1, nkv * hd, device="cuda", generator=gen)
        outl = torch.randperm(nkv * hd, device="cuda", generator=gen)[:6]      # 1 % of key channels x8
        k[:, outl] *= 8
        kv.append(0, b, k.data_ptr(), v.data_ptr(), n_rows=ctx - 1)
        kv.advance(b, ctx - 1)
    q = torch.randn(B, 1, nh, hd, device="cuda", generator=gen) * 0.125
    knew = torch.randn(B, nkv * hd, device="cuda", generator=gen)
    o = torch.empty(B, 1, nh, hd, device="cuda")
    kv.write_step(0, knew.data_ptr(), knew.data_ptr())
    fn = lambda: eng.decode(kv, 0, nh, q.data_ptr(), out=o.data_ptr())
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms = _timed(torch, dist, stream, fn, args.steps, max(3, args.warmup))
    clocks = sampler.stop() if sampler else None
    check = None
    if rank == 0 and not args.no_cpu:
        import oracle
        worst, ok = 0.0, True
        for b in (0, B - 1):
            kd, vd = kv.export_dequant(0, b)
            want = oracle.gqa_decode(q[b].cpu().numpy().reshape(-1), kd, vd, nh, nkv, hd, ctx)
            err = np.abs(o[b].cpu().numpy().reshape(-1) - want)
            worst = max(worst, float(err.max()))
            ok = ok and bool(np.all(err <= 2e-3 + 1e-3 * np.abs(want)))
        check = {"sequences_checked": 2, "max_abs_err": worst, "within_tolerance": ok}
    per_seq = (ctx - 128) * 384 + 128 * nkv * hd * 2 * 2
    nbytes = B * per_seq
    if rank == 0:
        peaks, kind = measured_peaks()
        ach = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "kivi_decode_attn_tokens_per_s", "value": world * B / (ms * 1e-3), "unit": "tok/s (one layer)", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "KIVI 2-bit (group 32, f16 scale+zero, 128-token f16 residual) decode attention, 32q/8kv, head_dim 64, ctx 32768, batch 16, 1 layer"},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                         "traffic": 222.4e6, "traffic_source": "ncu dram read+write of decode_g32_kernel, profiles/decode_g32_kernel_c3_ctx32768.md",
                         "peak_source": kind, "per_launch": f"{nbytes} algorithmic bytes (384 B per quantised token + residual rows)"},
            "gpu_launches": 2 * args.steps, "clocks": clocks, "parity_check": check}))
    kv.free()
    eng.close()
    if dist is not None:
        dist.destroy_process_group()


def case_f32(args):
    """BASELINE.json configs[0]: SmolLM2-135M-shaped f32 decode, 512 cached + 1, batch 1: latency."""
    torch, fb, dist, eng, stream, rank, world, local = _setup(args)
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
    ms = _timed(torch, dist, stream, fn, max(args.steps, 200), 10)
    t0 = time.perf_counter()
    for _ in range(200):
        host = eng.decode(kv, 0, nh, q.reshape(1, 1, nh, hd))
    ms_host = (time.perf_counter() - t0) / 200 * 1e3
    if rank == 0:
        import oracle
        want = oracle.gqa_decode(q, k, v, nh, nkv, hd, L + 1)
        t0 = time.perf_counter()
        for _ in range(200):
            oracle.gqa_decode(q, k, v, nh, nkv, hd, L + 1)
        ms_cpu = (time.perf_counter() - t0) / 200 * 1e3
        err = float(np.max(np.abs(host.reshape(-1) - want)))
        print(json.dumps({
            "metric": "f32_decode_attn_latency_us", "value": ms * 1e3, "unit": "us per call (device, stream-pipelined)", "n_gpus": 1,
            "steps": max(args.steps, 200), "warmup": 10, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "smollm2-135m-shaped f32 decode attention: 9q/3kv heads, head_dim 64, 512 cached + 1, batch 1, 1 layer",
                       "note": "787,968 B of K+V: latency-bound, a roofline fraction is not meaningful"},
            "host_call_us": ms_host * 1e3, "cpu_oracle_us": ms_cpu * 1e3, "max_abs_err": err}))
    kv.free()
    eng.close()


CASES = {"prefill": case_prefill, "longctx": case_longctx, "kivi": case_kivi, "f32": case_f32}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="decode", choices=["decode"] + sorted(CASES))
    ap.add_argument("--window", type=int, default=0, help="prefill: sliding window (4096 selects the S=8192 variant)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=LAYERS, help=argparse.SUPPRESS)      # smaller cases for ncu
    ap.add_argument("--batch", type=int, default=BATCH, help=argparse.SUPPRESS)
    ap.add_argument("--no-cpu", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.case != "decode":
        return CASES[args.case](args)

    import torch
    import flarellm_b200 as fb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    layers, batch = args.layers, args.batch
    layer_bytes = batch * CTX * 2 * ROW_BYTES

    eng = fb.Engine(local)
    # a side stream shared by torch and the library: the CUDA events below are recorded on the very
    # stream the kernels are launched on
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    eng.set_stream(stream.cuda_stream)
    kv = eng.kv_alloc(layers, batch, CTX, NKV, HD, fb.KV_Q8_0)
    gen = torch.Generator(device="cuda").manual_seed(1 + rank)
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

    # host-side buffers of the end-to-end arm (pinned)
    q_host = q_dev.cpu().pin_memory().numpy()
    k_host, v_host = knew.cpu().pin_memory().numpy(), vnew.cpu().pin_memory().numpy()
    out_host = torch.empty(layers, batch, 1, NH, HD).pin_memory().numpy()

    def step_e2e():
        for layer in range(layers):
            kv.write_step(layer, k_host[layer], v_host[layer])
            eng.decode(kv, layer, NH, q_host[layer], out=out_host[layer])

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = eng.launch_count()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps, eng.launch_count() - n0

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms_step, launches = timed(step_device, args.steps, max(3, args.warmup))
    clocks = sampler.stop() if sampler else None
    e2e_steps = max(3, min(args.steps, 20))
    ms_e2e, _ = timed(step_e2e, e2e_steps, 3)

    # parity spot check of what was just timed: a few (layer, sequence) pairs against the oracle
    check = None
    if rank == 0 and not args.no_cpu:
        import oracle
        worst, ok = 0.0, True
        out_np = out_dev.cpu().numpy()
        for layer, b in sorted({(0, 0), (layers - 1, batch - 1), (layers // 2, batch // 3), (1 % layers, batch - 1)}):
            kd, vd = kv.export_dequant(layer, b)
            want = oracle.gqa_decode(q_host[layer, b].reshape(-1), kd, vd, NH, NKV, HD, CTX)
            err = np.abs(out_np[layer, b].reshape(-1) - want)
            worst = max(worst, float(err.max()))
            ok = ok and bool(np.all(err <= 2e-3 + 1e-3 * np.abs(want)))
        check = {"pairs_checked": 4, "max_abs_err": worst, "within_tolerance": ok}

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        tok_s = world * batch / (ms_step * 1e-3)
        per_launch_s = ms_step * 1e-3 / layers
        achieved = layer_bytes / per_launch_s / 1e9
        out = {
            "metric": "decode_attn_tokens_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD if (layers, batch) == (LAYERS, BATCH) else
                       f"{WORKLOAD} [reduced: batch {batch}, {layers} layers]",
                       "kv_cache": "Q8_0 (int8 + f16 scale per 32)", "l2": "inputs larger than L2: %.2f GB of KV per step"
                       % (layers * layer_bytes / 1e9), "parallelism": f"{world} x independent batch-{batch} shards, no collective"},
            "hbm_gbs_total": world * achieved,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"],
                         "traffic": 148.5e6 if (layers, batch) == (LAYERS, BATCH) else None,
                         "traffic_source": "ncu dram read+write per launch of decode_q8_kernel, profiles/decode_q8_kernel_c2_batch32.md",
                         "peak_source": peak_kind,
                         "per_launch": f"{layer_bytes} algorithmic KV bytes per layer call / (step time / {layers} layers)"},
            "e2e": {"value": world * batch / (ms_e2e * 1e-3), "unit": "tok/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": int(layers * (batch * NH * HD * 4 + 2 * batch * KV_DIM * 4)),
                    "d2h_bytes_per_step": int(layers * batch * NH * HD * 4)},
            "gpu_launches": int(launches), "clocks": clocks, "parity_check": check,
        }
        if not args.no_cpu:
            tok_cpu, dt = cpu_attention_sample(1, 8, 2)
            out["cpu_baseline"] = {"value": tok_cpu, "unit": "tok/s", "cores": 1, "kind": "port",
                                   "sample": "8 of 32 sequences x 1 of 16 layers, 2 repeats, scaled linearly; "
                                             "single thread because flare-core's attention is single-threaded"}
        print(json.dumps(out))
    kv.free()
    eng.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
