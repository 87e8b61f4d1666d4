#!/usr/bin/env python
"""Decode-throughput benchmark of the quantized-inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one greedy decode step (one new token for each of the B sequences), run as the captured chain of
launches (the default of the library; the faster of its two implementations on the shapes measured); the headline
line also carries the same measurement through the one-launch persistent kernel (`persistent_step`).  The default workload
is the one the headline target is quoted on: the Llama-3-8B-shaped model, int4 (group 32) weights with
an int8 head, batch 1, 1024 cached positions.  Weights are seeded synthetic N(0, 0.02^2) generated and
quantized on the device; nothing is read from disk.  With N > 1 (launched by torch.distributed.run, one
process per GPU) the same model is sharded Megatron-style over the N GPUs (strong scaling).

Prints one JSON line (rank 0).  `value` is measured with the ids resident on the device, as the median
over several timed regions of exactly K steps each; `e2e` goes through the host-buffer call
`forward_cached(ids_host) -> logits_host` plus the host-side argmax per token, which is the reference's own
generate loop (generation.rs:102-104).  Before anything is timed the model's greedy tokens are compared
with tokens the CPU checker produced for the same full-depth model (tests/golden/greedy_golden.npz).
`--impl reference` times the CPU restatement of the reference's path (the reference itself is Rust and
cannot be built here) on the host cores.
"""
import argparse
import json
import os
import re
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    # name: (kind, dict of dims)
    "llama3-8b": ("llama", dict(V=128256, d=4096, ffn=14336, L=32, H=32, KV=8, hd=128, max_pos=2048, theta=500000.0, tied=False)),
    "tinyllama-1.1b": ("llama", dict(V=32000, d=2048, ffn=5632, L=22, H=32, KV=4, hd=64, max_pos=2048, theta=10000.0, tied=False)),
    "smollm2-135m": ("llama", dict(V=49152, d=576, ffn=1536, L=30, H=9, KV=3, hd=64, max_pos=2048, theta=10000.0, tied=True)),
    "gpt2-small": ("gpt2", dict(V=50257, n_pos=1024, d=768, L=12, H=12)),
}
DEFAULT_CTX = {"llama3-8b": 1024, "tinyllama-1.1b": 512, "smollm2-135m": 64, "gpt2-small": 16}
# measured alongside the default workload and carried in `other_workloads` of its line
OTHER_WORKLOADS = ["llama3-8b-int8-b1", "llama3-8b-int4-b16", "llama3-8b-int8-b16", "llama3-8b-int4-b128", "llama3-8b-int4-prefill1024",
                   "tinyllama-1.1b-int4-b1", "tinyllama-1.1b-int4-b64", "tinyllama-1.1b-int4-prefill512",
                   "smollm2-135m-int8-b1", "smollm2-135m-int4-b16", "gpt2-small-int8-b1"]
ARITHMETIC = ("f32 in and out; inside the GEMV the activations are block fixed point (int4 weights: 21 bits per group of 32; "
              "int8 weights: 28 bits per row of a CTA's slice), products exact in tcgen05 kind::i8, one f32 scale multiply-add "
              "per group, split-k sums met in 64-bit fixed point")
# steps of 5..16 sequences (and prefill-sized row counts): another arithmetic
ARITHMETIC_WIDE = ("f32 in and out; inside the Linears the activations are two bf16 pieces x = hi + lo (16 significant bits), the int4 / "
                   "int8 weights exact in bf16, products and sums in f32 in tcgen05 kind::f16, one f32 scale multiply-add per group "
                   "(int8: per column); Linears below 4M weights keep the block-fixed-point kernels")


def parse_workload(name):
    m = re.fullmatch(r"(.+)-int(8|4)-(b|prefill)(\d+)(?:-ctx(\d+))?", name)
    if not m or m.group(1) not in MODELS:
        raise SystemExit(f"unknown workload {name!r}; expected <{'|'.join(MODELS)}>-int<8|4>-b<B>[-ctx<len>] or ...-prefill<T>")
    model = m.group(1)
    prefill = m.group(3) == "prefill"
    return model, int(m.group(2)), (1 if prefill else int(m.group(4))), (int(m.group(4)) if prefill else int(m.group(5) or DEFAULT_CTX[model])), prefill


def make_cfg(mod, model, layers=None):
    kind, c = MODELS[model]
    if kind == "llama":
        return mod.LlamaConfig(c["V"], c["d"], c["ffn"], layers or c["L"], c["H"], c["KV"], c["hd"], c["max_pos"], 1e-5, c["theta"], int(c["tied"]))
    return mod.GPT2Config(c["V"], c["n_pos"], c["d"], layers or c["L"], c["H"])


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
        return float(j["hbm_gbs"]), float(j.get("bf16_tflops_sustained", 1398.3)), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return 6650.0, 1400.0, "fallback (6.65 TB/s, 1.4 PFLOP/s sustained: earlier measurements on this pool)"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def host_threads():
    """Host threads the CPU checker may use: all of the box's cores, whatever OMP_NUM_THREADS a launcher exported."""
    import oracle
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except Exception:
        pass
    oracle.set_threads(n)
    return oracle.threads()


def cpu_sample(model, bits, B, ctx, budget_s=20.0):
    """The checker (CPU restatement of the reference's path) timed on this host's cores on a bounded sample of the
    workload: the same widths, vocabulary, batch and context (zero keys and values), 2 layers and 1 layer, and the
    result scaled to the full layer count (layer time x L + head/embedding time)."""
    import oracle
    kind, c = MODELS[model]
    L_full = c["L"]
    threads = host_threads()
    t0 = time.time()
    tok = np.zeros((B, 1), np.int32)

    def step_time(layers):
        m = oracle.Model(make_cfg(oracle, model, layers=layers), seed=0, bits=bits, group=32)
        m.cache_assume(B, ctx)
        m.forward_cached(tok)
        n, t1 = 0, time.time()
        while n < 2 or (time.time() - t1 < budget_s / 4 and n < 8):
            m.cache_assume(B, ctx)
            m.forward_cached(tok)
            n += 1
        dt = (time.time() - t1) / n
        m.close()
        return dt, n

    t_two, n2 = step_time(min(2, L_full))
    t_one, n1 = step_time(1)
    t_layer = max(t_two - t_one, 1e-9) / max(min(2, L_full) - 1, 1)
    t_head = max(t_one - t_layer, 0.0)
    t_full = t_head + t_layer * L_full
    return {"value": B / t_full, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"oracle (C++ restatement of the reference's CPU path, OpenMP, {threads} threads): {n2}+{n1} decode steps at batch {B}, "
                      f"{ctx} cached positions, on 2-layer and 1-layer models of the full widths; per-layer and head times scaled to "
                      f"{L_full} layers ({time.time() - t0:.0f} s in all, builds included)"}


def reference_arm(model, bits, B, ctx, K, W, prefill):
    """`--impl reference`: the checker on the FULL model (all layers), the stated batch and context, all host threads."""
    import oracle
    kind, c = MODELS[model]
    threads = host_threads()
    t0 = time.time()
    m = oracle.Model(make_cfg(oracle, model), seed=0, bits=bits, group=32)
    build_s = time.time() - t0
    if prefill:
        ids = oracle.synth_tokens(0, 0x20000000, ctx, c["V"])[None, :]
        t1 = time.time()
        m.forward_cached(ids)
        dt = time.time() - t1
        return ctx / dt, 1, 0, threads, f"one prefill of {ctx} tokens through all {c['L']} layers (build {build_s:.0f} s not timed)"
    tok = np.zeros((B, 1), np.int32)
    m.cache_assume(B, ctx)
    warm = min(W, 1)
    for _ in range(warm):
        m.forward_cached(tok)
    steps, t1 = 0, time.time()
    while steps < K and (steps < 2 or time.time() - t1 < 45.0):  # bounded: about 45 s of stepping
        m.forward_cached(tok)
        steps += 1
    dt = (time.time() - t1) / steps
    return B / dt, steps, warm, threads, (f"all {c['L']} layers, batch {B}, {ctx} cached positions (zero keys and values), {steps} steps "
                                          f"after {warm} warm-up (build {build_s:.0f} s not timed)")


def golden_tokens(model, bits):
    try:
        g = np.load(os.path.join(ROOT, "tests", "golden", "greedy_golden.npz"))
        key = f"{model}-int{bits}"
        return g[key + "/ids"], g[key + "/margin"]
    except Exception:
        return None, None


def greedy_check(nn, m, model, bits, gather=None):
    """Greedy tokens of this (possibly sharded) model against the checker's tokens for the same full-depth model."""
    ids, margin = golden_tokens(model, bits)
    if ids is None:
        return {"checked": False, "why": f"no golden tokens for {model}-int{bits}"}
    prompt_len = 16
    n_new = len(ids) - prompt_len
    got = m.generate(ids[:prompt_len], n_new)
    same = 0
    for a, b in zip(ids[prompt_len:], got[prompt_len:]):
        if a != b:
            break
        same += 1
    res = {"checked": True, "against": "tests/golden/greedy_golden.npz (CPU checker, full depth, prompt 16)", "tokens": int(n_new),
           "identical_prefix": int(same), "ok": bool(same == n_new), "min_top2_margin": float(margin.min())}
    if gather is not None:
        all_ids = gather(got.tolist())
        res["ranks_agree"] = bool(all(x == all_ids[0] for x in all_ids))
        res["ok"] = bool(res["ok"] and res["ranks_agree"])
    m.cache_clear()
    return res


def time_regions(dev, run_region, barrier, regions):
    out = []
    for _ in range(regions):
        barrier()
        dev.timer_start()
        run_region()
        out.append(dev.timer_stop_ms())
    return out


def run_workload(nn, dev, name, K, W, regions, rank=0, world=1, dist=None, local_rank=0, headline=False, layers=None, persistent=False):
    """Loads the model of `name`, times it; returns the fields of its result."""
    model, bits, B, ctx, prefill = parse_workload(name)
    kind, dims = MODELS[model]
    peak, peak_tf, peak_src = measured_peaks()
    t0 = time.time()
    cfg = make_cfg(nn, model, layers=layers)
    m = nn.Llama(dev, cfg, nn.TP(rank, world) if world > 1 else None) if kind == "llama" else nn.GPT2(dev, cfg)
    m.load_synthetic(0, bits, 32)
    if persistent:
        m.use_persistent_step(True)
    if world > 1:
        handles = [None] * world
        dist.all_gather_object(handles, m.tp_export())
        m.tp_connect(handles)
        dist.barrier()
    load_s = time.time() - t0

    def barrier():
        dev.synchronize()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        import torch
        t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    res = {"workload": name, "load_seconds": load_s}
    V = dims["V"]
    if prefill:
        T = ctx
        ids = np.stack([np.arange(T, dtype=np.int32) * 7919 % V])
        for _ in range(2):
            m.cache_clear()
            m.forward_cached(ids, want_logits=False)
        ms = []
        for _ in range(max(3, min(regions, 5))):
            m.cache_clear()
            barrier()
            dev.timer_start()
            m.forward_cached(ids, want_logits=False)
            ms.append(max_over_ranks(dev.timer_stop_ms()))
        med = float(np.median(ms))
        c = dims
        nq, nkv = c["H"] * c["hd"], c["KV"] * c["hd"]
        lin_flops = 2.0 * T * c["L"] * (c["d"] * (nq + 2 * nkv) + nq * c["d"] + 3 * c["d"] * c["ffn"]) + 2.0 * c["d"] * V
        res.update({"metric": "prefill tokens/s", "value": T / (med / 1000.0), "unit": "tokens/s", "ms": med, "ms_min": float(min(ms)),
                    "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel (tcgen05 kind::f16 dequant GEMM) + attention", "achieved": lin_flops / (med / 1000.0) / 1e12,
                                 "peak": peak_tf, "unit": "TFLOP/s", "frac": lin_flops / (med / 1000.0) / 1e12 / peak_tf,
                                 "flops": "2 m k n of the quantized Linears (the hi/lo split of the activations is overhead, not counted)",
                                 "peak_source": peak_src + " bf16 sustained"}})
        m.close()
        return res

    parity = None
    if headline and kind == "llama" and not layers:
        gather = None
        if dist is not None:
            def gather(x):
                out = [None] * world
                dist.all_gather_object(out, x)
                return out
        parity = greedy_check(nn, m, model, bits, gather)

    ids0 = np.array([int(x) for x in range(B)], np.int32) % V
    ids_dev = nn.Tensor.from_numpy(dev, ids0)
    max_pos = dims.get("max_pos", dims.get("n_pos"))
    ctx = min(ctx, max_pos - (K + W + 9))
    m.cache_reserve(B, min(max_pos, ctx + K + W + 8))  # no growth while timing
    m.cache_assume(B, ctx)
    m.decode_step(B, ids_dev.ptr, fetch=True)
    for _ in range(W - 1):
        m.decode_step(B, None, fetch=False)
    barrier()
    sampler = ClockSampler(local_rank) if headline else None
    if sampler:
        sampler.start()

    def region():
        m.cache_assume(B, ctx)
        dev.synchronize()

    ms_all = []
    for _ in range(regions):
        region()
        barrier()
        dev.timer_start()
        for _ in range(K):
            m.decode_step(B, None, fetch=False)
        ms_all.append(max_over_ranks(dev.timer_stop_ms()))
    barrier()
    clocks = sampler.stop() if sampler else None
    ms = float(np.median(ms_all))
    launches = m.step_launches()
    step_bytes = m.step_bytes(B, ctx + K // 2)
    step_gbs = step_bytes / (ms / K / 1000.0) / 1e9
    res.update({"metric": "decode tokens/s", "value": B * K / (ms / 1000.0), "unit": "tokens/s", "ms_per_step": ms / K,
                "ms_per_step_min": float(min(ms_all)) / K, "regions": regions, "launches_per_step": launches, "context": ctx,
                "clocks": clocks, "parity": parity, "step_bytes": step_bytes, "step_gbs": step_gbs, "step_frac": step_gbs / peak})

    # ---- host-buffer path: `e2e` ----
    if headline:
        if world == 1:
            m.cache_assume(B, ctx)
            tok = ids0.reshape(B, 1).copy()
            for _ in range(3):
                logits = m.forward_cached(tok)
            m.cache_assume(B, ctx)
            barrier()
            dev.timer_start()
            for _ in range(K):
                logits = m.forward_cached(tok)                 # H2D ids, the step, D2H logits
                tok = logits.argmax(axis=1).astype(np.int32).reshape(B, 1)
            ms_e2e = dev.timer_stop_ms()
            res["e2e"] = {"value": B * K / (ms_e2e / 1000.0), "unit": "tokens/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B * V,
                          "ms_per_step": ms_e2e / K, "call": "forward_cached(ids_host [B,1]) -> logits_host [B,V], host argmax"}
        else:
            m.cache_assume(B, ctx)
            for _ in range(3):
                nxt = m.decode_step(B, ids_dev.ptr, fetch=True)
            m.cache_assume(B, ctx)
            barrier()
            dev.timer_start()
            nxt = ids0
            for _ in range(K):
                t = nn.Tensor.from_numpy(dev, nxt)             # H2D ids
                nxt = m.decode_step(B, t.ptr, fetch=True)      # D2H next ids
            ms_e2e = max_over_ranks(dev.timer_stop_ms())
            res["e2e"] = {"value": B * K / (ms_e2e / 1000.0), "unit": "tokens/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                          "ms_per_step": ms_e2e / K, "call": "decode_step(ids from host) -> next ids to host, every step"}

    # ---- the dominant kernel ----
    if launches == 1:
        traffic = None
        try:
            with open(os.path.join(ROOT, "profiles", "pstep_traffic.json")) as f:
                tr = json.load(f).get(f"int{bits}")
                if tr:
                    traffic = tr["dram_bytes_per_algorithmic_byte"] * step_bytes
        except Exception:
            pass
        res["roofline"] = {"bound": "hbm", "kernel": f"pstep_kernel<rows<={max(B, 1)}> (the whole decode step as one persistent cooperative kernel)",
                           "achieved": step_gbs, "peak": peak, "unit": "GB/s", "frac": step_gbs / peak, "peak_source": peak_src + " hbm_gbs",
                           "traffic": traffic, "bytes_per_launch": step_bytes, "us_per_launch": 1000.0 * ms / K, "launches_timed": K * regions,
                           "per_gpu": True, "frac_of_nominal_8TBs": step_gbs / 8000.0}
    else:
        iters = max(3, min(20, K // 8))
        lin_ms, lin_launches, lin_bytes = m.time_linears(B, iters)
        barrier()
        lin_ms = max_over_ranks(lin_ms)
        achieved = lin_bytes / (lin_ms / 1000.0) / 1e9
        traffic = None
        try:
            # DRAM bytes per algorithmic byte from one ncu capture per kernel family (narrow: up to 4 rows; 16-row tile: 5..16)
            with open(os.path.join(ROOT, "profiles", "gemv_traffic.json" if B <= 4 else "gemv_wide_traffic.json")) as f:
                tr = json.load(f).get(f"int{bits}")
                if tr and B <= 16:
                    traffic = tr["dram_bytes_per_algorithmic_byte"] * lin_bytes / lin_launches
        except Exception:
            pass
        if B > 16:
            kname = "gemm_tc_kernel (tcgen05 kind::f16 dequant GEMM, every Linear of the model)"
        elif B >= 5:
            kname = f"gemv_wide_kernel<{bits}> + xsplit16_kernel (tcgen05 kind::f16, one 16-row tile, weights streamed once; Linears of 4M weights and more)"
        elif bits == 4:
            kname = f"gemv_tc_int4_kernel<rows<={min(B, 8)}> (tcgen05 kind::i8 fused dequant GEMV; the int8 head runs gemv_tc_int8_kernel)"
        else:
            kname = f"gemv_tc_int8_kernel<rows<={min(B, 8)}> (tcgen05 kind::i8 fused dequant GEMV, every Linear of the model)"
        res["roofline"] = {"bound": "hbm", "kernel": kname, "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                           "peak_source": peak_src + " hbm_gbs", "traffic": traffic, "bytes_per_launch": lin_bytes / lin_launches,
                           "us_per_launch": 1000.0 * lin_ms / lin_launches, "launches_timed": lin_launches * iters, "per_gpu": True,
                           "note": "the quantized Linears of one step timed back to back (zero activations, no norm prologue: the bytes are the same)",
                           "whole_step": {"achieved": step_gbs, "frac": step_gbs / peak, "bytes_per_step_per_gpu": step_bytes,
                                          "frac_of_nominal_8TBs": step_gbs / 8000.0}}
    # ---- the same steps as ONE persistent cooperative kernel per token (opt-in implementation of the step) ----
    if headline and world == 1 and kind == "llama" and B <= 2 and not layers and not persistent:
        m.use_persistent_step(True)
        if m.uses_persistent_step(B):
            par2 = greedy_check(nn, m, model, bits, None)
            m.cache_reserve(B, min(max_pos, ctx + K + W + 8))
            m.cache_assume(B, ctx)
            m.decode_step(B, ids_dev.ptr, fetch=True)
            for _ in range(W - 1):
                m.decode_step(B, None, fetch=False)
            ms2 = []
            for _ in range(max(3, min(regions, 6))):
                region()
                barrier()
                dev.timer_start()
                for _ in range(K):
                    m.decode_step(B, None, fetch=False)
                ms2.append(dev.timer_stop_ms())
            med2 = float(np.median(ms2))
            gbs2 = step_bytes / (med2 / K / 1000.0) / 1e9
            res["persistent_step"] = {"value": B * K / (med2 / 1000.0), "unit": "tokens/s", "ms_per_step": med2 / K, "launches_per_step": m.step_launches(),
                                      "regions": len(ms2), "achieved_gbs": gbs2, "frac": gbs2 / peak, "parity": par2,
                                      "kernel": "pstep_kernel (the whole step as one cooperative launch; ruai_model_use_persistent_step)"}
        m.use_persistent_step(False)
    m.close()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default="llama3-8b-int4-b1")
    ap.add_argument("--impl", default="ruai_b200", choices=["ruai_b200", "reference"])
    ap.add_argument("--regions", type=int, default=12, help="timed regions of exactly --steps steps; the median is reported")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="skip the other workloads measured alongside the default one")
    ap.add_argument("--profile-layers", type=int, default=0,
                    help="profiling aid (not a benchmark configuration): build the model with this many layers so that a profiler's capture stays small; "
                         "the line says so in config.layers and skips the golden-token check")
    ap.add_argument("--persistent", action="store_true", help="profiling aid: time the persistent one-launch step as the main measurement")
    args = ap.parse_args()
    model, bits, B, ctx, prefill = parse_workload(args.workload)
    kind, dims = MODELS[model]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    W = max(args.warmup, 3)
    K = max(args.steps, 1)
    config = {"workload": args.workload, "model_shape": model, "layers": dims["L"], "weights": f"int{bits}" + (" group 32, int8 head" if bits == 4 else ""),
              "batch": B, "context": ctx, "kv_dtype": "f32", "activations": ARITHMETIC if B <= 4 else ARITHMETIC_WIDE,
              "parallelism": f"tp{world}" if world > 1 else "single GPU",
              "l2": "every step streams the whole quantized model (far larger than the 126 MB L2), so no flush is needed"}

    if args.impl == "reference":
        if rank != 0:
            return
        value, steps, warm, threads, sample = reference_arm(model, bits, B, ctx, K, W, prefill)
        cb = {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
        line = {"impl": "reference", "metric": "prefill tokens/s" if prefill else "decode tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": steps, "warmup": warm, "steps_requested": K, "warmup_requested": W,
                "ms_per_step": 1000.0 * B / value, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": "CPU restatement of the reference's quantized path (the reference is Rust; no Rust toolchain exists here), all host threads"}
        print(json.dumps(line))
        return

    from ruai_b200 import nn
    dist = None
    if world > 1:
        if kind != "llama":
            raise SystemExit("only the Llama models shard")
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = nn.Device.cuda(local_rank)
    if args.profile_layers:
        config["layers"] = args.profile_layers
        config["note"] = "reduced layer count for a profiler capture: not a benchmark configuration"
    r = run_workload(nn, dev, args.workload, K, W, max(args.regions, 1), rank, world, dist, local_rank, headline=True,
                     layers=args.profile_layers or None, persistent=args.persistent)
    others = []
    if world == 1 and not args.no_others and args.workload == "llama3-8b-int4-b1":
        for name in OTHER_WORKLOADS:
            try:
                o = run_workload(nn, dev, name, min(K, 32), 3, 3)
                keep = {k: o[k] for k in ("workload", "metric", "value", "unit", "ms_per_step", "ms", "launches_per_step", "context", "step_frac") if k in o}
                keep["roofline"] = {k: o["roofline"][k] for k in ("bound", "kernel", "achieved", "peak", "unit", "frac") if k in o.get("roofline", {})}
                others.append(keep)
            except Exception as e:  # one workload failing must not cost the headline line
                others.append({"workload": name, "error": str(e)[:200]})
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    config["context"] = r.get("context", ctx)
    line = {"metric": r["metric"], "value": r["value"], "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": r.get("ms_per_step", r.get("ms")), "ms_per_step_min": r.get("ms_per_step_min"), "timed_regions": r.get("regions"),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config, "clocks": r.get("clocks"), "e2e": r.get("e2e"), "gpu_launches": (r.get("launches_per_step") or 0) * K * (r.get("regions") or 1),
            "launches_per_step": r.get("launches_per_step"), "roofline": r.get("roofline"), "load_seconds": r["load_seconds"]}
    if r.get("parity") is not None:
        line["tp_parity" if world > 1 else "parity"] = r["parity"]
    if r.get("persistent_step") is not None:
        line["persistent_step"] = r["persistent_step"]
    if others:
        line["other_workloads"] = others
    if world == 1 and not args.no_cpu_baseline and not prefill:
        line["cpu_baseline"] = cpu_sample(model, bits, B, ctx)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
