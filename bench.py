#!/usr/bin/env python
"""Decode-throughput benchmark of the quantized-inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one greedy decode step (one new token for each of the B sequences) through the
captured decode graph.  The default workload is the one the headline target is quoted on:
the Llama-3-8B-shaped model, int4 (group 32) weights with an int8 head, batch 1, 1024 cached
positions.  Weights are seeded synthetic N(0, 0.02^2) generated and quantized on the device;
nothing is read from disk.  With N > 1 (launched by torch.distributed.run, one process per
GPU) the same model is sharded Megatron-style over the N GPUs (strong scaling).

Prints one JSON line (rank 0).  `value` is measured with the ids resident on the device;
`e2e` goes through the host-buffer call `forward_cached(ids_host) -> logits_host` plus the
host-side argmax per token, which is the reference's own generate loop (generation.rs:102-104).
`--impl reference` times the CPU restatement of the reference's path (the reference itself is
Rust and cannot be built here) on the host cores, on a bounded layer-reduced sample.
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


def parse_workload(name):
    m = re.fullmatch(r"(.+)-int(8|4)-b(\d+)(?:-ctx(\d+))?", name)
    if not m or m.group(1) not in MODELS:
        raise SystemExit(f"unknown workload {name!r}; expected <{'|'.join(MODELS)}>-int<8|4>-b<B>[-ctx<len>]")
    model = m.group(1)
    return model, int(m.group(2)), int(m.group(3)), int(m.group(4) or DEFAULT_CTX[model])


def make_cfg(mod, model, layers=None):
    kind, c = MODELS[model]
    if kind == "llama":
        return mod.LlamaConfig(c["V"], c["d"], c["ffn"], layers or c["L"], c["H"], c["KV"], c["hd"], c["max_pos"], 1e-5, c["theta"], int(c["tied"]))
    return mod.GPT2Config(c["V"], c["n_pos"], c["d"], layers or c["L"], c["H"])


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
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
        time.sleep(0.15)
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


def cpu_reference(model, bits, B, ctx, steps, warmup):
    """The checker (CPU restatement of the reference's path) timed on this host's cores on a bounded sample:
    the same widths, vocabulary and batch with 2 layers, a short context, and the result scaled to the
    full layer count (layer time x L + head/embedding time)."""
    import oracle
    kind, c = MODELS[model]
    L_full = c["L"]
    L_s = min(2, L_full)
    ctx_s = min(ctx, 16)
    cores = os.cpu_count() or 1
    t0 = time.time()
    m0 = oracle.Model(make_cfg(oracle, model, layers=L_s), seed=0, bits=bits, group=32)
    build_s = time.time() - t0
    ids = np.stack([oracle.synth_tokens(0, 0x20000000 + b, ctx_s, c["V"]) for b in range(B)])
    m0.forward_cached(ids)
    tok = np.zeros((B, 1), np.int32)
    n = max(1, min(steps, 4))
    for _ in range(min(warmup, 1)):
        m0.forward_cached(tok)
    t0 = time.time()
    for _ in range(n):
        m0.forward_cached(tok)
    t_small = (time.time() - t0) / n
    # head + embedding + final norm alone: a 0-layer model would need another build; estimate from a 1-layer one
    m1 = oracle.Model(make_cfg(oracle, model, layers=1), seed=0, bits=bits, group=32)
    m1.forward_cached(ids)
    t0 = time.time()
    for _ in range(n):
        m1.forward_cached(tok)
    t_one = (time.time() - t0) / n
    t_layer = max(t_small - t_one, 1e-9) / max(L_s - 1, 1)
    t_head = max(t_one - t_layer, 0.0)
    t_full = t_head + t_layer * L_full
    return {"value": B / t_full, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"oracle (C++ restatement, OpenMP {cores} threads): {n} decode steps at batch {B}, context {ctx_s}, on {L_s}-layer and 1-layer "
                      f"models of the full widths; per-layer and head times scaled to {L_full} layers (build {build_s:.1f} s not timed)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default="llama3-8b-int4-b1")
    ap.add_argument("--impl", default="ruai_b200", choices=["ruai_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    model, bits, B, ctx = parse_workload(args.workload)
    kind, dims = MODELS[model]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    W = max(args.warmup, 3)
    K = max(args.steps, 1)
    config = {"workload": args.workload, "model_shape": model, "weights": f"int{bits}" + (" group 32, int8 head" if bits == 4 else ""),
              "batch": B, "context": ctx, "kv_dtype": "f32", "activations": "f32",
              "parallelism": f"tp{world}" if world > 1 else "single GPU",
              "l2": "every step streams the whole quantized model (far larger than the 126 MB L2), so no flush is needed"}

    if args.impl == "reference":
        if rank != 0:
            return
        cb = cpu_reference(model, bits, B, ctx, K, W)
        line = {"impl": "reference", "metric": "decode tokens/s", "value": cb["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": K, "warmup": W,
                "ms_per_step": 1000.0 * B / cb["value"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": "CPU restatement of the reference's quantized path (the reference is Rust; no Rust toolchain exists here)"}
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
    cfg = make_cfg(nn, model)
    t0 = time.time()
    if kind == "llama":
        m = nn.Llama(dev, cfg, nn.TP(rank, world) if world > 1 else None)
    else:
        m = nn.GPT2(dev, cfg)
    m.load_synthetic(0, bits, 32)
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

    ids0 = np.array([int(x) for x in range(B)], np.int32) % dims["V"]
    ids_dev = nn.Tensor.from_numpy(dev, ids0)

    # ---- device-resident decode: `value` ----
    m.cache_reserve(B, min(dims.get("max_pos", dims.get("n_pos")), ctx + K + W + 8))  # no growth, no re-capture while timing
    m.cache_assume(B, ctx)
    m.decode_step(B, ids_dev.ptr, fetch=True)            # captures the graph
    for _ in range(W - 1):
        m.decode_step(B, None, fetch=False)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    m.cache_assume(B, ctx)
    barrier()
    dev.timer_start()
    for _ in range(K):
        m.decode_step(B, None, fetch=False)
    ms = dev.timer_stop_ms()
    barrier()
    ms = max_over_ranks(ms)
    clocks = sampler.stop()
    launches = m.step_launches()
    step_bytes_local = m.step_bytes(B, ctx + K // 2)

    # ---- host-buffer path: `e2e` ----
    V = dims["V"]
    e2e = None
    if world == 1:
        m.cache_assume(B, ctx)
        tok = ids0.reshape(B, 1).copy()
        for _ in range(3):
            logits = m.forward_cached(tok)
        m.cache_assume(B, ctx)
        barrier()
        dev.timer_start()
        for _ in range(K):
            logits = m.forward_cached(tok)                 # H2D ids, graph, D2H logits
            tok = logits.argmax(axis=1).astype(np.int32).reshape(B, 1)
        ms_e2e = dev.timer_stop_ms()
        e2e = {"value": B * K / (ms_e2e / 1000.0), "unit": "tokens/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B * V,
               "ms_per_step": ms_e2e / K, "call": "forward_cached(ids_host [B,1]) -> logits_host [B,V], host argmax"}
    else:
        # sharded head: the next ids (not the logits) come back; the host-visible result of a step is the token
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
        e2e = {"value": B * K / (ms_e2e / 1000.0), "unit": "tokens/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
               "ms_per_step": ms_e2e / K, "call": "decode_step(ids from host) -> next ids to host, every step"}

    # ---- the dominant kernel alone: the quantized GEMV over every Linear of the model ----
    peak, peak_src = measured_peak()
    iters = max(3, min(20, K // 8))
    lin_ms, lin_launches, lin_bytes = m.time_linears(B, iters)
    barrier()
    lin_ms = max_over_ranks(lin_ms)
    achieved = lin_bytes / (lin_ms / 1000.0) / 1e9
    step_gbs = step_bytes_local / (ms / K / 1000.0) / 1e9
    traffic = None
    try:
        with open(os.path.join(ROOT, "profiles", "gemv_traffic.json")) as f:
            tr = json.load(f).get(f"int{bits}")
            if tr:
                traffic = tr["dram_bytes_per_algorithmic_byte"] * lin_bytes / lin_launches
    except Exception:
        pass
    if B > 16:
        kname = "gemm_tc_kernel (tcgen05 kind::f16 dequant GEMM, every Linear of the model)"
    elif bits == 4:
        kname = f"gemv_tc_int4_kernel<rows<={min(B, 8)}> (tcgen05 kind::i8 fused dequant GEMV; the int8 head runs gemv_tc_int8_kernel)"
    else:
        kname = f"gemv_tc_int8_kernel<rows<={min(B, 8)}> (tcgen05 kind::i8 fused dequant GEMV, every Linear of the model)"
    roofline = {"bound": "hbm", "kernel": kname,
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                "traffic": traffic, "bytes_per_launch": lin_bytes / lin_launches, "us_per_launch": 1000.0 * lin_ms / lin_launches,
                "launches_timed": lin_launches * iters, "per_gpu": True,
                "whole_step": {"achieved": step_gbs, "frac": step_gbs / peak, "bytes_per_step_per_gpu": step_bytes_local,
                               "frac_of_nominal_8TBs": step_gbs / 8000.0}}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    line = {"metric": "decode tokens/s", "value": B * K / (ms / 1000.0), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config, "clocks": clocks, "e2e": e2e, "gpu_launches": launches * K, "launches_per_step": launches,
            "roofline": roofline, "load_seconds": load_s}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_reference(model, bits, B, ctx, 4, 1)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
