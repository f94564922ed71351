#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Llama 3.2 1B shape, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

Prints ONE JSON line.  A step is one decode step of ``--batch`` requests, each with a
512-token prompt in the cache and up to 256 generated tokens.  ``value`` is decoded
tokens per second timed on the device; ``e2e`` is the same through the Python entry
point (``ContinuousBatchEngine.step``), token ids from the host in and sampled ids back
every step.  The weights are random (seeded), the token ids synthetic.

``--impl reference`` would run lumia431/photon_infer itself; it cannot be installed
here (see the ``unavailable`` line it prints).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The sizes of the Llama 3.2 1B shape (the third configuration of BASELINE.json).
LLAMA_1B = dict(
    architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=128256,
    max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=True, bos_token_id=128000, eos_token_id=128001)
PROMPT_LEN, GEN_LEN, CONTEXT, PREFILL_TOKENS = 512, 256, 4096, 2048
PUBLISHED_BATCH8_TOK_S = 720.0       # the reference's README: batch 8, A100, INT8 weights

REFERENCE_UNAVAILABLE = ("lumia431/photon_infer is a CMake/C++ project without a Python package (pip finds no "
                         "setup.py or pyproject.toml) and needs glog, Eigen and gtest, which are not installed; "
                         "no network")


def peaks():
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            hbm = float(d.get("hbm_gbs", hbm))
            tf = float(d.get("bf16_tflops", tf))
            src = "measured"
        except (ValueError, OSError):
            pass
    return hbm, tf, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.monotonic(), line.strip()))

    def window(self, t0, t1):
        rows = [s for t, s in self.samples if t0 <= t <= t1] or [s for _, s in self.samples[-3:]]
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            parts = [p.strip() for p in r.split(",")]
            try:
                sm.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except (ValueError, IndexError):
                continue
            for n, p in zip(names, parts[2:]):
                if p.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=LLAMA_1B["num_hidden_layers"])
    ap.add_argument("--impl", default="photon_b200", choices=["photon_b200", "reference"])
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one phase only (for profiling); the JSON line then lacks the other figures")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    args.steps = max(1, min(args.steps, GEN_LEN - args.warmup - 1))

    import torch
    from photon_infer_b200 import EngineOptions
    from photon_infer_b200.engine.engine import ContinuousBatchEngine
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    from photon_infer_b200.kernels import ops
    from photon_infer_b200.weights import write_random_model

    hbm_peak, tf_peak, peak_src = peaks()
    cfg = dict(LLAMA_1B, num_hidden_layers=args.layers)
    torch.manual_seed(0)
    clocks = ClockSampler()
    clocks.start()
    with tempfile.TemporaryDirectory(prefix="photon_bench_") as folder:
        t_w = time.time()
        write_random_model(folder, cfg, seed=0, init_std=0.02, norm_std=0.0)
        print(f"[bench] random weights written in {time.time() - t_w:.1f} s", file=sys.stderr, flush=True)
        max_b = args.batch if args.no_points else max(args.batch, 64)
        options = EngineOptions(dtype=args.dtype, block_size=args.block_size,
                                max_cache_tokens=max_b * (PROMPT_LEN + GEN_LEN + args.block_size),
                                max_sequences=max_b, max_batch_size=max_b, chunk_size=PREFILL_TOKENS,
                                max_num_batched_tokens=max(PREFILL_TOKENS, max_b * PROMPT_LEN // 8),
                                max_model_len=CONTEXT, use_cuda_graphs=not args.no_graphs)
        runner = build_runner(folder, options)
    model, cache = runner.model, runner.cache
    vocab = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(1)

    def rand_ids(n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    def fill(batch):
        """Prompts of PROMPT_LEN tokens into the cache, a few requests per step."""
        for i in range(batch):
            cache.add_request(("d", i))
        per = max(1, options.max_num_batched_tokens // PROMPT_LEN)
        for lo in range(0, batch, per):
            runner.step([StepEntry(("d", i), rand_ids(PROMPT_LEN), []) for i in range(lo, min(batch, lo + per))])

    def decode_region(batch, steps, warmup):
        """Device-timed decode steps: tokens in, logits, sampled ids on the device."""
        fill(batch)
        ids = [rand_ids(batch) for _ in range(steps + warmup)]
        greedy = ([0.0] * batch, [0.0] * batch)
        def one(k):
            return runner.step([StepEntry(("d", i), [ids[k][i]], [0]) for i in range(batch)], sampling=greedy).tokens
        for k in range(warmup):
            one(k)
        torch.cuda.synchronize()
        launches0 = ops.launch_count() + runner.graph_kernel_launches
        kv_bytes = cache.cached_bytes([("d", i) for i in range(batch)])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.monotonic()
        torch.cuda.profiler.start()          # for `ncu --profile-from-start off`; no effect otherwise
        e0.record()
        for k in range(warmup, warmup + steps):
            one(k)
        e1.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        t1 = time.monotonic()
        ms = e0.elapsed_time(e1)
        kv_bytes = (kv_bytes + cache.cached_bytes([("d", i) for i in range(batch)])) // 2
        launches = ops.launch_count() + runner.graph_kernel_launches - launches0
        runner.check_device_errors()
        for i in range(batch):
            cache.free_request(("d", i))
        return ms / steps, kv_bytes, launches, (t0, t1)

    # ---- prefill of 2,048 tokens (one request, one step), timed alone
    prompt = rand_ids(PREFILL_TOKENS)
    pf_ms = []
    for rep in range(4 if args.only != "decode" else 0):
        cache.add_request("p")
        torch.cuda.synchronize()
        if rep == 3 and args.only == "prefill":
            torch.cuda.profiler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry("p", prompt, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        if rep == 3 and args.only == "prefill":
            torch.cuda.profiler.stop()
        pf_ms.append(e0.elapsed_time(e1))
        cache.free_request("p")
    prefill_ms = min(pf_ms[1:]) if pf_ms else float("nan")
    H, I, L, d = cfg["hidden_size"], cfg["intermediate_size"], args.layers, cfg["head_dim"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    per_token = 2 * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    attn = 4 * nq * d * (PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2)          # QK^T and PV over the causal half
    prefill_flops = L * (PREFILL_TOKENS * per_token + attn) + 2 * H * vocab
    prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3), "frac": round(prefill_flops / (prefill_ms / 1e3) / (tf_peak * 1e12), 4)}

    if args.only == "prefill":
        clocks.stop()
        print(json.dumps({"only": "prefill", "prefill": prefill}))
        return 0
    # ---- the headline: decode at --batch
    ms_step, kv_bytes, launches, (t0, t1) = decode_region(args.batch, args.steps, args.warmup)
    clock_info = clocks.window(t0, t1)
    value = args.batch / (ms_step / 1e3)
    step_bytes = model.step_weight_bytes() + kv_bytes
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    if args.only == "decode":
        clocks.stop()
        print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": round(ms_step, 4),
                          "value": round(value, 1), "roofline_frac": round(achieved / hbm_peak, 4),
                          "gpu_launches": launches}))
        return 0
    points = {}
    if not args.no_points:
        for b in (1, 64):
            m, _, _, _ = decode_region(b, min(args.steps, 64), args.warmup)
            points[f"decode_b{b}"] = round(b / (m / 1e3), 1)

    # ---- end to end through the entry point: host ids in, sampled ids out, every step
    engine = ContinuousBatchEngine(None, options, runner=runner)
    for i in range(args.batch):
        engine.add_request(rand_ids(PROMPT_LEN), max_new_tokens=args.warmup + args.steps + 16, ignore_eos=True)
    while any(r.num_generated() < 1 for r in engine.scheduler.requests.values()):
        engine.step()
    for _ in range(args.warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d0, d2h0 = runner.h2d_bytes, engine.d2h_bytes
    w0 = time.perf_counter()
    for _ in range(args.steps):
        engine.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - w0
    e2e = {"value": round(args.batch * args.steps / e2e_s, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": (runner.h2d_bytes - h2d0) // args.steps,
           "d2h_bytes_per_step": (engine.d2h_bytes - d2h0) // args.steps}
    clocks.stop()

    line = {
        "metric": "decode tokens/s, Llama 3.2 1B shape, batch %d" % args.batch,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / PUBLISHED_BATCH8_TOK_S, 2) if args.batch == 8 else None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic token ids, random weights N(0, 0.02)",
        "impl": "photon_b200",
        "config": {"model": "llama-3.2-1b-shape", "layers": args.layers, "layers_of_model": LLAMA_1B["num_hidden_layers"],
                   "hidden": H, "q_heads": nq, "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": vocab,
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "generated": GEN_LEN,
                   "page_size": args.block_size, "parallelism": "single", "cuda_graphs": not args.no_graphs,
                   "l2": "weights 2.5 GB per step exceed L2", "peaks": peak_src},
        "clocks": clock_info,
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
