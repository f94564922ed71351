#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Llama 3.2 1B shape, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--workloads all|headline]

Prints ONE JSON line.  A step is one decode step of ``--batch`` requests, each with a
512-token prompt in the cache and up to 256 generated tokens.  ``value`` is decoded
tokens per second timed on the device; ``e2e`` is the same through the Python entry
point (``ContinuousBatchEngine.step``), token ids from the host in and sampled ids back
every step.  The weights are random (seeded), the token ids synthetic.

Two more workloads go into ``points`` of the same line (``--workloads headline`` leaves them out):

* ``llama3b_*``: the Llama 3.2 3B shape under continuous batching: 64 requests with prompts of 128 to
  2,048 tokens and 256 generated tokens each, one request arriving per scheduler step, through
  ``ContinuousBatchEngine.step`` (host ids in, sampled ids out);
* ``llama8b_*``: the Llama 3.1 8B shape at long context: eight prompts of 16,384 tokens fed in portions
  of 2,048, then 256 decode steps of all eight.

``--impl reference`` runs lumia431/photon_infer itself where it could be built (``baseline/``); else it
prints an ``unavailable`` line.
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

# The sizes of the Llama 3.2 1B shape: 16 layers, 2,048 wide, 32/8 heads of 64, vocabulary 128,256.
LLAMA_1B = dict(
    architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=128256,
    max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=True, bos_token_id=128000, eos_token_id=128001)
LLAMA_3B = dict(LLAMA_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, head_dim=128)
LLAMA_8B = dict(LLAMA_1B, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, head_dim=128,
                rope_scaling=dict(LLAMA_1B["rope_scaling"], factor=8.0), tie_word_embeddings=False)
PROMPT_LEN, GEN_LEN, CONTEXT, PREFILL_TOKENS = 512, 256, 4096, 2048
PUBLISHED_BATCH8_TOK_S = 720.0       # the reference's README: batch 8, A100, INT8 weights

REFERENCE_BINARY = os.path.join(ROOT, "baseline", "_ref", "bin", "photon_ref_bench")


def run_reference(args) -> int:
    """The reference arm: lumia431/photon_infer, unmodified, built by ``baseline/build_reference.sh`` with its
    own CMake project, driven through its own API by ``baseline/reference_bench.cpp``.  Nothing of this
    package runs on that path.  Prints the harness's JSON line with the clocks seen meanwhile, or an
    ``unavailable`` line when the binary is not there or does not run."""
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    if args.gpus != 1:
        return unavailable("lumia431/photon_infer runs on one GPU only")
    if not os.path.isfile(REFERENCE_BINARY):
        return unavailable("pip cannot install lumia431/photon_infer (a CMake/C++ project without setup.py or "
                           "pyproject.toml); its CMake build, baseline/build_reference.sh <checkout>, has not been run here")
    clocks = ClockSampler()
    clocks.start()
    t0 = time.monotonic()
    try:
        proc = subprocess.run([REFERENCE_BINARY, "--batch", str(args.batch), "--steps", str(max(1, args.steps)),
                               "--warmup", str(max(3, args.warmup)), "--prompt", str(PROMPT_LEN),
                               "--generated", str(GEN_LEN)],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
    except (OSError, subprocess.TimeoutExpired) as e:
        clocks.stop()
        return unavailable(f"the reference's binary did not run to its end: {type(e).__name__}")
    t1 = time.monotonic()
    clocks.stop()
    sys.stderr.write(proc.stderr[-2000:])
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    if proc.returncode != 0 or not lines:
        return unavailable(f"the reference's binary ended with code {proc.returncode}: {proc.stderr.strip()[-200:]}")
    line = json.loads(lines[-1])
    if "unavailable" not in line:
        # the timed decode steps are the last part of the run
        line["clocks"] = clocks.window(max(t0, t1 - 2.0), t1)
        line["vs_baseline"] = round(line["value"] / PUBLISHED_BATCH8_TOK_S, 2) if args.batch == 8 else None
        line["gpu_launches"] = 0            # none of this package's kernels: the reference's own and cuBLAS
    print(json.dumps(line))
    return 0


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


def layer_flops_per_token(cfg) -> int:
    """Multiply-adds x 2 of the products of one layer for one token (attention over the keys not included)."""
    H, I, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    return 2 * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)


def step_flops(cfg, layers, entries, wanted_rows) -> int:
    """``entries``: (tokens in the step, tokens cached before) per request.  Products of every token, QK^T and
    PV of every token over the keys it sees, the output head on the wanted rows."""
    nq, d = cfg["num_attention_heads"], cfg["head_dim"]
    tokens = sum(n for n, _ in entries)
    keys = sum(n * c + n * (n + 1) // 2 for n, c in entries)
    return layers * (tokens * layer_flops_per_token(cfg) + 4 * nq * d * keys) \
        + 2 * cfg["hidden_size"] * cfg["vocab_size"] * wanted_rows


def run_3b_continuous(args, hbm_peak, tf_peak):
    """Continuous batching at the Llama 3.2 3B shape through the engine's entry point."""
    import torch
    from photon_infer_b200 import EngineOptions
    from photon_infer_b200.engine.engine import ContinuousBatchEngine
    from photon_infer_b200.engine.loading import build_runner, random_model

    n_req, gen, lo, hi = 64, 256, 128, 2048
    cfg = dict(LLAMA_3B, num_hidden_layers=args.layers_3b or LLAMA_3B["num_hidden_layers"])
    layers = cfg["num_hidden_layers"]
    model = random_model(cfg, args.dtype, seed=3)
    options = EngineOptions(dtype=args.dtype, block_size=args.block_size, max_cache_tokens=n_req * (hi + gen + 16),
                            max_sequences=n_req, max_batch_size=n_req, chunk_size=2048, max_num_batched_tokens=2048,
                            max_model_len=CONTEXT, use_cuda_graphs=not args.no_graphs)
    runner = build_runner(None, options, model=model)
    cache = runner.cache
    gen_rng = torch.Generator().manual_seed(33)
    lengths = torch.randint(lo, hi + 1, (n_req,), generator=gen_rng).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=gen_rng).tolist() for n in lengths]

    log = []                                   # per launched step: (call index, [(tokens, cached before)], wanted rows)
    call = [0]
    real_step = runner.step

    def logged_step(entries, **kw):
        log.append((call[0], [(len(e.tokens), cache.length(e.request_id)) for e in entries],
                    sum(len(e.want) for e in entries)))
        return real_step(entries, **kw)
    runner.step = logged_step

    def one_pass(timed):
        engine = ContinuousBatchEngine(None, options, runner=runner)
        pending = list(prompts)
        events = []
        del log[:]
        call[0] = 0
        torch.cuda.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        t0 = time.perf_counter()
        while pending or engine.has_work():
            if pending:                         # one arrival per scheduler step
                engine.add_request(pending.pop(0), max_new_tokens=gen, ignore_eos=True)
            engine.step()
            if timed:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                events.append(ev)
            call[0] += 1
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        runner.check_device_errors()
        done = sum(r.num_generated() for r in engine.scheduler.requests.values())
        assert done == n_req * gen, (done, n_req * gen)
        return wall, start, events, engine

    one_pass(False)                             # modules, graphs of every batch size and table width
    h2d0 = runner.h2d_bytes
    wall, start, events, engine = one_pass(True)
    # device time between the events of consecutive calls belongs to the step launched in the later call
    ms = [(events[i - 1] if i else start).elapsed_time(events[i]) for i in range(len(events))]
    weight_bytes = model.step_weight_bytes()
    kv_per_token = cache.bytes_per_token()
    dec_ms = dec_bytes = dec_steps = dec_tokens = 0
    mix_ms = mix_flops = mix_steps = mix_tokens = 0
    for idx, entries, wanted in log:
        if all(n == 1 for n, _ in entries):
            dec_ms += ms[idx]
            dec_bytes += weight_bytes + kv_per_token * sum(c + 1 for _, c in entries)
            dec_steps += 1
            dec_tokens += len(entries)
        else:
            mix_ms += ms[idx]
            mix_flops += step_flops(cfg, layers, entries, wanted)
            mix_steps += 1
            mix_tokens += sum(n for n, _ in entries)
    total_ms = start.elapsed_time(events[-1])
    stats = engine.get_stats()
    out = {
        "llama3b_continuous_tok_s": round(n_req * gen / wall, 1),
        "llama3b_device_tok_s": round(n_req * gen / (total_ms / 1e3), 1),
        "llama3b_steps": len(log),
        "llama3b_decode_steps": dec_steps,
        "llama3b_decode_ms_per_step": round(dec_ms / max(dec_steps, 1), 4),
        "llama3b_decode_batch_mean": round(dec_tokens / max(dec_steps, 1), 1),
        "llama3b_decode_hbm_frac": round(dec_bytes / max(dec_ms, 1e-9) / 1e6 / hbm_peak, 4),
        "llama3b_mixed_steps": mix_steps,
        "llama3b_mixed_tokens_per_step": round(mix_tokens / max(mix_steps, 1), 1),
        "llama3b_mixed_ms_per_step": round(mix_ms / max(mix_steps, 1), 4),
        "llama3b_mixed_tensor_frac": round(mix_flops / max(mix_ms, 1e-9) / 1e9 / tf_peak, 4),
        "llama3b_h2d_bytes_per_step": (runner.h2d_bytes - h2d0) // max(len(log), 1),
        "llama3b_preemptions": stats.preemptions,
        "llama3b_layers": layers, "llama3b_layers_of_model": LLAMA_3B["num_hidden_layers"],
    }
    runner.step = real_step
    del engine, runner, model
    torch.cuda.empty_cache()
    return out


def run_8b_long(args, hbm_peak, tf_peak):
    """Long context at the Llama 3.1 8B shape: 16,384-token prompts in portions of 2,048, then decode."""
    import torch
    from photon_infer_b200 import EngineOptions
    from photon_infer_b200.engine.loading import build_runner, random_model
    from photon_infer_b200.engine.runner import StepEntry

    batch, prompt_len, chunk, gen = args.batch_8b, 16384, 2048, 256
    cfg = dict(LLAMA_8B, num_hidden_layers=args.layers_8b or LLAMA_8B["num_hidden_layers"])
    layers = cfg["num_hidden_layers"]
    model = random_model(cfg, args.dtype, seed=8)
    options = EngineOptions(dtype=args.dtype, block_size=args.block_size,
                            max_cache_tokens=batch * (prompt_len + gen + 64), max_sequences=batch + 1,
                            max_batch_size=batch, chunk_size=chunk, max_num_batched_tokens=chunk,
                            max_model_len=prompt_len + gen + 64, use_cuda_graphs=not args.no_graphs)
    runner = build_runner(None, options, model=model)
    cache = runner.cache
    rng = torch.Generator().manual_seed(88)
    vocab = cfg["vocab_size"]

    def prefill(rid):
        ids = torch.randint(0, vocab, (prompt_len,), generator=rng).tolist()
        cache.add_request(rid)
        for lo in range(0, prompt_len, chunk):
            runner.step([StepEntry(rid, ids[lo:lo + chunk], [chunk - 1] if lo + chunk == prompt_len else [])])

    prefill("warm")                             # modules, the rotation table up to 16,384 positions
    cache.free_request("warm")
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(batch):
        prefill(("l", i))
    e1.record()
    torch.cuda.synchronize()
    pf_ms = e0.elapsed_time(e1)
    pf_flops = batch * sum(step_flops(cfg, layers, [(chunk, lo)], 1 if lo + chunk == prompt_len else 0)
                           for lo in range(0, prompt_len, chunk))
    rids = [("l", i) for i in range(batch)]
    warm = 8
    ids = [torch.randint(0, vocab, (batch,), generator=rng).tolist() for _ in range(gen)]
    greedy = ([0.0] * batch, [0.0] * batch)

    def one(k):
        return runner.step([StepEntry(r, [ids[k][i]], [0]) for i, r in enumerate(rids)], sampling=greedy).tokens
    for k in range(warm):
        one(k)
    torch.cuda.synchronize()
    kv0 = cache.cached_bytes(rids)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(warm, gen):
        one(k)
    e1.record()
    torch.cuda.synchronize()
    runner.check_device_errors()
    dec_ms = e0.elapsed_time(e1) / (gen - warm)
    kv = (kv0 + cache.cached_bytes(rids)) // 2
    step_bytes = model.step_weight_bytes() + kv
    out = {
        "llama8b_prefill_tok_s": round(batch * prompt_len / (pf_ms / 1e3), 1),
        "llama8b_prefill_ms_per_portion": round(pf_ms / (batch * prompt_len // chunk), 3),
        "llama8b_prefill_tensor_frac": round(pf_flops / (pf_ms / 1e3) / (tf_peak * 1e12), 4),
        "llama8b_decode_tok_s": round(batch / (dec_ms / 1e3), 1),
        "llama8b_decode_ms_per_step": round(dec_ms, 4),
        "llama8b_decode_hbm_frac": round(step_bytes / (dec_ms / 1e3) / 1e9 / hbm_peak, 4),
        "llama8b_batch": batch, "llama8b_context": prompt_len,
        "llama8b_layers": layers, "llama8b_layers_of_model": LLAMA_8B["num_hidden_layers"],
    }
    for r in rids:
        cache.free_request(r)
    del runner, model
    torch.cuda.empty_cache()
    return out


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
    ap.add_argument("--shape", default="1b", choices=["1b", "3b", "8b"],
                    help="layer sizes of the single steps that --only decode / --only prefill time (for profiles)")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "3b", "8b"],
                    help="run one phase or workload only (for profiling); the JSON line then lacks the other figures")
    ap.add_argument("--workloads", default="all", choices=["all", "headline"],
                    help="headline: leave the 3B and 8B workloads out of points")
    ap.add_argument("--layers-3b", type=int, default=0, help="fewer layers for the 3B workload (0: all 28)")
    ap.add_argument("--layers-8b", type=int, default=0, help="fewer layers for the 8B workload (0: all 32)")
    ap.add_argument("--batch-8b", type=int, default=8)
    args = ap.parse_args()

    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    args.steps = max(1, min(args.steps, GEN_LEN - args.warmup - 1))

    import torch

    hbm_peak, tf_peak, peak_src = peaks()
    if args.only in ("3b", "8b"):
        fn = run_3b_continuous if args.only == "3b" else run_8b_long
        print(json.dumps({"only": args.only, "points": fn(args, hbm_peak, tf_peak)}))
        return 0
    line = run_headline(args, hbm_peak, tf_peak, peak_src)
    if line is None:
        return 0
    if args.workloads == "all":
        torch.cuda.empty_cache()
        line["points"].update(run_3b_continuous(args, hbm_peak, tf_peak))
        line["points"].update(run_8b_long(args, hbm_peak, tf_peak))
    print(json.dumps(line))
    return 0


def run_headline(args, hbm_peak, tf_peak, peak_src):
    """The headline: decode at ``--batch`` and the 2,048-token prefill at the Llama 3.2 1B shape, the same
    through the entry point, batch 1 and 64.  Returns the JSON line as a dict (None: a partial line was printed)."""
    import torch
    from photon_infer_b200 import EngineOptions
    from photon_infer_b200.engine.engine import ContinuousBatchEngine
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    from photon_infer_b200.kernels import ops
    from photon_infer_b200.weights import write_random_model

    shapes = {"1b": LLAMA_1B, "3b": LLAMA_3B, "8b": LLAMA_8B}
    if args.shape != "1b" and args.only not in ("decode", "prefill"):
        raise SystemExit("--shape 3b/8b goes with --only decode or --only prefill (a profile of single steps)")
    cfg = dict(shapes[args.shape], num_hidden_layers=min(args.layers, shapes[args.shape]["num_hidden_layers"]))
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
    cut_error = None
    if pf_ms:
        # the same 2,048 tokens as one portion and as two of 1,024: the last row's logits must agree
        # within a rounding of the activations (the kernels differ with the number of rows)
        cache.add_request("p")
        whole = runner.step([StepEntry("p", prompt, [PREFILL_TOKENS - 1])]).logits.float().clone()
        cache.free_request("p")
        cache.add_request("p")
        runner.step([StepEntry("p", prompt[:PREFILL_TOKENS // 2], [])])
        halves = runner.step([StepEntry("p", prompt[PREFILL_TOKENS // 2:], [PREFILL_TOKENS // 2 - 1])]).logits.float()
        cache.free_request("p")
        cut_error = float((whole - halves).abs().max() / whole.abs().max())
    prefill_ms = min(pf_ms[1:]) if pf_ms else float("nan")
    H, I, L, d = cfg["hidden_size"], cfg["intermediate_size"], args.layers, cfg["head_dim"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    per_token = 2 * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    attn = 4 * nq * d * (PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2)          # QK^T and PV over the causal half
    prefill_flops = L * (PREFILL_TOKENS * per_token + attn) + 2 * H * vocab
    prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3), "frac": round(prefill_flops / (prefill_ms / 1e3) / (tf_peak * 1e12), 4),
               "cut_check": None if cut_error is None else round(cut_error, 5)}

    if args.only == "prefill":
        clocks.stop()
        print(json.dumps({"only": "prefill", "prefill": prefill}))
        return None
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
        return None
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
    return line


if __name__ == "__main__":
    sys.exit(main())
