"""Command line in the manner of the reference's ``llama_infer``
(demo/llama_infer.cpp:127-275): ``llama_infer <checkpoint_path> [device] [options]``,
prompts in, generated tokens and tokens per second out, temperature 0.8 by default
(demo/llama_infer.cpp:62).  The checkpoint is a model folder (``config.json``,
``model.safetensors``); there is no tokenizer argument because prompts are token ids.
``--quantize`` / ``--no-quantize`` are accepted for compatibility: INT8 weights are
not part of this engine, so ``--quantize`` is refused.
"""
from __future__ import annotations

import argparse
import sys
import time
from typing import List

from ..config.engine_options import EngineOptions, normalize_dtype
from ..errors import PhotonError


def _ids(text: str) -> List[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llama_infer", description="Generate token ids with a Llama model folder on one GPU.")
    ap.add_argument("checkpoint_path", nargs="?", help="model folder (config.json + model.safetensors)")
    ap.add_argument("device", nargs="?", default="cuda", help="cuda or cuda:N (there is no cpu path)")
    ap.add_argument("--quantize", action="store_true", help="refused: INT8 weights are not part of this engine")
    ap.add_argument("--no-quantize", action="store_true", help="accepted, no effect")
    ap.add_argument("--prompt-ids", action="append", default=[], help="one request: token ids separated by commas or spaces")
    ap.add_argument("--prompt-ids-file", help="file with one request per line")
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", help="bfloat16 (bf16) or float32 (fp32)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--num-blocks", type=int, default=None, help="cache pages (default: from free memory)")
    ap.add_argument("--max-batch-size", type=int, default=32)
    ap.add_argument("--max-sequences", type=int, default=32)
    ap.add_argument("--chunk-size", type=int, default=256, help="longest prompt portion of a request in one step")
    ap.add_argument("--max-batched-tokens", type=int, default=2048, help="token budget of one step")
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--random-weights", metavar="CONFIG_JSON",
                    help="write a model folder with random weights from this config.json into checkpoint_path first")
    ap.add_argument("--init-std", type=float, default=0.02)
    ap.add_argument("--norm-std", type=float, default=0.0)
    ap.add_argument("--print-stats", action="store_true")
    args = ap.parse_args(argv)
    if args.checkpoint_path is None:
        ap.print_usage(sys.stderr)
        return 1
    if args.quantize:
        print("llama_infer: --quantize is refused: INT8 weights are not part of this engine", file=sys.stderr)
        return 1
    device = "cuda:0" if args.device.lower() == "cuda" else args.device.lower()
    if not device.startswith("cuda"):
        print(f"llama_infer: device {args.device!r}: this engine runs on CUDA only", file=sys.stderr)
        return 1
    try:
        if args.random_weights:
            from ..config.model_config import read_config_json
            from ..weights.random_init import write_random_model
            write_random_model(args.checkpoint_path, read_config_json(args.random_weights), seed=args.seed,
                               init_std=args.init_std, norm_std=args.norm_std)
        prompts = [_ids(p) for p in args.prompt_ids]
        if args.prompt_ids_file:
            with open(args.prompt_ids_file) as f:
                prompts += [_ids(line) for line in f if line.strip()]
        if not prompts:
            print("llama_infer: no prompt (use --prompt-ids or --prompt-ids-file)", file=sys.stderr)
            return 1
        from .engine import ContinuousBatchEngine
        options = EngineOptions(dtype=normalize_dtype(args.dtype), block_size=args.block_size, num_blocks=args.num_blocks,
                                max_sequences=args.max_sequences, max_batch_size=args.max_batch_size,
                                chunk_size=args.chunk_size, max_num_batched_tokens=args.max_batched_tokens,
                                max_model_len=args.max_model_len, seed=args.seed, device=device)
        print("PhotonInfer B200 - LLaMA Inference", file=sys.stderr)
        engine = ContinuousBatchEngine(args.checkpoint_path, options)
        ids = [engine.add_request(p, args.max_new_tokens, args.temperature, args.seed, args.ignore_eos) for p in prompts]
        t0 = time.perf_counter()
        out = engine.run_until_complete(print_progress=args.print_stats)
        dt = time.perf_counter() - t0
        total = 0
        for rid in ids:
            req = engine.result(rid)
            total += len(out[rid])
            print(f"request {rid} ({req.finish_reason}): " + " ".join(str(t) for t in out[rid]))
        print(f"Generated {total} tokens in {dt:.3f} s ({total / dt:.1f} tokens/s)", file=sys.stderr)
        if args.print_stats:
            print(engine.get_stats(), file=sys.stderr)
        return 0
    except PhotonError as e:
        print(f"llama_infer: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
