"""Command line: ``python -m openinfer_b200 --model-path DIR --prompt-ids 1,2,3 --max-tokens 16``.

The reference's binary serves HTTP; this one generates for prompts given as token ids and
prints one JSON line per prompt. Options the reference has keep its names, meanings and
defaults: --model-path, --cuda-graph, --device-ordinal, --max-prefill-tokens
(pegainfer-frontend/src/model_line.rs:85-187), --gpu-memory-utilization,
--kv-cache-memory-margin-mib, --kv-page-size (pegainfer-qwen3/src/model_line.rs:32-118),
and the sampling parameters temperature / top-k / top-p / min-p / seed / ignore-eos
(pegainfer-frontend/src/sampler.rs:2-38). Serving-only options (--port, --served-model-name,
--tp-size, offload, LoRA, speculative decoding) do not exist here.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional


def _bool(v: str) -> bool:
    if v.lower() in ("true", "1", "yes"):
        return True
    if v.lower() in ("false", "0", "no"):
        return False
    raise argparse.ArgumentTypeError(f"expected true or false, got {v!r}")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="openinfer_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    src = ap.add_argument_group("model")
    src.add_argument("--model-path", help="model directory containing config.json and safetensors")
    src.add_argument("--random-config", help="a config.json to build a random-weights model from (with --seed)")
    src.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    src.add_argument("--write-random-model", metavar="DIR",
                     help="write config.json + model.safetensors with random weights to DIR and exit")
    src.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    eng = ap.add_argument_group("engine")
    eng.add_argument("--device-ordinal", type=int, default=0, help="CUDA device ordinal")
    eng.add_argument("--cuda-graph", type=_bool, default=True, metavar="BOOL",
                     help="capture/replay CUDA graphs on the decode path (--cuda-graph=false to disable)")
    eng.add_argument("--max-prefill-tokens", type=int, default=1024,
                     help="cap on total prompt tokens forwarded in one scheduler step")
    eng.add_argument("--gpu-memory-utilization", type=float, default=0.90,
                     help="fraction of device memory the engine may use (weights + cache)")
    eng.add_argument("--kv-cache-memory-margin-mib", type=int, default=150,
                     help="memory left free beside the cache pool")
    eng.add_argument("--kv-page-size", type=int, default=16, help="tokens per cache page")
    eng.add_argument("--num-pages", type=int, default=None, help="size the cache pool explicitly (pages)")
    eng.add_argument("--batch-invariant", action="store_true",
                     help="a request's results do not depend, bit for bit, on what it is batched with (slower)")
    eng.add_argument("--no-prefix-cache", action="store_true",
                     help="do not share registered prompt pages between requests")
    gen = ap.add_argument_group("generation")
    gen.add_argument("--prompt-ids", action="append", default=[],
                     help="comma-separated token ids of one prompt (repeatable)")
    gen.add_argument("--prompt-file", help="JSON file: a list of token-id lists")
    gen.add_argument("--max-tokens", type=int, default=16)
    gen.add_argument("--temperature", type=float, default=0.0)
    gen.add_argument("--top-k", type=int, default=-1)
    gen.add_argument("--top-p", type=float, default=1.0)
    gen.add_argument("--min-p", type=float, default=0.0)
    gen.add_argument("--sampling-seed", type=int, default=None, help="per-request sampling seed")
    gen.add_argument("--ignore-eos", action="store_true")
    gen.add_argument("--logprobs", type=int, default=0, help="report each token's log-probability and this many top ones")
    gen.add_argument("--echo", action="store_true", help="with --logprobs: also the prompt tokens' log-probabilities")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    from .config.base import read_config_json, resolve_architecture

    config = None
    if args.random_config:
        import os

        folder = os.path.dirname(os.path.abspath(args.random_config))
        with open(args.random_config) as fh:
            raw = json.load(fh)
        config = resolve_architecture(raw).config_cls.from_dict(raw)
    if args.write_random_model:
        if config is None:
            print("--write-random-model needs --random-config", file=sys.stderr)
            return 2
        from .weights import write_random_model

        write_random_model(config, args.write_random_model, args.seed)
        print(json.dumps({"written": args.write_random_model, "seed": args.seed}))
        return 0
    if not args.model_path and config is None:
        print("give --model-path DIR or --random-config CONFIG.json", file=sys.stderr)
        return 2
    prompts: List[List[int]] = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as fh:
            prompts += [list(map(int, p)) for p in json.load(fh)]
    if not prompts:
        print("no prompts: give --prompt-ids or --prompt-file", file=sys.stderr)
        return 2

    if args.batch_invariant and not args.no_prefix_cache:
        print("--batch-invariant requires --no-prefix-cache: prefix-cache hits move a prompt's portions off the "
              "request's own grid, so bit-identical results cannot be promised", file=sys.stderr)
        return 2

    from .engine.engine import LLM
    from .sampling.params import SamplingParams

    llm = LLM(args.model_path, config=config, seed=args.seed if config is not None else None, dtype=args.dtype,
              device_ordinal=args.device_ordinal, kv_page_size=args.kv_page_size, num_pages=args.num_pages,
              gpu_memory_utilization=args.gpu_memory_utilization,
              kv_cache_memory_margin_mib=args.kv_cache_memory_margin_mib,
              max_prefill_tokens=args.max_prefill_tokens, cuda_graph=args.cuda_graph,
              prefix_cache=not args.no_prefix_cache, batch_invariant=True if args.batch_invariant else None)
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                        seed=args.sampling_seed, ignore_eos=args.ignore_eos)
    def lp(entry):
        return None if entry is None else {"logprob": entry.logprob, "top_logprobs": entry.top_logprobs}

    for i, r in enumerate(llm.generate_detailed(prompts, sp, args.max_tokens, logprobs=args.logprobs, echo=args.echo)):
        line = {"prompt": i, "token_ids": r.token_ids, "finish_reason": r.finish_reason}
        if r.logprobs is not None:
            line["logprobs"] = [lp(e) for e in r.logprobs]
        if r.prompt_logprobs is not None:
            line["prompt_logprobs"] = [lp(e) for e in r.prompt_logprobs]
        print(json.dumps(line), flush=True)
    return 0
