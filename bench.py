#!/usr/bin/env python3
"""Benchmark: decode tokens per second of the engine at Qwen3-8B sizes with random weights.

    python bench.py --gpus 1 --steps K --warmup W

A "step" is one decode step of a batch of 8 requests, each with a 2,048-token context
(16-token pages). ``value`` is device-timed (CUDA events around exactly K steps of the
engine's step function plus on-device argmax); ``e2e`` is the same through the Python
entry point ``LLM.step()`` with host token ids in and out every step. The line also
reports a 2,048-token prefill, the decode step's fraction of the HBM roofline, and decode
at batch 1 and 64. Prints ONE JSON line. The engine runs on one GPU: for --gpus > 1 it
says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# the headline configuration: Qwen3-8B sizes
QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
    max_position_embeddings=4096)
# the other two Qwen3 sizes of the reference's benchmarks (selected with --model)
QWEN3_06B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                 intermediate_size=25600)
MODELS = {"8b": ("Qwen3-8B sizes", QWEN3_8B), "0.6b": ("Qwen3-0.6B sizes", QWEN3_06B), "32b": ("Qwen3-32B sizes", QWEN3_32B)}
CONTEXT = 2048
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as fh:
                raw = json.load(fh)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            return out, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for name, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz)}


def sampler_mode(args, torch, ops, vocab: int) -> int:
    """The sampling kernels alone on rows whose few dozen largest logits stand out, as a trained model's do."""
    dev = torch.device("cuda:0")
    rows = args.batch
    torch.manual_seed(0)
    logits = torch.randn(rows, vocab, device=dev) * 3
    logits[:, :40] += torch.linspace(16, 6, 40, device=dev)
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    scratch = torch.empty(rows * vocab, device=dev)
    settings = {"temperature": (0.8, 0, 1.0, 0.0), "top_k": (0.8, 20, 1.0, 0.0), "top_p": (0.8, 0, 0.9, 0.0),
                "top_k_top_p": (0.6, 20, 0.95, 0.0), "top_k_top_p_min_p": (0.8, 50, 0.9, 0.05)}

    def tensors(t, k, p, mp):
        return (torch.full((rows,), t, device=dev), torch.full((rows,), k, dtype=torch.int32, device=dev),
                torch.full((rows,), p, device=dev), torch.full((rows,), mp, device=dev), torch.full((rows,), 0.37, device=dev))

    if args.profile == "sampler":
        T, K, P, MP, U = tensors(*settings["top_k_top_p"])
        for i in range(args.warmup + 1):
            if i == args.warmup:
                torch.cuda.synchronize()
                torch.cuda.profiler.start()
            ops.sample(out, logits, scratch, T, K, P, MP, U)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled": "sampler", "rows": rows, "vocab": vocab}))
        return 0
    result = {}
    for clusters in (True, False):
        ops.sample_use_clusters(clusters)
        for name, setting in settings.items():
            T, K, P, MP, U = tensors(*setting)
            for _ in range(3):
                ops.sample(out, logits, scratch, T, K, P, MP, U)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(10):
                    ops.sample(out, logits, scratch, T, K, P, MP, U)
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            result[("clusters/" if clusters else "one_block/") + name] = round(e0.elapsed_time(e1) / 50 * 1000, 1)
    ops.sample_use_clusters(True)
    print(json.dumps({"sampler_us_per_call": result, "rows": rows, "vocab": vocab,
                      "note": "temperature, top_k, top_p, min_p per setting: " + json.dumps(settings)}))
    return 0


def main() -> int:
    global CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT, help="tokens each request holds when decoding starts")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--model", default="8b", choices=sorted(MODELS), help="layer sizes (default: the headline 8B)")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch-1/64 points and the prefill")
    ap.add_argument("--batch-invariant", action="store_true",
                    help="measure under the batch-invariant numeric policy (one product kernel, fixed key slices)")
    ap.add_argument("--timeline", default=None, metavar="FILE",
                    help="write the start and end of every kernel of one decode step (CUPTI through torch.profiler: kernels "
                         "overlap under programmatic dependent launch, which a serialising profiler cannot show) and exit")
    ap.add_argument("--sampler", action="store_true",
                    help="time the sampling kernels alone (vocabulary of the model, --batch rows, recorded into a CUDA "
                         "graph): one JSON line of microseconds per call and setting, then exit")
    ap.add_argument("--profile", choices=["decode", "prefill", "sampler"], default=None,
                    help="run warm-up, then ONE step between cudaProfilerStart/Stop and exit "
                         "(for `ncu --profile-from-start off`); prints no benchmark line")
    args = ap.parse_args()
    CONTEXT = args.context

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust + CUDA workspace (no setup.py/pyproject.toml: pip reports "
                          "'not installable'); no Rust toolchain in this image"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on ONE GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from openinfer_b200.config.base import resolve_architecture
    from openinfer_b200.engine.engine import LLM
    from openinfer_b200.engine.runner import ModelRunner, StepEntry
    from openinfer_b200.kernels import lib as klib
    from openinfer_b200.kernels import ops
    from openinfer_b200.sampling.params import SamplingParams

    if args.batch_invariant:
        from openinfer_b200.kernels import policy
        policy.set_batch_invariant(True)
    if args.sampler or args.profile == "sampler":
        return sampler_mode(args, torch, ops, MODELS[args.model][1]["vocab_size"])
    peaks, peaks_src = read_peaks()
    model_name, model_cfg = MODELS[args.model]
    cfg_dict = dict(model_cfg)
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    cfg_dict["max_position_embeddings"] = max(cfg_dict["max_position_embeddings"],
                                              CONTEXT + args.steps + args.warmup + max(args.batch, 8) * -(-CONTEXT // PREFILL_TOKENS) + 128)
    config = resolve_architecture(cfg_dict).config_cls.from_dict(cfg_dict)
    K, W, B = args.steps, args.warmup, args.batch
    max_batch = B if args.skip_points else max(B, 64)
    # Through the entry point the requests' prompts are computed one portion a step, and a request that has its
    # prompt decodes while the others' are still computed: it must not finish before all of them decode.
    e2e_prompt_steps = max(B, 8) * -(-CONTEXT // PREFILL_TOKENS)
    e2e_new_tokens = W + K + e2e_prompt_steps + 8
    per_req = CONTEXT + e2e_new_tokens + 16 + 2 * PAGE
    pool_tokens = max_batch * per_req + PREFILL_TOKENS + 64
    dev = torch.device("cuda:0")
    runner = ModelRunner.build(config, 0, dtype=args.dtype, device=dev, page_size=PAGE,
                               max_tokens=pool_tokens, max_requests=max_batch + 8)
    runner.cuda_graph = True
    cache = runner.cache
    esize = 2 if args.dtype == "bfloat16" else 4
    for g in cache.groups:  # contexts are not computed but filled: decode reads the same bytes
        g.tensor.normal_(0.0, 0.5)
    rng = random.Random(0)
    vocab = config.vocab_size

    def fake_context(rid, n):
        cache.open(rid)
        cache.reserve(rid, n)
        cache.commit(rid)

    def decode_run(batch, steps, warmup):
        """Device-timed decode: `steps` steps of `batch` requests at context CONTEXT."""
        ids = [f"b{batch}_{i}" for i in range(batch)]
        for rid in ids:
            fake_context(rid, CONTEXT)
        toks = [[rng.randrange(vocab)] for _ in ids]
        out = torch.empty(batch, dtype=torch.int32, device=dev)

        def one():
            logits = runner.step([StepEntry(rid, t, [0]) for rid, t in zip(ids, toks)])
            ops.argmax(out, logits)

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        l0 = klib.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = klib.launches - l0
        for rid in ids:
            runner.end(rid)
        return ms, launches

    if args.timeline:
        from torch.profiler import ProfilerActivity, profile
        ids = [f"p{i}" for i in range(B)]
        for rid in ids:
            fake_context(rid, CONTEXT)
        out_ids = torch.empty(B, dtype=torch.int32, device=dev)

        def one():
            logits = runner.step([StepEntry(rid, [1], [0]) for rid in ids])
            ops.argmax(out_ids, logits)

        for _ in range(W):
            one()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                one()
            torch.cuda.synchronize()
        evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                     key=lambda e: e.time_range.start)
        first = [i for i, e in enumerate(evs) if "embedding" in e.name][-1]   # the last of the three steps
        evs = evs[first:]
        t0 = evs[0].time_range.start
        with open(args.timeline, "w") as f:
            f.write("start_us end_us us_after_the_end_of_everything_before kernel\n")
            done = 0.0
            for e in evs:
                a, b = e.time_range.start - t0, e.time_range.end - t0
                f.write(f"{a:9.1f} {b:9.1f} {b - max(done, a) if b > done else 0.0:7.1f}  {e.name[:60]}\n")
                done = max(done, b)
        print(json.dumps({"timeline": args.timeline, "batch": B, "layers": config.num_hidden_layers,
                          "kernels": len(evs), "step_us": round(done, 1)}))
        return 0

    if args.profile:
        if args.profile == "decode":
            ids = [f"p{i}" for i in range(B)]
            for rid in ids:
                fake_context(rid, CONTEXT)
            out_ids = torch.empty(B, dtype=torch.int32, device=dev)
            for i in range(W + 1):
                if i == W:
                    torch.cuda.synchronize()
                    torch.cuda.profiler.start()
                logits = runner.step([StepEntry(rid, [1], [0]) for rid in ids])
                ops.argmax(out_ids, logits)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        else:
            toks = [rng.randrange(vocab) for _ in range(PREFILL_TOKENS)]
            for i in range(W + 1):
                if i == W:
                    torch.cuda.synchronize()
                    torch.cuda.profiler.start()
                runner.step([StepEntry(f"pf{i}", toks, [PREFILL_TOKENS - 1])])
                torch.cuda.synchronize()
                runner.end(f"pf{i}")
            torch.cuda.profiler.stop()
        print(json.dumps({"profiled": args.profile, "batch": B, "layers": config.num_hidden_layers}))
        return 0

    sampler = ClockSampler(0)
    sampler.start()
    ms_step, launches = decode_run(B, K, W)
    clocks = sampler.stop()
    value = B * 1000.0 / ms_step

    # roofline of the decode step: every weight once + the cache of the live requests
    kv_tokens = B * (CONTEXT + W + K // 2)
    step_bytes = runner.model.weight_bytes() + kv_tokens * cache.bytes_per_token(esize)
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peaks_src}

    # end to end through the Python entry point: host token ids in and out every step
    llm = LLM(config=config, runner=runner, max_prefill_tokens=PREFILL_TOKENS, max_decode_batch=max_batch)
    for i in range(B):
        llm.submit([rng.randrange(vocab) for _ in range(CONTEXT)], SamplingParams(ignore_eos=True), e2e_new_tokens)
    for _ in range(e2e_prompt_steps + 8):
        if len(llm.scheduler.active) == B:
            break
        for ev in llm.step():
            if ev.kind in ("error", "rejected"):
                raise RuntimeError(f"bench: request {ev.request_id} {ev.kind}: {ev.reason}")
    if len(llm.scheduler.active) != B:
        raise RuntimeError(f"bench: only {len(llm.scheduler.active)} of {B} requests decode after their prompts")
    for _ in range(W):
        llm.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_tok = 0
    for _ in range(K - 1):  # the prompt's last step produced the first token; K - 1 more decode steps are left
        n_tok += sum(1 for ev in llm.step() if ev.kind == "token")
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    while llm.has_work():
        llm.step()
    e2e = {"value": round(n_tok / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": B * 4,
           "ms_per_step": round(e2e_s * 1000 / max(K - 1, 1), 4)}
    # bytes of step metadata copied host->device each step (token ids, positions, block tables, ...)
    e2e["h2d_bytes_per_step"] = int(runner._staging_last_bytes) if hasattr(runner, "_staging_last_bytes") else None

    out = {
        "metric": f"decode tokens/s ({model_name}, random weights, batch {B}, context {CONTEXT})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "ours",
        "config": {
            "model": model_name, "layers": config.num_hidden_layers, "layers_full": full_layers,
            "hidden": config.hidden_size, "q_heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
            "intermediate": config.intermediate_size, "vocab": config.vocab_size,
            "rope_theta": config.rope_theta, "rms_norm_eps": config.rms_norm_eps, "tied": config.tie_word_embeddings,
            "global_batch": B, "seq_len": CONTEXT, "kv_page": PAGE, "new_tokens": K,
            "parallelism": "single GPU", "l2": "weights (>15 GB) exceed L2; no flush needed",
        },
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
    }
    if args.batch_invariant:
        out["config"]["batch_invariant"] = True

    if not args.skip_points:
        points = {}
        for b in (1, 64):
            steps = max(16, K // 2)
            ms_b, _ = decode_run(b, steps, max(3, W // 2))
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
        out["points"] = points

        # prefill of one 2,048-token prompt in one step
        toks = [rng.randrange(vocab) for _ in range(PREFILL_TOKENS)]
        times = []
        for i in range(3 + 3):
            rid = f"pf{i}"
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step([StepEntry(rid, toks, [PREFILL_TOKENS - 1])])
            e1.record()
            torch.cuda.synchronize()
            runner.end(rid)
            if i >= 3:
                times.append(e0.elapsed_time(e1))
        pf_ms = statistics.median(times)
        L, H, I = config.num_hidden_layers, config.hidden_size, config.intermediate_size
        dq, dkv = config.q_dim, config.kv_dim
        T = PREFILL_TOKENS
        flops = L * (2 * T * H * (dq + 2 * dkv) + 2 * T * dq * H + 2 * T * H * 2 * I + 2 * T * I * H
                     + 4 * config.num_attention_heads * config.head_dim * T * T / 2) + 2 * vocab * H
        peak_tf = peaks["bf16_tflops"] if args.dtype == "bfloat16" else 75.0
        out["prefill"] = {"value": round(T * 1000.0 / pf_ms, 1), "tokens": T, "ms": round(pf_ms, 3),
                          "frac": round(flops / (pf_ms * 1e-3) / (peak_tf * 1e12), 4), "peaks": peaks_src}
        if args.dtype == "bfloat16":
            # the step is timed back to back after the decode runs, i.e. under the power cap: also against the
            # library product's SUSTAINED rate (a burst after idle runs this step in 23.6 ms instead of 26.5)
            out["prefill"]["frac_of_sustained"] = round(flops / (pf_ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
