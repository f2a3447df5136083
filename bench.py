#!/usr/bin/env python3
"""Benchmark: decode tokens per second of the engine at Qwen3-8B sizes with random weights.

    python bench.py --gpus 1 --steps K --warmup W

A "step" is one decode step of a batch of 8 requests, each with a 2,048-token context
(16-token pages). ``value`` is device-timed (CUDA events around exactly K steps of the
engine's step function plus on-device argmax); ``e2e`` is the same through the Python
entry point ``LLM.step()`` with host token ids in and out every step. The line also
reports a 2,048-token prefill, the decode step's fraction of the HBM roofline, and decode
at batch 1 and 64; then, as flat entries of ``points`` (and once more, grouped, under
``sizes``), prefills of 8,192 and 32,768 tokens and decoding at longer contexts (batch 8 at
16,384 tokens, batch 1 at 32,768) at the headline sizes, and the other two
sizes of the reference's benchmarks, each built, measured and freed in turn: Qwen3-0.6B
sizes (decode at batch 1/8/64, prefill, and the mixed step of 8 prompt portions of 512
tokens beside 56 decoding requests, device-timed and through ``LLM.step()``) and Qwen3-32B
sizes (decode at batch 1/8/64, prefill), each with its own roofline fractions and clock
sample. Prints ONE JSON line. The engine runs on one GPU: for --gpus > 1 it says so and
exits with 2.
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


class Bench:
    """One model size on the GPU: the runner, its pool, and the measurements taken on it."""

    def __init__(self, torch, mods, cfg_dict, dtype, max_batch, steps_room, context, prefill_room=PREFILL_TOKENS,
                 layers=None, page=PAGE):
        self.torch, self.mods = torch, mods
        cfg_dict = dict(cfg_dict)
        self.full_layers = cfg_dict["num_hidden_layers"]
        if layers:
            cfg_dict["num_hidden_layers"] = layers
        self.context = context
        per_req = context + steps_room + 16 + 2 * page
        cfg_dict["max_position_embeddings"] = max(cfg_dict["max_position_embeddings"], per_req + 128, prefill_room + 128)
        self.config = mods["resolve_architecture"](cfg_dict).config_cls.from_dict(cfg_dict)
        self.dtype = dtype
        self.esize = 2 if dtype == "bfloat16" else 4
        self.dev = torch.device("cuda:0")
        pool_tokens = max_batch * per_req + max(prefill_room, 8 * 512) + 64
        self.runner = mods["ModelRunner"].build(self.config, 0, dtype=dtype, device=self.dev, page_size=page,
                                                max_tokens=pool_tokens, max_requests=max_batch + 16)
        self.runner.cuda_graph = True
        self.cache = self.runner.cache
        for g in self.cache.groups:  # contexts are not computed but filled: decode reads the same bytes
            g.tensor.normal_(0.0, 0.5)
        self.rng = random.Random(0)
        self.vocab = self.config.vocab_size

    def close(self):
        import gc
        self.runner = self.cache = None
        gc.collect()
        self.torch.cuda.synchronize()
        self.torch.cuda.empty_cache()

    def fake_context(self, rid, n):
        self.cache.open(rid)
        self.cache.reserve(rid, n)
        self.cache.commit(rid)

    def decode_run(self, batch, steps, warmup):
        """Device-timed decode: `steps` steps of `batch` requests at the context length. Returns (ms, launches)."""
        torch, runner, ops, klib, StepEntry = self.torch, self.runner, self.mods["ops"], self.mods["klib"], self.mods["StepEntry"]
        ids = [f"b{batch}_{i}" for i in range(batch)]
        for rid in ids:
            self.fake_context(rid, self.context)
        toks = [[self.rng.randrange(self.vocab)] for _ in ids]
        out = torch.empty(batch, dtype=torch.int32, device=self.dev)

        def one():
            logits = runner.step([StepEntry(rid, t, [0]) for rid, t in zip(ids, toks)])
            ops.argmax(out, logits)

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        l0 = klib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = klib.launch_count() - l0
        for rid in ids:
            runner.end(rid)
        return ms, launches

    def decode_bytes(self, batch, steps, warmup):
        """What a decode step has to read: every weight it uses once, and the cache of the live requests."""
        kv_tokens = batch * (self.context + warmup + steps // 2)
        return self.runner.model.weight_bytes() + kv_tokens * self.cache.bytes_per_token(self.esize)

    def linear_flops_per_token(self):
        c = self.config
        return c.num_hidden_layers * 2 * (c.hidden_size * (c.q_dim + 2 * c.kv_dim) + c.q_dim * c.hidden_size
                                          + 3 * c.hidden_size * c.intermediate_size)

    def prefill_flops(self, T):
        c = self.config
        return (T * self.linear_flops_per_token() + c.num_hidden_layers * 4 * c.num_attention_heads * c.head_dim * T * T / 2
                + 2 * self.vocab * c.hidden_size)

    def prefill_run(self, T, reps=3, warm=3):
        """One prompt of T tokens in one step, back to back; the median of `reps` after `warm`."""
        torch, runner, StepEntry = self.torch, self.runner, self.mods["StepEntry"]
        toks = [self.rng.randrange(self.vocab) for _ in range(T)]
        times = []
        for i in range(warm + reps):
            rid = f"pf{T}_{i}"
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step([StepEntry(rid, toks, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            runner.end(rid)
            if i >= warm:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times)

    def mixed_flops(self, n_decode, n_portions, portion):
        c = self.config
        rows = n_decode + n_portions * portion
        att = 4 * c.num_attention_heads * c.head_dim * (n_decode * self.context + n_portions * portion * portion / 2)
        return rows * self.linear_flops_per_token() + c.num_hidden_layers * att + 2 * (n_decode + n_portions) * self.vocab * c.hidden_size

    def mixed_run(self, n_decode, n_portions, portion, steps, warmup):
        """The general step: `n_portions` prompt portions of `portion` tokens (each the start of a new prompt)
        beside `n_decode` requests decoding at the context length, one logits row each. Device-timed."""
        torch, runner, ops, StepEntry = self.torch, self.runner, self.mods["ops"], self.mods["StepEntry"]
        ids = [f"mx{i}" for i in range(n_decode)]
        for rid in ids:
            self.fake_context(rid, self.context)
        tok = [[self.rng.randrange(self.vocab)] for _ in ids]
        parts = [[self.rng.randrange(self.vocab) for _ in range(portion)] for _ in range(n_portions)]
        out = torch.empty(n_decode + n_portions, dtype=torch.int32, device=self.dev)

        def one(i):
            entries = [StepEntry(rid, t, [0]) for rid, t in zip(ids, tok)]
            entries += [StepEntry(f"mxp{i}_{j}", p, [portion - 1]) for j, p in enumerate(parts)]
            ops.argmax(out, runner.step(entries))
            for j in range(n_portions):
                runner.end(f"mxp{i}_{j}")

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            one(warmup + i)
        e1.record()
        torch.cuda.synchronize()
        for rid in ids:
            runner.end(rid)
        return e0.elapsed_time(e1) / steps

    def mixed_e2e(self, n_decode, n_portions, portion, steps, warmup):
        """The same step through LLM.step(): every call the host submits `n_portions` new prompts of `portion`
        token ids (one token each to generate) and reads the step's sampled ids. Returns seconds per step."""
        torch, LLM, SamplingParams = self.torch, self.mods["LLM"], self.mods["SamplingParams"]
        llm = LLM(config=self.config, runner=self.runner, max_prefill_tokens=max(PREFILL_TOKENS, n_portions * portion),
                  max_decode_batch=n_decode + 2 * n_portions)
        long = warmup + steps + 16 + n_decode * -(-self.context // PREFILL_TOKENS)
        for _ in range(n_decode):
            llm.submit([self.rng.randrange(self.vocab) for _ in range(self.context)], SamplingParams(ignore_eos=True), long)
        for _ in range(n_decode * -(-self.context // PREFILL_TOKENS) + 8):
            if len(llm.scheduler.active) == n_decode and not llm.scheduler.prefilling:
                break
            for ev in llm.step():
                if ev.kind in ("error", "rejected"):
                    raise RuntimeError(f"bench: request {ev.request_id} {ev.kind}: {ev.reason}")
        if len(llm.scheduler.active) != n_decode:
            raise RuntimeError(f"bench: only {len(llm.scheduler.active)} of {n_decode} requests decode after their prompts")

        def one():
            for _ in range(n_portions):
                llm.submit([self.rng.randrange(self.vocab) for _ in range(portion)], SamplingParams(ignore_eos=True), 1)
            return sum(1 for ev in llm.step() if ev.kind == "token")

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n_tok = 0
        for _ in range(steps):
            n_tok += one()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        for a in list(llm.scheduler.active) + [p for p in llm.scheduler.prefilling]:
            llm.cancel(a.req.request_id)
        while llm.has_work():
            llm.step()
        return dt / steps, n_tok / steps


def measure_size(torch, mods, key, args, peaks, mixed: bool):
    """Decode at batch 1/8/64, a 2,048-token prefill and (0.6B) the mixed step at one of the other sizes, with its
    own clock sample. Returns (flat points, grouped record)."""
    name, cfg = MODELS[key]
    steps, warm = max(16, args.steps // 4), max(3, args.warmup // 2)
    room = 2 * (steps + warm) + 64 * -(-CONTEXT // PREFILL_TOKENS) + 64
    b = Bench(torch, mods, cfg, args.dtype, 64, room, CONTEXT)
    sampler = ClockSampler(0)
    sampler.start()
    flat, rec = {}, {"model": name, "layers": b.config.num_hidden_layers}
    try:
        for batch in (1, 8, 64):
            ms, _ = b.decode_run(batch, steps, warm)
            gbs = b.decode_bytes(batch, steps, warm) / (ms * 1e-3) / 1e9
            flat[f"{key}_decode_b{batch}"] = round(batch * 1000.0 / ms, 1)
            flat[f"{key}_decode_b{batch}_hbm_frac"] = round(gbs / peaks["hbm_gbs"], 4)
        pf_ms = b.prefill_run(PREFILL_TOKENS)
        flat[f"{key}_prefill_{PREFILL_TOKENS}"] = round(PREFILL_TOKENS * 1000.0 / pf_ms, 1)
        flat[f"{key}_prefill_{PREFILL_TOKENS}_frac"] = round(b.prefill_flops(PREFILL_TOKENS) / (pf_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)
        if mixed:
            nd, npor, por = 56, 8, 512
            rows = nd + npor * por
            ms = b.mixed_run(nd, npor, por, steps, warm)
            flat[f"mixed_{key}"] = round(rows * 1000.0 / ms, 1)
            flat[f"mixed_{key}_ms"] = round(ms, 3)
            flat[f"mixed_{key}_frac"] = round(b.mixed_flops(nd, npor, por) / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)
            # the step is bound on both sides: the decoding requests' cache and the weights have to be read, the
            # portions' products computed; the third figure is the time both would take one after the other at their
            # measured peaks, divided by the step's time
            mixed_bytes = b.runner.model.weight_bytes() + nd * CONTEXT * b.cache.bytes_per_token(b.esize)
            t_floor = b.mixed_flops(nd, npor, por) / (peaks["bf16_tflops_sustained"] * 1e12) + mixed_bytes / (peaks["hbm_gbs"] * 1e9)
            flat[f"mixed_{key}_hbm_frac"] = round(mixed_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
            flat[f"mixed_{key}_frac_of_both"] = round(t_floor / (ms * 1e-3), 4)
            s_step, tok_step = b.mixed_e2e(nd, npor, por, steps, warm)
            flat[f"mixed_{key}_e2e"] = round(rows / s_step, 1)
            flat[f"mixed_{key}_e2e_ms"] = round(s_step * 1000, 3)
            rec["mixed"] = {"rows_per_step": rows, "logit_rows": nd + npor, "sampled_per_step_e2e": round(tok_step, 1),
                            "what": f"{npor} prompt portions of {por} tokens (each the start of a prompt) beside {nd} "
                                    f"requests decoding at context {CONTEXT}; tokens/s counts all {rows} rows"}
    finally:
        clocks = sampler.stop()
        b.close()
    flat[f"{key}_sm_mhz"] = clocks.get("sm_mhz")
    rec.update({k[len(key) + 1:] if k.startswith(key + "_") else k: v for k, v in flat.items()})
    rec["clocks"] = clocks
    return flat, rec


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
    ap.add_argument("--skip-points", action="store_true", help="skip the batch-1/64 points, the prefills and the other sizes")
    ap.add_argument("--sizes", default=None,
                    help="other sizes to measure after the headline one, comma separated (default: 0.6b,32b when the headline "
                         "is the full 8B model in bfloat16; 'none' to skip)")
    ap.add_argument("--long-prefill", default=None,
                    help="further prefill lengths at the headline sizes, comma separated (default 8192,32768 with the "
                         "full model; 'none' to skip)")
    ap.add_argument("--long-decode", default=None,
                    help="further decode points at the headline sizes as BATCHxCONTEXT, comma separated (default 8x16384,1x32768 "
                         "with the full model; 'none' to skip)")
    ap.add_argument("--batch-invariant", action="store_true",
                    help="measure under the batch-invariant numeric policy (one product kernel, fixed key slices)")
    ap.add_argument("--timeline", default=None, metavar="FILE",
                    help="write the start and end of every kernel of one decode step (CUPTI through torch.profiler: kernels "
                         "overlap under programmatic dependent launch, which a serialising profiler cannot show) and exit")
    ap.add_argument("--sampler", action="store_true",
                    help="time the sampling kernels alone (vocabulary of the model, --batch rows, recorded into a CUDA "
                         "graph): one JSON line of microseconds per call and setting, then exit")
    ap.add_argument("--profile", choices=["decode", "prefill", "mixed", "sampler"], default=None,
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

    mods = {"resolve_architecture": resolve_architecture, "LLM": LLM, "ModelRunner": ModelRunner, "StepEntry": StepEntry,
            "klib": klib, "ops": ops, "SamplingParams": SamplingParams}
    if args.batch_invariant:
        from openinfer_b200.kernels import policy
        policy.set_batch_invariant(True)
    if args.sampler or args.profile == "sampler":
        return sampler_mode(args, torch, ops, MODELS[args.model][1]["vocab_size"])
    peaks, peaks_src = read_peaks()
    model_name, model_cfg = MODELS[args.model]
    K, W, B = args.steps, args.warmup, args.batch
    headline_full = args.model == "8b" and not args.layers and args.dtype == "bfloat16" and not args.batch_invariant
    long_prefill = [] if args.skip_points else \
        ([8192, 32768] if headline_full else []) if args.long_prefill is None else \
        [int(x) for x in args.long_prefill.split(",") if x and x != "none"]
    long_decode = ([(8, 16384), (1, 32768)] if headline_full else []) if args.long_decode is None else \
        [tuple(int(v) for v in x.split("x")) for x in args.long_decode.split(",") if x and x != "none"]
    sizes = [] if args.skip_points else \
        (["0.6b", "32b"] if headline_full else []) if args.sizes is None else \
        [x for x in args.sizes.split(",") if x and x != "none"]
    for x in sizes:
        if x not in MODELS:
            ap.error(f"--sizes: unknown size {x!r}")
    max_batch = max(B, 64) if (not args.skip_points or args.profile == "mixed") else B
    # Through the entry point the requests' prompts are computed one portion a step, and a request that has its
    # prompt decodes while the others' are still computed: it must not finish before all of them decode.
    e2e_prompt_steps = max(B, 8) * -(-CONTEXT // PREFILL_TOKENS)
    e2e_new_tokens = W + K + e2e_prompt_steps + 8
    bench = Bench(torch, mods, model_cfg, args.dtype, max_batch, e2e_new_tokens, CONTEXT,
                  prefill_room=max([PREFILL_TOKENS] + long_prefill), layers=args.layers)
    runner, config, cache, dev, rng, vocab = bench.runner, bench.config, bench.cache, bench.dev, bench.rng, bench.vocab
    full_layers = bench.full_layers
    fake_context = bench.fake_context

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
        elif args.profile == "mixed":
            ids = [f"p{i}" for i in range(56)]
            for rid in ids:
                fake_context(rid, CONTEXT)
            parts = [[rng.randrange(vocab) for _ in range(512)] for _ in range(8)]
            for i in range(W + 1):
                if i == W:
                    torch.cuda.synchronize()
                    torch.cuda.profiler.start()
                runner.step([StepEntry(rid, [1], [0]) for rid in ids]
                            + [StepEntry(f"pp{i}_{j}", p, [511]) for j, p in enumerate(parts)])
                torch.cuda.synchronize()
                for j in range(8):
                    runner.end(f"pp{i}_{j}")
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
    ms_step, launches = bench.decode_run(B, K, W)
    clocks = sampler.stop()
    value = B * 1000.0 / ms_step

    # roofline of the decode step: every weight once + the cache of the live requests
    step_bytes = bench.decode_bytes(B, K, W)
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
    del llm

    weights_gb = runner.model.weight_bytes() / 1e9
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
            "parallelism": "single GPU",
            "l2": f"no flush: a step reads {step_bytes / 1e9:.2f} GB ({weights_gb:.2f} GB of weights), L2 holds 0.126 GB",
        },
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
    }
    if args.batch_invariant:
        out["config"]["batch_invariant"] = True

    if not args.skip_points:
        points = {}
        for b in (1, 64):
            steps = max(16, K // 2)
            ms_b, _ = bench.decode_run(b, steps, max(3, W // 2))
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
        out["points"] = points

        # prefill of one 2,048-token prompt in one step
        T = PREFILL_TOKENS
        pf_ms = bench.prefill_run(T)
        flops = bench.prefill_flops(T)
        peak_tf = peaks["bf16_tflops"] if args.dtype == "bfloat16" else 75.0
        out["prefill"] = {"value": round(T * 1000.0 / pf_ms, 1), "tokens": T, "ms": round(pf_ms, 3),
                          "frac": round(flops / (pf_ms * 1e-3) / (peak_tf * 1e12), 4), "peaks": peaks_src}
        if args.dtype == "bfloat16":
            # the step is timed back to back after the decode runs, i.e. under the power cap: also against the
            # library product's SUSTAINED rate (a burst after idle runs this step in 23.6 ms instead of 26.5)
            out["prefill"]["frac_of_sustained"] = round(flops / (pf_ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)
        for T in long_prefill:
            ms_t = bench.prefill_run(T, reps=2, warm=1)
            points[f"prefill_{T}"] = round(T * 1000.0 / ms_t, 1)
            points[f"prefill_{T}_frac"] = round(bench.prefill_flops(T) / (ms_t * 1e-3) / (peak_tf * 1e12), 4)
    runner = cache = None
    bench.close()
    if long_decode and not args.skip_points:
        # decoding at longer contexts, where the cache outweighs the weights: (batch, context) pairs at the headline sizes
        for b, ctx in long_decode:
            steps = max(16, K // 4)
            lb = Bench(torch, mods, model_cfg, args.dtype, b, 2 * steps + 32, ctx, layers=args.layers)
            try:
                warm = max(3, W // 2)
                ms_b, _ = lb.decode_run(b, steps, warm)
                gbs = lb.decode_bytes(b, steps, warm) / (ms_b * 1e-3) / 1e9
                out["points"][f"decode_b{b}_ctx{ctx}"] = round(b * 1000.0 / ms_b, 1)
                out["points"][f"decode_b{b}_ctx{ctx}_hbm_frac"] = round(gbs / peaks["hbm_gbs"], 4)
            finally:
                lb.close()
    if sizes:
        out["sizes"] = {}
        for key in sizes:
            flat, rec = measure_size(torch, mods, key, args, peaks, mixed=(key == "0.6b"))
            out["points"].update(flat)
            out["sizes"][key] = rec
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
