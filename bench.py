"""Decode and prefill throughput of the engine at the Llama-3.1-8B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line. `value`: decoded tokens per second at batch 8, timed on the device
with CUDA events over K decode steps after W warm-up steps, each request holding
a 2,048-token prompt (real prefill through the engine) and decoding from there.
`e2e`: the same through the Python entry point (Engine.submit / Engine.step),
host token lists in and host token ids out every step. `prefill`: one 2,048-token
prompt in one step. `roofline`: bytes the decode step must read (every weight
once, the cache of the live requests) over its time, against the measured copy
bandwidth. `points`: decode at batch 1 and 64 at the same context, and at batch 1,
8 and 64 at the end of the configuration's context (the K timed steps end at 4,096
tokens); their caches are filled with random keys and values instead of being
prefilled: a decode step's time does not depend on the cache's contents. Each has
its own entry in `rooflines`. Two serving runs through Engine.submit / Engine.step
follow, each with its own model (`serving`): `mixed_1b`, 64 requests with prompts of
128 to 4,096 tokens on the Llama-3.2-1B shape, prompts cut into portions of 512
beside the decoding requests, 512 new tokens each (and the same with a third of the
pages, so that requests are preempted and recomputed); `serve_13b`, 32 requests of
1,024 prompt tokens and 512 new tokens on the Llama-2-13B shape. They report
all tokens per second (prompt and generated, over the whole run) and generated
tokens per second of the phase in which every request decodes, against the bytes
such a step must read. Weights are random (N(0, 0.02)) and drawn on the device;
token ids are uniform random. The weights (16 GB) and caches are far larger than L2
(126 MB), so no L2 flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 32,
    "hidden_size": 4096,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "intermediate_size": 14336,
    "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 131072,
}
LLAMA32_1B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 16,
    "hidden_size": 2048,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 64,
    "intermediate_size": 8192,
    "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "max_position_embeddings": 131072,
}
LLAMA2_13B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 40,
    "hidden_size": 5120,
    "num_attention_heads": 40,
    "num_key_value_heads": 40,
    "head_dim": 128,
    "intermediate_size": 13824,
    "vocab_size": 32000,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 4096,
}
PROMPT_LEN = 2048
CONTEXT_LEN = 4096
PAGE_SIZE = 16


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timed work runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int = 0):
        self.index = index
        self.samples: list[list[str]] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=5)

    def summary(self) -> dict:
        sm, sm_max, reasons = [], [], set()
        for row in self.samples:
            try:
                sm.append(float(row[0]))
                sm_max.append(float(row[1]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(self.NAMES, row[2:]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_config(layers: int) -> dict:
    cfg = dict(LLAMA31_8B)
    cfg["num_hidden_layers"] = layers
    return cfg


def weight_bytes(cfg: dict, width: int = 2) -> int:
    """Bytes of every weight a decode step reads once: all layer matrices and norms,
    the final norm and the lm_head (embedding rows are gathered, not streamed)."""
    h, i = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * h + h * nh * hd + 3 * i * h + 2 * h
    return (cfg["num_hidden_layers"] * per_layer + cfg["vocab_size"] * h + h) * width


def kv_bytes_per_token(cfg: dict, width: int = 2) -> int:
    return cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * width


def prefill_flops(cfg: dict, tokens: int, logit_rows: int = 1) -> float:
    h, i = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = 2.0 * tokens * ((nh + 2 * nkv) * hd * h + h * nh * hd + 3 * i * h)
    attention = 4.0 * nh * hd * tokens * (tokens + 1) / 2
    return cfg["num_hidden_layers"] * (per_layer + attention) + 2.0 * logit_rows * cfg["vocab_size"] * h


def fill_cache(engine, batch: int, length: int, tag: str) -> list:
    """Opens `batch` requests holding `length` tokens each without running a
    prefill; the pools are filled with small random numbers once."""
    ids = []
    for b in range(batch):
        rid = (tag, b)
        assert engine.cache.open(rid) is not None, "too few slots"
        assert engine.cache.reserve(rid, length), "too few pages"
        engine.cache.commit(rid, length)
        ids.append(rid)
    return ids


def time_decode(engine, ids: list, steps: int, warmup: int, vocab: int):
    """K graph-replayed decode steps on the device (CUDA events). Tokens fed are
    fixed (the step's time does not depend on them); positions advance."""
    import torch

    from pulsarlm_b200.engine.runner import StepEntry
    from pulsarlm_b200.sampling.params import SamplingParams

    params = [SamplingParams()] * len(ids)
    seeds = [0] * len(ids)
    entries = [StepEntry(r, [(7 * i + 3) % vocab], [0]) for i, r in enumerate(ids)]
    for _ in range(warmup):
        engine.runner.decode_step(entries, params, seeds, [0] * len(ids))
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before_steps = engine.runner.graph_steps
    start.record()
    for _ in range(steps):
        engine.runner.decode_step(entries, params, seeds, [0] * len(ids))
    end.record()
    torch.cuda.synchronize()
    engine.runner.check_status()
    graph = engine.runner.last_graph
    launches = graph.launches * (engine.runner.graph_steps - before_steps)
    return start.elapsed_time(end) / steps, launches


def describe(cfg: dict) -> str:
    return (f"{cfg['num_hidden_layers']} layers, hidden {cfg['hidden_size']}, heads {cfg['num_attention_heads']}/"
            f"{cfg['num_key_value_heads']}, head_dim {cfg['head_dim']}, intermediate {cfg['intermediate_size']}, "
            f"vocab {cfg['vocab_size']}, {'tied' if cfg['tie_word_embeddings'] else 'untied'} head")


def serve(engine, cfg: dict, prompts: list, max_new: int, pk: dict) -> dict:
    """Submits every prompt at once and steps the engine until all are done (host token
    lists in, host token ids out). Times the whole run, and within it the phase in
    which every request is decoding (from the step after the last prompt ends to the
    first request's end), whose steps are compared with the bytes they must read."""
    import torch

    from pulsarlm_b200 import SamplingParams

    greedy = SamplingParams(temperature=0.0)
    captures_before = engine.runner.graph_captures
    steps_before = engine.runner.steps
    preempted_before = engine.scheduler.preemptions
    torch.cuda.synchronize()
    t_start = time.perf_counter()
    requests = [engine.submit(p, sampling=greedy, max_tokens=max_new, ignore_eos=True) for p in prompts]
    weights = weight_bytes(cfg)
    per_token = kv_bytes_per_token(cfg)
    phase = None  # [seconds at start, tokens generated at start, steps, bytes]
    closed = None
    while engine.has_work():
        everyone_decodes = closed is None and all(r.output and not r.finished for r in requests)
        if everyone_decodes and phase is None:
            engine.sync()
            torch.cuda.synchronize()
            phase = [time.perf_counter(), sum(len(r.output) for r in requests), 0, 0.0]
        elif phase is not None and closed is None and not everyone_decodes:
            engine.sync()
            torch.cuda.synchronize()
            closed = (time.perf_counter(), sum(len(r.output) for r in requests))
        if phase is not None and closed is None:
            phase[2] += 1
            phase[3] += weights + per_token * sum(len(r.prompt) + len(r.output) for r in requests)
        engine.step()
    engine.sync()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t_start
    engine.runner.check_status()
    assert all(r.finish_reason == "length" and len(r.output) == max_new for r in requests), "a request fell short"
    prompt_tokens = sum(len(p) for p in prompts)
    generated = sum(len(r.output) for r in requests)
    out = {"requests": len(prompts), "prompt_tokens": prompt_tokens, "generated_tokens": generated,
           "seconds": seconds, "tok_s": (prompt_tokens + generated) / seconds,
           "steps": engine.runner.steps - steps_before,
           "preemptions": engine.scheduler.preemptions - preempted_before,
           "graph_captures_in_run": engine.runner.graph_captures - captures_before}
    if phase is not None and closed is not None and phase[2] > 0:
        span = closed[0] - phase[0]
        bytes_per_step = phase[3] / phase[2]
        ms = span / phase[2] * 1e3
        out.update({"decode_tok_s": (closed[1] - phase[1]) / span, "decode_steps": phase[2], "decode_ms_per_step": ms,
                    "decode_bytes_per_step": bytes_per_step,
                    "decode_floor_ms": bytes_per_step / (pk["hbm_gbs"] * 1e9) * 1e3,
                    "decode_frac": bytes_per_step / (ms / 1e3) / 1e9 / pk["hbm_gbs"]})
    return out


def run_serving(name: str, cfg: dict, lengths: list, max_new: int, pk: dict, tight: bool) -> dict:
    """Builds the model, serves a warm-up pass over the same prompts (library set-up,
    the decode steps' captures), then the timed pass; with `tight`, once more with a third
    of the pages, so that the scheduler has to preempt and recompute."""
    import gc

    import torch

    from pulsarlm_b200 import Engine

    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
    need_pages = sum(-(-(n + max_new + 2) // PAGE_SIZE) for n in lengths)
    engine = Engine(cfg, dtype="bfloat16", device="cuda:0", n_pages=need_pages + 64, page_size=PAGE_SIZE,
                    prefill_tokens_per_step=512, max_requests=len(lengths), seed=0)
    # The warm-up pass is the whole workload once: every shape of decode step that the timed
    # pass meets has then been captured, as in an engine that has been serving for a while.
    serve(engine, cfg, prompts, max_new, pk)
    result = serve(engine, cfg, prompts, max_new, pk)
    result["model"] = describe(cfg)
    result["prefill_tokens_per_step"] = 512
    if tight:
        small = Engine(engine.model, n_pages=max(need_pages // 3, -(-(max(lengths) + max_new + 2) // PAGE_SIZE) + 1),
                       page_size=PAGE_SIZE, prefill_tokens_per_step=512, max_requests=len(lengths))
        serve(small, cfg, prompts, min(128, max_new), pk)  # (warm-up: this engine's own captures)
        pressed = serve(small, cfg, prompts, min(128, max_new), pk)
        result["tight_pages"] = {k: pressed[k] for k in ("tok_s", "seconds", "steps", "preemptions",
                                                          "generated_tokens")}
        result["tight_pages"]["pages"] = small.cache.n_pages
        result["tight_pages"]["pages_for_everyone"] = need_pages
        del small
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    return result


def run_ours(args) -> dict:
    import torch

    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.engine.runner import StepEntry

    pk = peaks()
    cfg = model_config(args.layers)
    batch = args.batch
    torch.manual_seed(0)
    device = "cuda:0"
    max_batch = max(64, batch)
    phases = set(args.phases.split(","))
    per_request = CONTEXT_LEN + 64 if "ctx4096" in phases else PROMPT_LEN + 2 * (args.steps + args.warmup) + 128
    tokens_room = max_batch * per_request + 4 * PROMPT_LEN
    tokens_room = max(tokens_room, args.prefill_tokens + 4 * PROMPT_LEN)
    n_pages = -(-tokens_room // PAGE_SIZE)
    t0 = time.time()
    engine = Engine(cfg, dtype="bfloat16", device=device, n_pages=n_pages, page_size=PAGE_SIZE,
                    prefill_tokens_per_step=PROMPT_LEN, max_requests=max_batch + 2, seed=0)
    for g in engine.cache.groups:
        g.tensor.normal_(0.0, 0.5)
    vocab = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(1)
    setup_s = time.time() - t0

    prefill = e2e = None
    points: dict = {}
    rooflines: dict = {}
    serving: dict = {}

    def decode_point(name: str, b: int, first_context: int, steps: int) -> None:
        ids = fill_cache(engine, b, first_context, name)
        ms, _ = time_decode(engine, ids, steps, args.warmup, vocab)
        mid_context = first_context + args.warmup + steps / 2
        step_bytes = weight_bytes(cfg) + b * mid_context * kv_bytes_per_token(cfg)
        points[name] = b / (ms / 1e3)
        rooflines[name] = {"ms": ms, "context": mid_context, "bytes_per_step": step_bytes,
                           "achieved": step_bytes / (ms / 1e3) / 1e9,
                           "frac": step_bytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"]}
        for rid in ids:
            engine.cache.close(rid)

    ms_per_step, launches, achieved, step_bytes = None, 0, None, None
    clocks = ClockSampler()

    # ---- prefill: one 2,048-token prompt in one step, logits of the last token.
    if "prefill" in phases:
        n_prompt = args.prefill_tokens
        prompt = torch.randint(0, vocab, (n_prompt,), generator=gen).tolist()
        times = []
        for i in range(3 + 5):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.runner.step([StepEntry(("prefill", i), prompt, [n_prompt - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.runner.end(("prefill", i))
            if i >= 3:
                times.append(start.elapsed_time(end))
        prefill_ms = statistics.median(times)
        flops = prefill_flops(cfg, n_prompt)
        prefill = {"value": n_prompt / (prefill_ms / 1e3), "tokens": n_prompt, "ms": prefill_ms,
                   "frac": flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), "unit": "tok/s",
                   "peak_tflops": pk["bf16_tflops"]}

    # ---- end to end through the public API: batch prompts in, tokens out per step.
    if "e2e" in phases:
        prompts = [torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist() for _ in range(batch)]
        sampling = SamplingParams(temperature=0.0)
        # Requests finish their prompts one step apart, so the first is `batch` tokens
        # ahead of the last: give all of them room to still be decoding at the end.
        total_new = args.warmup + args.steps + batch + 8
        requests = [engine.submit(p, sampling=sampling, max_tokens=total_new, ignore_eos=True) for p in prompts]
        while any(len(r.output) < 1 for r in requests):
            engine.step()  # prefill (untimed)
        for _ in range(args.warmup):
            engine.step()
        engine.sync()  # the engine pipelines decode steps one deep: nothing in flight at the start,
        torch.cuda.synchronize()
        t_start = time.perf_counter()
        for _ in range(args.steps):
            engine.step()
        engine.sync()  # and every timed step's tokens read on the host at the end
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t_start
        assert all(not r.finished and len(r.output) >= args.warmup + args.steps + 1 for r in requests)
        graph = next(g for (n, _), g in engine.runner._graphs.items() if n == batch)
        e2e = {"value": batch * args.steps / e2e_s, "unit": "tok/s", "ms_per_step": e2e_s / args.steps * 1e3,
               "h2d_bytes_per_step": graph.layout.nbytes, "d2h_bytes_per_step": 4 * batch}
        for r in requests:
            r.cancel()
        engine.step()

    # ---- device-timed decode at the headline batch, same context.
    if "decode" in phases:
        ids = fill_cache(engine, batch, PROMPT_LEN + args.warmup, "main")
        with clocks:
            ms_per_step, launches = time_decode(engine, ids, args.steps, args.warmup, vocab)
        mid_context = PROMPT_LEN + 2 * args.warmup + args.steps / 2
        step_bytes = weight_bytes(cfg) + batch * mid_context * kv_bytes_per_token(cfg)
        achieved = step_bytes / (ms_per_step / 1e3) / 1e9
        for rid in ids:
            engine.cache.close(rid)

    # ---- other batch sizes.
    if "points" in phases:
        for b in (1, 64):
            decode_point(f"decode_b{b}", b, PROMPT_LEN, max(8, args.steps // 2))

        # a long prompt in the default portions: 8,192 tokens, 256 a step (tokens a second)
        long_prompt = torch.randint(0, vocab, (4 * PROMPT_LEN,), generator=gen).tolist()
        for attempt in ("warm", "timed"):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for at in range(0, len(long_prompt), 256):
                last = at + 256 >= len(long_prompt)
                engine.runner.step([StepEntry(("long", attempt), long_prompt[at:at + 256], [255] if last else [])])
            end.record()
            torch.cuda.synchronize()
            engine.runner.end(("long", attempt))
        points["prefill_8192_by_256"] = len(long_prompt) / (start.elapsed_time(end) / 1e3)
        # the same through the public entry point: milliseconds from submit to the first
        # token of a 2,048-token prompt, the scheduler cutting it into its default portions
        served = Engine(engine.model, n_pages=PROMPT_LEN // PAGE_SIZE + 8, page_size=PAGE_SIZE,
                        prefill_tokens_per_step=256, max_requests=2)
        first_prompt = torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist()
        for attempt in ("warm", "timed"):
            torch.cuda.synchronize()
            t_start = time.perf_counter()
            request = served.submit(first_prompt, sampling=SamplingParams(temperature=0.0), max_tokens=1,
                                    ignore_eos=True)
            while not request.finished:
                served.step()
            served.sync()
            points["first_token_ms_2048_by_256"] = (time.perf_counter() - t_start) * 1e3

    # ---- the end of the configuration's context: the timed steps end at 4,096 tokens.
    if "ctx4096" in phases:
        steps = max(8, args.steps // 2)
        for b in (1, 8, 64):
            decode_point(f"decode_b{b}_ctx4096", b, CONTEXT_LEN - steps - args.warmup, steps)

    # ---- serving runs on the other two shapes, each with its own model.
    if phases & {"mixed_1b", "serve_13b"}:
        import gc

        served = None
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        if "mixed_1b" in phases:
            lengths = torch.randint(128, 4097, (64,), generator=torch.Generator().manual_seed(3)).tolist()
            serving["mixed_1b"] = run_serving("mixed_1b", LLAMA32_1B, lengths, 512, pk, tight=True)
        if "serve_13b" in phases:
            serving["serve_13b"] = run_serving("serve_13b", LLAMA2_13B, [1024] * 32, 512, pk, tight=False)
        for name, run in serving.items():
            points[f"{name}_tok_s"] = run["tok_s"]
            if "decode_tok_s" in run:
                points[f"{name}_decode_tok_s"] = run["decode_tok_s"]
                rooflines[f"{name}_decode"] = {"ms": run["decode_ms_per_step"],
                                               "bytes_per_step": run["decode_bytes_per_step"],
                                               "achieved": run["decode_bytes_per_step"] / run["decode_ms_per_step"] / 1e6,
                                               "frac": run["decode_frac"]}

    clock_summary = clocks.summary()
    return {
        "metric": "decode tok/s at batch 8 (Llama-3.1-8B shape, 2,048-token prompts)",
        "value": batch / (ms_per_step / 1e3) if ms_per_step else None,
        "unit": "tok/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02) drawn on the device, uniform random token ids",
        "impl": "ours",
        "config": {
            "model": "Llama-3.1-8B shape", "layers": cfg["num_hidden_layers"], "layers_full": 32,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": batch, "seq_len": CONTEXT_LEN, "prompt_len": PROMPT_LEN,
            "decode_context_start": PROMPT_LEN + args.warmup, "page_size": PAGE_SIZE,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 16 GB)",
            "peaks": pk["source"],
            "mixed_1b_model": "Llama-3.2-1B shape: " + describe(LLAMA32_1B),
            "serve_13b_model": "Llama-2-13B shape: " + describe(LLAMA2_13B),
        },
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"] if achieved else None, "bytes_per_step": step_bytes},
        "points": points,
        "rooflines": rooflines,
        "serving": serving,
        "clocks": {"sm_mhz": clock_summary["sm_mhz"], "sm_max_mhz": clock_summary["sm_max_mhz"],
                   "reasons": clock_summary["reasons"]},
        "setup_s": setup_s,
    }


# ----------------------------------------------------------------------------- --design rerilorn
def rerilorn_config(width: int, layers: int, vocab: int = 32000) -> dict:
    """A Rerilorn model at a real model's layer sizes: every third layer a delta-rule layer
    (heads of 64), the others latent attention (16 heads of 64 over a latent of 128, window
    1,024), feed-forward 4 x width, four taps."""
    delta = {"type": "general_delta", "mixer": {"heads": width // 64, "dim": 64, "decay_rank": 64},
             "mlp": {"kind": "dense", "ff": 4 * width}}
    latent = {"type": "latent_attention",
              "mixer": {"heads": 16, "dim": 64, "vdim": 64, "kv_rank": 128, "mask": {"size": 1024}, "scale": 0.125},
              "mlp": {"kind": "dense", "ff": 4 * width}}
    return {"architecture": "Rerilorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "embedding": {"scale": float(width) ** 0.5}, "canon": {"taps": 4},
            "layers": [delta if i % 3 == 0 else latent for i in range(layers)]}


def bunosun_config(width: int, runs: int, vocab: int = 32000) -> dict:
    """A Bunosun model at a real model's layer sizes whose layers run `runs` times in all: a first
    layer, then a looped pair (run twice), the rest after it. Every third run is a channel-wise
    gated delta rule (heads of 64 x 64, four taps), the others differential attention (heads of two
    maps of 64 over values of 128, four heads per kv head, window 1,024, half of each map rotated).
    Feed-forward: 32 experts of width / 2 of which 4 are used, in 4 groups of which 2 stay, beside a
    shared expert of width / 2 (2.5 x width active per token)."""
    mlp = {"kind": "moe", "expert": {"ff": width // 2}, "shared": {"ff": width // 2},
           "router": {"experts": 32, "top": 4, "groups": {"count": 4, "keep": 2}}}
    heads = max(1, width // 128)
    attention = {"type": "attention", "mlp": mlp,
                 "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 64, "vdim": 128, "diff": 0.5,
                           "scale": 0.125, "mask": {"size": 1024},
                           "rot": {"base": 10000.0, "dims": 32, "scaling": {"factor": 4.0}}}}
    delta = {"type": "channel_delta", "mlp": mlp,
             "mixer": {"heads": width // 64, "kv_heads": width // 64, "dim": 64, "vdim": 64, "conv": 4,
                       "decay_rank": 64, "gate_rank": 64}}
    if runs >= 5:
        layers = [attention, attention, delta] + [attention if i % 3 else delta for i in range(1, runs - 4)]
        loop = {"start": 1, "stop": 3, "times": 2}
    else:
        layers = [attention, delta] + [attention] * (runs - 3)
        loop = {"start": 0, "stop": 1, "times": 2}
    return {"architecture": "Bunosun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "embedding": {"scale": float(width) ** 0.5}, "layers": layers, "loop": loop}


def simetar_config(width: int, layers: int, vocab: int = 32000) -> dict:
    """A Simetar model at a real model's layer sizes: conv attention (heads of 64 in groups of
    four whose values are their keys, four taps, window 1,024, scores capped at 50, all of a head
    rotated in neighbouring pairs with frequency bands) alternating with latent attention (16 heads
    of 64 + 32 over a latent of 96 and a shared rotated part of 32, values of 64, ramped
    frequencies); every fourth layer reads the latent cache of the layer two before it. Gated
    feed-forward of 8/3 x width, the Llama layer's."""
    ff = (8 * width // 3 + 255) // 256 * 256
    mlp = {"kind": "dense", "ff": ff}
    heads = width // 64
    conv = {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 64, "vdim": 64, "conv": 4, "scale": 0.125,
                      "softcap": 50.0, "mask": {"size": 1024},
                      "rot": {"base": 500000.0, "dims": 64,
                              "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": {"heads": 16, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 96, "scale": 0.1,
                        "rot": {"base": 10000.0, "dims": 32,
                                "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    out = []
    for i in range(layers):
        if i % 2 == 0:
            out.append(conv)
        elif i % 4 == 3:
            out.append({**latent, "mixer": {**latent["mixer"], "kv_from": i - 2}})
        else:
            out.append(latent)
    return {"architecture": "Simetar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": out}


def llama_config_like(width: int, layers: int, vocab: int = 32000) -> dict:
    """The Llama decoder at the same width, depth and vocabulary: heads of 64 in groups of
    four, gated feed-forward of 8/3 x width (the parameters of a plain one of 4 x width)."""
    cfg = dict(LLAMA32_1B)
    cfg.update({"num_hidden_layers": layers, "hidden_size": width, "num_attention_heads": width // 64,
                "num_key_value_heads": max(1, width // 256), "head_dim": 64,
                "intermediate_size": (8 * width // 3 + 255) // 256 * 256, "vocab_size": vocab,
                "tie_word_embeddings": True, "rope_scaling": None, "max_position_embeddings": 8192})
    return cfg


def time_kernel(fn, reps: int = 20, warmup: int = 3) -> float:
    """Milliseconds per call, CUDA events around `reps` calls after `warmup`; a 256 MB buffer is
    rewritten between calls so that no call finds its inputs in L2."""
    import torch

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda:0")
    for _ in range(warmup):
        fn()
    total = 0.0
    for _ in range(reps):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        total += start.elapsed_time(end)
    return total / reps


def design_kernels(width: int, pk: dict) -> dict:
    """The new design's kernels alone at one layer's sizes, beside the like kernel of the
    Llama layer where there is one: milliseconds, algorithmic bytes, fraction of the copy
    bandwidth."""
    import torch

    from pulsarlm_b200.kernels import ops

    dev, bf = "cuda:0", torch.bfloat16
    out: dict = {}

    def note(name, ms, nbytes):
        out[name] = {"ms": ms, "bytes": nbytes, "frac_of_hbm": nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"]}

    for tokens, entries in ((2048, 1), (64, 64)):
        tag = f"T{tokens}_E{entries}"
        per = tokens // entries
        entry = torch.arange(entries, dtype=torch.int32, device=dev).repeat_interleave(per)
        slots = torch.arange(entries, dtype=torch.int32, device=dev)
        first = torch.arange(0, tokens, per, dtype=torch.int32, device=dev)
        count = torch.full((entries,), per, dtype=torch.int32, device=dev)
        x = torch.randn((tokens, width), device=dev)
        y = torch.randn((tokens, width), device=dev).to(bf)
        h = torch.empty_like(y)
        w32 = torch.ones(width, device=dev)
        note(f"add_normed_rmsnorm_{tag}", time_kernel(lambda: ops.add_normed_rmsnorm(x, y, w32, 0.5, 1e-6, w32, 1e-6, h)),
             tokens * width * (4 + 4 + 2 + 2))
        note(f"add_rmsnorm_{tag} (Llama)", time_kernel(lambda: ops.add_rmsnorm(x, y, w32, 1e-6, h)),
             tokens * width * (4 + 4 + 2 + 2))
        state = torch.zeros((entries + 1, 3, width), dtype=bf, device=dev)
        cw = torch.randn((width, 4), device=dev)

        def conv():
            ops.short_conv(y, cw, state, entry, slots, h)
            ops.short_conv_state(y, entry, slots, state)
        note(f"short_conv_{tag}", time_kernel(conv), tokens * width * 4 + entries * 3 * width * 4)
        heads = width // 64
        proj = torch.randn((tokens, 5 * width + 64), device=dev).to(bf)
        w_pre = torch.randn((tokens, width), device=dev).to(bf)
        S = torch.zeros((entries + 1, heads, 64, 64), device=dev)
        o = torch.empty((tokens, width), dtype=bf, device=dev)
        parts = [proj[:, i * width:(i + 1) * width] for i in range(5)]
        note(f"delta_rule_{tag}",
             time_kernel(lambda: ops.delta_rule(*parts, w_pre, w32, w32, w32, S, first, count, slots, o, heads, 64,
                                                0.6065, 1e-6, 1e-6)),
             tokens * width * 2 * 7 + entries * heads * 64 * 64 * 4 * 2)
    # attention of 64 single tokens over 1,024 keys: 16 heads over a latent of 128 with sink,
    # gate and split weights, beside 16 heads in 4 groups over keys and values of 128 without
    page, keys, batch = 16, 1024, 64
    n_pages = batch * keys // page
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, keys // page)
    pos = torch.full((batch,), keys - 1, dtype=torch.int32, device=dev)
    ent = torch.arange(batch, dtype=torch.int32, device=dev)
    q = torch.randn((batch, 16, 128), device=dev).to(bf)
    res = torch.empty_like(q)
    latent = torch.randn((n_pages, 1, page, 128), device=dev).to(bf)
    sinks = torch.zeros(16, device=dev)
    gate = torch.zeros((batch, 16), dtype=bf, device=dev)
    extras = ops.attention_extras(q, sinks, gate, True)
    for splits in (1, 2, 4):
        scratch = torch.empty(ops.attention_decode_scratch_floats(batch, 16, 128, splits), device=dev)
        note(f"attention_decode_latent_b64_k1024_splits{splits}",
             time_kernel(lambda: ops.attention_decode(q, latent, latent, table, pos, ent, res, page, 1024, 0.1, splits,
                                                      scratch, extras=extras)), batch * keys * 128 * 2)
    kv = torch.randn((2, n_pages, 4, page, 128), device=dev).to(bf)
    for splits in (1, 2, 4):
        scratch = torch.empty(ops.attention_decode_scratch_floats(batch, 16, 128, splits), device=dev)
        note(f"attention_decode_b64_k1024_splits{splits} (Llama, 4 kv heads)",
             time_kernel(lambda: ops.attention_decode(q, kv[0], kv[1], table, pos, ent, res, page, 1024, 0.1, splits,
                                                      scratch)), batch * keys * 4 * 128 * 2 * 2)
    # a 2,048-token prompt: the tiled kernel over the latent with and without the extras
    tokens = 2048
    n_pages = tokens // page
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, n_pages)
    q = torch.randn((tokens, 16, 128), device=dev).to(bf)
    res = torch.empty_like(q)
    latent = torch.randn((n_pages, 1, page, 128), device=dev).to(bf)
    gate = torch.zeros((tokens, 16), dtype=bf, device=dev)
    rows = ops.attention_prefill_tile_rows()
    tiles = torch.tensor([(r, min(rows, tokens - r), r, 0) for r in range(0, tokens, rows)], dtype=torch.int32,
                         device=dev)
    flops = 4.0 * 16 * 128 * sum(min(p + 1, 1024) for p in range(tokens))
    for name, ex in (("latent, sink, gate, split weights", ops.attention_extras(q, sinks, gate, True)),
                     ("latent, sink, gate", ops.attention_extras(q, sinks, gate, False)), ("plain", None)):
        ms = time_kernel(lambda: ops.attention_prefill(q, latent, latent, table, tiles, res, page, 1024, 0.1, extras=ex))
        out[f"attention_prefill_T2048_w1024 ({name})"] = {"ms": ms, "tflops": flops / (ms / 1e3) / 1e12}
    return out


def bunosun_kernels(width: int, pk: dict) -> dict:
    """The Bunosun design's kernels alone at one layer's sizes, each beside the like kernel of
    the Llama or Rerilorn layer: milliseconds, algorithmic bytes or FLOPs, fraction of the copy
    bandwidth."""
    import torch

    from pulsarlm_b200.kernels import ops
    from pulsarlm_b200.parts import moe as moe_part
    from pulsarlm_b200.parts.linear import gated_feed_forward
    from pulsarlm_b200.parts.registry import BuildContext
    from pulsarlm_b200.parts.spec import PartSpec

    dev, bf = "cuda:0", torch.bfloat16
    out: dict = {}

    def note(name, ms, nbytes=None, flops=None):
        out[name] = {"ms": ms}
        if nbytes is not None:
            out[name].update(bytes=nbytes, frac_of_hbm=nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"])
        if flops is not None:
            out[name].update(tflops=flops / (ms / 1e3) / 1e12, frac_of_bf16=flops / (ms / 1e3) / 1e12 / pk["bf16_tflops"])

    experts, top, ff = 32, 4, width // 2
    spec = PartSpec("moe", {"hidden_size": width, "expert_size": ff, "n_experts": experts, "top": top, "groups": 4,
                            "keep_groups": 2, "shared_size": None},
                    {"router": "r", "correction": "c", "expert_gate": "e{e}.g", "expert_up": "e{e}.u",
                     "expert_down": "e{e}.d"})
    part = moe_part.RoutedExperts(spec, BuildContext(bf, torch.device(dev)))
    tensors = {"r": torch.randn((experts, width), device=dev) * 0.02, "c": torch.zeros(experts, device=dev)}
    for e in range(experts):
        tensors[f"e{e}.g"] = (torch.randn((ff, width), device=dev) * 0.02).to(bf)
        tensors[f"e{e}.u"] = (torch.randn((ff, width), device=dev) * 0.02).to(bf)
        tensors[f"e{e}.d"] = (torch.randn((width, ff), device=dev) * 0.02).to(bf)
    part.load(tensors)
    del tensors
    dense_ff = top * ff
    dense_gate_up = (torch.randn((2 * dense_ff, width), device=dev) * 0.02).to(bf)
    dense_down = (torch.randn((width, dense_ff), device=dev) * 0.02).to(bf)
    for tokens, entries in ((2048, 1), (8, 8), (64, 64)):
        tag = f"T{tokens}_E{entries}"
        per = tokens // entries
        entry = torch.arange(entries, dtype=torch.int32, device=dev).repeat_interleave(per)
        slots = torch.arange(entries, dtype=torch.int32, device=dev)
        first = torch.arange(0, tokens, per, dtype=torch.int32, device=dev)
        count = torch.full((entries,), per, dtype=torch.int32, device=dev)
        x = torch.randn((tokens, width), device=dev)
        y = torch.randn((tokens, width), device=dev).to(bf)
        h, h2 = torch.empty_like(y), torch.empty_like(y)
        w32 = torch.ones(width, device=dev)
        note(f"pair_residual_norm_{tag}", time_kernel(lambda: ops.pair_residual_norm(x, y, w32, y, w32, None, w32, w32,
                                                                                     h, h2, 1e-6)),
             tokens * width * (4 + 4 + 2 + 2 + 2 + 2))
        note(f"add_rmsnorm_{tag} (Llama)", time_kernel(lambda: ops.add_rmsnorm(x, y, w32, 1e-6, h)),
             tokens * width * (4 + 4 + 2 + 2))
        # the routed feed-forward beside a dense gated one of the same active size
        hb = torch.randn((tokens, width), device=dev).to(bf)
        ids, _ = ops.moe_route(hb, part.router, part.correction, top, 4, 2)
        used = int(torch.unique(ids).numel())
        weight_bytes = used * 3 * ff * width * 2
        note(f"routed_experts_{tag} ({used} experts used)", time_kernel(lambda: part.forward(hb, None)),
             weight_bytes + tokens * width * 4, 2.0 * tokens * top * 3 * ff * width)
        note(f"gated_feed_forward_{tag} (Llama, the same active size)",
             time_kernel(lambda: gated_feed_forward(hb, dense_gate_up, dense_down)),
             3 * dense_ff * width * 2 + tokens * width * 4, 2.0 * tokens * 3 * dense_ff * width)
        note(f"moe_route_{tag}", time_kernel(lambda: ops.moe_route(hb, part.router, part.correction, top, 4, 2)),
             tokens * width * 2 + experts * width * 4)
        # the recurrence beside the generalized delta rule's (heads of 64 x 64 both)
        heads = width // 64
        qkv = torch.randn((tokens, 3 * width), device=dev).to(bf)
        b_pre = torch.randn((tokens, heads), device=dev).to(bf)
        a_pre = torch.randn((tokens, width), device=dev).to(bf)
        g_pre = torch.randn((tokens, width), device=dev).to(bf)
        S = torch.zeros((entries + 1, heads, 64, 64), device=dev)
        o = torch.empty((tokens, width), dtype=bf, device=dev)
        a_log = torch.zeros(heads, device=dev)
        note(f"gated_delta_{tag}",
             time_kernel(lambda: ops.gated_delta(qkv[:, :width], qkv[:, width:2 * width], qkv[:, 2 * width:], b_pre, a_pre,
                                                 g_pre, a_log, w32, torch.ones(64, device=dev), S, first, count, slots, o,
                                                 heads, heads, 64, 64, 1e-6, 0.125, 1e-6)),
             tokens * width * 2 * 6 + entries * heads * 64 * 64 * 4 * 2)
        proj = torch.randn((tokens, 5 * width + 64), device=dev).to(bf)
        parts = [proj[:, i * width:(i + 1) * width] for i in range(5)]
        note(f"delta_rule_{tag} (Rerilorn)",
             time_kernel(lambda: ops.delta_rule(*parts, a_pre, w32, w32, w32, S, first, count, slots, o, heads, 64,
                                                0.6065, 1e-6, 1e-6)),
             tokens * width * 2 * 7 + entries * heads * 64 * 64 * 4 * 2)
        state = torch.zeros((entries + 1, 3, 3 * width), dtype=bf, device=dev)
        cw = torch.randn((3 * width, 4), device=dev)
        filtered = torch.empty((tokens, 3 * width), dtype=bf, device=dev)

        def conv():
            if per == 1 and ops.short_conv_single(qkv, cw, state, entry, slots, filtered, residual=False, act="silu"):
                return
            ops.short_conv_act(qkv, cw, state, entry, slots, filtered, residual=False, act="silu")
            ops.short_conv_state_strided(qkv, entry, slots, state)
        note(f"short_conv_silu_{tag} (3 x width channels)", time_kernel(conv), tokens * 3 * width * 4 + entries * 9 * width * 4)
        # the maps' layout, rotation and cache write beside the Llama layer's rotation and write
        n_heads, n_kv, page = width // 128, max(1, width // 512), 16
        n_pages = tokens // page + entries + 1
        pools = torch.zeros((2, n_pages, n_kv, page, 128), dtype=bf, device=dev)
        table = torch.arange(entries * (per // page + 1), dtype=torch.int32, device=dev).view(entries, -1)
        pos = torch.arange(per, dtype=torch.int32, device=dev).repeat(entries)
        mixed = torch.randn((tokens, (n_heads + 2 * n_kv) * 128), device=dev).to(bf)
        q_end, k_end = n_heads * 128, (n_heads + n_kv) * 128
        q_out = torch.empty((tokens, 2 * n_heads, 128), dtype=bf, device=dev)
        inv = torch.rand(16, dtype=torch.float64, device=dev)
        note(f"rope_maps_write_{tag}",
             time_kernel(lambda: ops.rope_maps_write(mixed[:, :q_end], mixed[:, q_end:k_end], mixed[:, k_end:], pos, entry,
                                                     table, pools[0], pools[1], page, inv, 32, n_heads, n_kv, 2, 64, 128,
                                                     q_out, None)),
             tokens * (n_heads * 128 * 2 * 3 + n_kv * 128 * 2 * 4))
        inv64 = torch.rand(64, dtype=torch.float64, device=dev)
        note(f"rope_kv_write_{tag} (Llama)",
             time_kernel(lambda: ops.rope_kv_write(mixed[:, :q_end].view(tokens, n_heads, 128),
                                                   mixed[:, q_end:k_end].view(tokens, n_kv, 128),
                                                   mixed[:, k_end:].view(tokens, n_kv, 128), pos, entry, table, pools[0],
                                                   pools[1], page, inv64, 128, None)),
             tokens * (n_heads * 128 * 2 * 2 + n_kv * 128 * 2 * 4))
        combined = torch.empty((tokens, n_heads * 128), dtype=bf, device=dev)
        note(f"diff_combine_{tag}", time_kernel(lambda: ops.diff_combine(q_out, combined, n_heads, 128, 0.4, 1e-6, 0.5)),
             tokens * n_heads * 128 * 2 * 3)
    return out


def simetar_kernels(width: int, pk: dict) -> dict:
    """The Simetar design's kernels alone at one layer's sizes, each beside the like kernel of the
    Llama layer: milliseconds, algorithmic bytes or FLOPs, fraction of the copy bandwidth."""
    import torch

    from pulsarlm_b200.kernels import ops

    dev, bf = "cuda:0", torch.bfloat16
    out: dict = {}

    def note(name, ms, nbytes=None, flops=None):
        out[name] = {"ms": ms}
        if nbytes is not None:
            out[name].update(bytes=nbytes, frac_of_hbm=nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"])
        if flops is not None:
            out[name].update(tflops=flops / (ms / 1e3) / 1e12, frac_of_bf16=flops / (ms / 1e3) / 1e12 / pk["bf16_tflops"])

    heads, kv, hd, page, taps = width // 64, max(1, width // 256), 64, 16, 4
    ff = (8 * width // 3 + 255) // 256 * 256
    for tokens, entries in ((2048, 1), (8, 8), (64, 64)):
        tag = f"T{tokens}_E{entries}"
        per = tokens // entries
        entry = torch.arange(entries, dtype=torch.int32, device=dev).repeat_interleave(per)
        slots = torch.arange(entries, dtype=torch.int32, device=dev)
        pos = torch.arange(per, dtype=torch.int32, device=dev).repeat(entries)
        n_pages = entries * (per // page + 1)
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(entries, -1)
        x = torch.randn((tokens, width), device=dev)
        y = torch.randn((tokens, width), device=dev).to(bf)
        h = torch.empty_like(y)
        w32 = torch.ones(width, device=dev)
        # a sublayer's output normed into the stream, and the next reader's input, in one pass
        note(f"add_layernorm_{tag}", time_kernel(lambda: ops.add_layernorm(x, y, w32, w32, 1e-6, h)),
             tokens * width * (4 + 4 + 2 + 2))
        note(f"add_rmsnorm_{tag} (Llama)", time_kernel(lambda: ops.add_rmsnorm(x, y, w32, 1e-6, h)),
             tokens * width * (4 + 4 + 2 + 2))
        # projection -> bias, convolution, two whole-projection norms, rotation, cache write
        c = (heads + kv) * hd
        proj = torch.randn((tokens, c + heads * hd), device=dev).to(bf)
        bias, cw = torch.randn(c, device=dev), torch.randn((c, taps), device=dev)
        state = torch.zeros((entries + 1, taps - 1, c), dtype=bf, device=dev)
        pools = torch.zeros((2, n_pages, kv, page, hd), dtype=bf, device=dev)
        q_out = torch.empty((tokens, heads * hd), dtype=bf, device=dev)
        inv = torch.rand(hd // 2, dtype=torch.float64, device=dev)
        qn, kn = torch.ones(heads * hd, device=dev), torch.ones(kv * hd, device=dev)

        def conv_write():
            ops.conv_norm_rope_write(proj[:, :c], bias, cw, state, slots, per == 1, qn, kn, 1e-6, inv, hd, True, 1.0,
                                     pos, entry, table, q_out, pools[0], pools[1], page, heads, kv, hd)
        note(f"conv_norm_rope_write_{tag}", time_kernel(conv_write),
             tokens * (c * 2 + heads * hd * 2 + 2 * kv * hd * 2) + entries * (taps - 1) * c * 2 * (2 if per == 1 else 1))
        if per > 1:  # (steps of single tokens move the stored inputs on in the launch above)
            note(f"short_conv_state_strided_{tag} (the portions' last inputs, kept for the next step)",
                 time_kernel(lambda: ops.short_conv_state_strided(proj[:, :c], entry, slots, state)),
                 entries * (taps - 1) * c * 2 * 2)
        mixed = torch.randn((tokens, (heads + 2 * kv) * hd), device=dev).to(bf)
        q_end, k_end = heads * hd, (heads + kv) * hd
        note(f"rope_kv_write_{tag} (Llama)",
             time_kernel(lambda: ops.rope_kv_write(mixed[:, :q_end].view(tokens, heads, hd),
                                                   mixed[:, q_end:k_end].view(tokens, kv, hd),
                                                   mixed[:, k_end:].view(tokens, kv, hd), pos, entry, table, pools[0],
                                                   pools[1], page, inv, hd, None)),
             tokens * (heads * hd * 2 * 2 + kv * hd * 2 * 4))
        # the latent layer: norm of the latent, rotation of the shared key part and of the queries' rotated part
        lh, ld, rot, rank = 16, 64, 32, 96
        lq = torch.randn((tokens, lh, ld + rot), device=dev).to(bf)
        lq_out = torch.empty((tokens, lh, rank + rot), dtype=bf, device=dev)
        z = torch.randn((tokens, rank + rot), device=dev).to(bf)
        lpool = torch.zeros((n_pages, 1, page, rank + rot), dtype=bf, device=dev)
        inv16 = torch.rand(rot // 2, dtype=torch.float64, device=dev)
        note(f"latent_rope_write_{tag}",
             time_kernel(lambda: ops.latent_rope_write(lq, lq_out, z, torch.ones(rank, device=dev), 1e-6, rank, rot, inv16,
                                                       False, 1.2, pos, entry, table, lpool, page)),
             tokens * (lh * rot * 2 * 2 + (rank + rot) * 2 * 2))
        # the feed-forward's and the mixers' gates
        gate_up = torch.randn((tokens, 2 * ff), device=dev).to(bf)
        act = torch.empty((tokens, ff), dtype=bf, device=dev)
        note(f"gated_act_gelu_tanh_{tag}", time_kernel(lambda: ops.gated_act(gate_up, act, "gelu_tanh")), tokens * ff * 6)
        note(f"swiglu_{tag} (Llama)", time_kernel(lambda: ops.swiglu(gate_up, act)), tokens * ff * 6)
        note(f"sigmoid_gate_{tag}", time_kernel(lambda: ops.sigmoid_gate(q_out, proj[:, c:])), tokens * heads * hd * 6)
    # attention of 64 single tokens over the last 1,024 of 2,048 keys: the cap and the sink, values
    # in a pool of their own, beside the Llama layer's kernel at the same shape
    keys, batch, window = 2048, 64, 1024
    n_pages = batch * keys // page
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, keys // page)
    pos = torch.full((batch,), keys - 1, dtype=torch.int32, device=dev)
    ent = torch.arange(batch, dtype=torch.int32, device=dev)
    q = torch.randn((batch, heads, hd), device=dev).to(bf)
    res = torch.empty_like(q)
    kvp = torch.randn((2, n_pages, kv, page, hd), device=dev).to(bf)
    sinks = torch.zeros(heads, device=dev)
    capped = ops.attention_extras(q, sinks, None, True, 50.0)
    read = batch * window * kv * hd * 2 * 2
    for splits in (1, 2, 4):
        scratch = torch.empty(ops.attention_decode_scratch_floats(batch, heads, hd, splits), device=dev)
        note(f"attention_decode_cap_sink_b64_w1024_splits{splits}",
             time_kernel(lambda: ops.attention_decode(q, kvp[0], kvp[1], table, pos, ent, res, page, window, 0.125, splits,
                                                      scratch, extras=capped)), read)
        note(f"attention_decode_b64_w1024_splits{splits} (Llama)",
             time_kernel(lambda: ops.attention_decode(q, kvp[0], kvp[1], table, pos, ent, res, page, window, 0.125, splits,
                                                      scratch)), read)
    note("attention_simt_cap_sink_b64_w1024 (the kernel of shapes the tensor-core kernels do not take)",
         time_kernel(lambda: ops.attention_simt(q, kvp[0], kvp[1], table, pos, ent, res, page, window, 0.125,
                                                softcap=50.0, sinks=sinks)), read)
    # a 2,048-token prompt through the tiled kernel, with and without the cap and the sink
    tokens = 2048
    n_pages = tokens // page
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, n_pages)
    q = torch.randn((tokens, heads, hd), device=dev).to(bf)
    res = torch.empty_like(q)
    kvp = torch.randn((2, n_pages, kv, page, hd), device=dev).to(bf)
    rows = ops.attention_prefill_tile_rows()
    tiles = torch.tensor([(r, min(rows, tokens - r), r, 0) for r in range(0, tokens, rows)], dtype=torch.int32,
                         device=dev)
    flops = 4.0 * heads * hd * sum(min(p + 1, window) for p in range(tokens))
    for name, ex in (("cap, sink, split weights", ops.attention_extras(q, sinks, None, True, 50.0)),
                     ("sink, split weights", ops.attention_extras(q, sinks, None, True)),
                     ("plain: Llama", None)):
        ms = time_kernel(lambda: ops.attention_prefill(q, kvp[0], kvp[1], table, tiles, res, page, window, 0.125,
                                                       extras=ex))
        note(f"attention_prefill_T2048_w1024 ({name})", ms, None, flops)
    return out


def puvirax_config(width: int, layers: int, vocab: int = 32000) -> dict:
    """A Puvirax model at a real model's layer sizes: heads of 64 in groups of four throughout; the layers
    cycle through attention with a norm over the whole q and k projections and a bias by distance (32 rows
    reaching 4,096 tokens back) over a dense feed-forward of 4 x width, rotary attention (half of every head
    rotated, frequency bands, unit q and k, a gate per head) over routed experts (16 of size width in 4 groups
    of which 2 stay, 2 chosen, beside a shared expert of 2 x width: the active parameters of the dense layer),
    rotary attention over a dense feed-forward, and attention with a norm per head, the same kind of bias and a
    window of 1,024 over routed experts. Every layer mixes its values with the first layer's. A pair table of
    65,521 rows; the head is the embedding table."""
    heads, kv = width // 64, max(1, width // 256)
    dense = {"kind": "dense", "ff": 4 * width}
    routed = {"kind": "moe", "expert": {"ff": width}, "shared": {"ff": 2 * width},
              "router": {"experts": 16, "top": 2, "groups": {"count": 4, "keep": 2}}}
    base = {"heads": heads, "kv_heads": kv, "dim": 64, "vdim": 64, "scale": 0.125, "v_mix": True}
    rot = {"base": 500000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    biased = {**base, "bias_max": 4096, "bias_rows": 32}
    cycle = [{"type": "attention_3", "mixer": biased, "mlp": dense},
             {"type": "attention", "mixer": {**base, "rot": rot}, "mlp": routed},
             {"type": "attention", "mixer": {**base, "rot": rot}, "mlp": dense},
             {"type": "attention_2", "mixer": {**biased, "mask": {"size": 1024}}, "mlp": routed}]
    return {"architecture": "Puvirax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "logit_scale": 0.5,
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}},
            "layers": [cycle[i % 4] for i in range(layers)]}


def puvirax_kernels(width: int, pk: dict) -> dict:
    """The Puvirax design's kernels alone at one layer's sizes, each beside the like kernel of the Llama layer
    (or, for the router and the experts, of the Bunosun layer): milliseconds, algorithmic bytes or FLOPs,
    fraction of the copy bandwidth."""
    import torch

    from pulsarlm_b200.kernels import ops
    from pulsarlm_b200.parts.normed_attention import bias_by_distance

    dev, bf = "cuda:0", torch.bfloat16
    out: dict = {}

    def note(name, ms, nbytes=None, flops=None):
        out[name] = {"ms": ms}
        if nbytes is not None:
            out[name].update(bytes=nbytes, frac_of_hbm=nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"])
        if flops is not None:
            out[name].update(tflops=flops / (ms / 1e3) / 1e12, frac_of_bf16=flops / (ms / 1e3) / 1e12 / pk["bf16_tflops"])

    heads, kv, hd, page, vocab, buckets = width // 64, max(1, width // 256), 64, 16, 32000, 65521
    experts, top, ff = 16, 2, width
    table_w = torch.randn((vocab, width), device=dev).to(bf)
    pairs_w = torch.randn((buckets + 1, width), device=dev).to(bf)
    router = torch.randn((experts, width), device=dev)
    correction = torch.randn(experts, device=dev) * 0.1
    gate_up = torch.randn((experts, 2 * ff, width), device=dev).to(bf)
    up, down = gate_up[:, :ff].contiguous(), torch.randn((experts, width, ff), device=dev).to(bf)
    for tokens, entries in ((2048, 1), (8, 8), (64, 64)):
        tag = f"T{tokens}_E{entries}"
        per = tokens // entries
        entry = torch.arange(entries, dtype=torch.int32, device=dev).repeat_interleave(per)
        slots = torch.arange(entries, dtype=torch.int32, device=dev)
        pos = torch.arange(1, per + 1, dtype=torch.int32, device=dev).repeat(entries)
        n_pages = entries * ((per + 1) // page + 1)
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(entries, -1)
        ids = torch.randint(0, vocab, (tokens,), dtype=torch.int32, device=dev)
        x = torch.empty((tokens, width), device=dev)
        last = torch.zeros(entries + 1, dtype=torch.int32, device=dev)
        note(f"pair_embed_{tag}", time_kernel(lambda: ops.pair_embed(table_w, pairs_w, ids, pos, entry, slots, last, x,
                                                                    1000003, 31, per == 1)), tokens * width * (2 + 2 + 4))
        note(f"embed_{tag} (Llama)", time_kernel(lambda: ops.embed(table_w, ids, x)), tokens * width * (2 + 4))
        # projection -> norms, rotation, value mixing, cache write
        proj = torch.randn((tokens, (heads + 2 * kv) * hd + 8), device=dev).to(bf)
        q_end, k_end, v_end = heads * hd, (heads + kv) * hd, (heads + 2 * kv) * hd
        q, k, v = (proj[:, :q_end].view(tokens, heads, hd), proj[:, q_end:k_end].view(tokens, kv, hd),
                   proj[:, k_end:v_end].view(tokens, kv, hd))
        first = torch.randn((tokens, kv, hd), device=dev).to(bf)
        pools = torch.zeros((2, n_pages, kv, page, hd), dtype=bf, device=dev)
        q_out = torch.empty((tokens, heads, hd), dtype=bf, device=dev)
        inv = torch.rand(hd // 4, dtype=torch.float64, device=dev)
        moved = tokens * ((heads + 3 * kv) * hd * 2 + (heads + 2 * kv) * hd * 2)
        for mode, wq, wk, rot in (("unit_after", None, None, inv), ("per_head", torch.ones(hd, device=dev), torch.ones(hd, device=dev), None),
                                  ("whole", torch.ones(heads * hd, device=dev), torch.ones(kv * hd, device=dev), None)):
            note(f"norm_rope_mix_write_{mode}_{tag}",
                 time_kernel(lambda: ops.norm_rope_mix_write(q, k, v, first, 0.3, q_out, pos, entry, table, pools[0], pools[1],
                                                             page, rot, hd // 2, mode, wq, wk, 1e-6)), moved)
        inv_full = torch.rand(hd // 2, dtype=torch.float64, device=dev)
        note(f"rope_kv_write_{tag} (Llama)",
             time_kernel(lambda: ops.rope_kv_write(q, k, v, pos, entry, table, pools[0], pools[1], page, inv_full, hd, None)),
             tokens * (heads * hd * 2 * 2 + kv * hd * 2 * 4))
        # the router, and the experts pair by pair (steps of few tokens)
        h = torch.randn((tokens, width), device=dev).to(bf)
        route_bytes = tokens * width * 2 + experts * width * 4
        note(f"moe_route_sigmoid_two_best_{tag}",
             time_kernel(lambda: ops.moe_route(h, router, correction, top, 4, 2, True, 2, False)), route_bytes)
        note(f"moe_route_softmax_{tag} (Bunosun)",
             time_kernel(lambda: ops.moe_route(h, router, correction, top, 4, 2)), route_bytes)
        if tokens <= 8:
            chosen, weights = ops.moe_route(h, router, correction, top, 4, 2, True, 2, False)
            act = torch.empty((tokens * top, ff), dtype=bf, device=dev)
            res = torch.empty((tokens, width), dtype=bf, device=dev)
            note(f"moe_up_{tag}", time_kernel(lambda: ops.moe_up(h, up, chosen, act)), tokens * top * ff * width * 2)
            note(f"moe_gate_up_{tag} (Bunosun)", time_kernel(lambda: ops.moe_gate_up(h, gate_up, chosen, act)),
                 tokens * top * 2 * ff * width * 2)
            note(f"moe_down_{tag} (both)", time_kernel(lambda: ops.moe_down(act, down, chosen, weights, None, res)),
                 tokens * top * ff * width * 2)
        z = torch.randn((tokens, 4 * width), device=dev).to(bf)
        squared = torch.empty_like(z)
        note(f"bias_act_relu2_{tag}", time_kernel(lambda: ops.bias_act(z, None, squared, "relu2")), tokens * 4 * width * 4)
        half = torch.empty((tokens, 2 * width), dtype=bf, device=dev)
        note(f"swiglu_{tag} (Llama)", time_kernel(lambda: ops.swiglu(z, half)), tokens * 4 * width * 3)
    # attention of 64 single tokens over 2,048 keys (a window of 1,024, and none): the bias by distance and the
    # gate per head beside the Llama layer's kernel at the same shape
    keys, batch = 2048, 64
    n_pages = batch * keys // page
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, keys // page)
    pos = torch.full((batch,), keys - 1, dtype=torch.int32, device=dev)
    ent = torch.arange(batch, dtype=torch.int32, device=dev)
    q = torch.randn((batch, heads, hd), device=dev).to(bf)
    res = torch.empty_like(q)
    kvp = torch.randn((2, n_pages, kv, page, hd), device=dev).to(bf)
    bias = bias_by_distance(torch.randn((32, heads), device=dev), 4096.0)
    gate = torch.randn((batch, heads), device=dev).to(bf)
    for window in (1024, None):
        read = batch * (window or keys) * kv * hd * 2 * 2
        name = f"w{window}" if window else "causal"
        for splits in (1, 4):
            scratch = torch.empty(ops.attention_decode_scratch_floats(batch, heads, hd, splits), device=dev)
            note(f"attention_decode_bias_b64_{name}_splits{splits}",
                 time_kernel(lambda: ops.attention_decode(q, kvp[0], kvp[1], table, pos, ent, res, page, window, 0.125, splits,
                                                          scratch, extras=ops.attention_extras(q, None, None, False, 0.0, bias))),
                 read)
            note(f"attention_decode_bias_gate_b64_{name}_splits{splits}",
                 time_kernel(lambda: ops.attention_decode(q, kvp[0], kvp[1], table, pos, ent, res, page, window, 0.125, splits,
                                                          scratch, extras=ops.attention_extras(q, None, gate, False, 0.0, bias))),
                 read)
            note(f"attention_decode_b64_{name}_splits{splits} (Llama)",
                 time_kernel(lambda: ops.attention_decode(q, kvp[0], kvp[1], table, pos, ent, res, page, window, 0.125, splits,
                                                          scratch)), read)
    # a 2,048-token prompt through the tiled kernels: the bias inside (mma.sync, the build with extras), the gate after
    # the plain kernel, and the Llama layer's tcgen05 kernel at the same shape (pages as the cache manager lays them out)
    tokens = 2048
    n_pages = tokens // page
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, n_pages)
    q = torch.randn((tokens, heads, hd), device=dev).to(bf)
    res = torch.empty_like(q)
    kvp = torch.randn((n_pages, 2, kv, page, hd), device=dev).to(bf)
    k_pool, v_pool = kvp[:, 0], kvp[:, 1]
    gate = torch.randn((tokens, heads), device=dev).to(bf)
    rows = ops.attention_prefill_tile_rows()
    tiles = torch.tensor([(r, min(rows, tokens - r), r, 0) for r in range(0, tokens, rows)], dtype=torch.int32, device=dev)
    note("sigmoid_gate_heads_T2048 (the gate of a layer without a bias, after its attention)",
         time_kernel(lambda: ops.sigmoid_gate_heads(res, gate)), tokens * heads * hd * 4)
    for window in (1024, None):
        flops = 4.0 * heads * hd * sum(min(p + 1, window or tokens) for p in range(tokens))
        name = f"w{window}" if window else "causal"
        for what, ex in (("bias", ops.attention_extras(q, None, None, False, 0.0, bias)),
                         ("bias, weights in two terms", ops.attention_extras(q, None, None, True, 0.0, bias)),
                         ("plain, mma.sync", None)):
            ms = time_kernel(lambda: ops.attention_prefill(q, k_pool, v_pool, table, tiles, res, page, window, 0.125, extras=ex))
            note(f"attention_prefill_T2048_{name} ({what})", ms, None, flops)
        if ops.attention_prefill_tcgen05_supports(q, k_pool, page):
            ms = time_kernel(lambda: ops.attention_prefill_tcgen05(q, k_pool, v_pool, table, tiles, res, page, window, 0.125,
                                                                   None, 1, None, False))
            note(f"attention_prefill_T2048_{name} (tcgen05: Llama, and the layers without a bias)", ms, None, flops)
            ms = time_kernel(lambda: ops.attention_prefill_tcgen05(q, k_pool, v_pool, table, tiles, res, page, window, 0.125,
                                                                   None, 1, None, False, distance_bias=bias))
            note(f"attention_prefill_T2048_{name} (tcgen05 with the bias)", ms, None, flops)
    return out


def run_design(args) -> dict:
    """Prefill and decode throughput of the named design at a few sizes beside the Llama
    decoder at the same width, depth and vocabulary (random weights), and the design's own
    kernels alone."""
    import gc

    import torch

    from pulsarlm_b200 import Engine
    from pulsarlm_b200.engine.runner import StepEntry

    pk = peaks()
    results: dict = {}
    prompt, batch, context = 2048, 8, 2048
    with ClockSampler() as clocks:
        for width, layers in ((1024, 6), (2048, 6), (4096, 3)):
            mine = {"bunosun": bunosun_config, "rerilorn": rerilorn_config, "simetar": simetar_config,
                    "puvirax": puvirax_config}[args.design](width, layers)
            for name, cfg in ((args.design, mine), ("llama", llama_config_like(width, layers))):
                vocab = cfg.get("vocab", cfg.get("vocab_size"))
                n_pages = (batch * (context + 256) + 4 * prompt) // PAGE_SIZE
                engine = Engine(cfg, dtype="bfloat16", device="cuda:0", n_pages=n_pages, page_size=PAGE_SIZE,
                                prefill_tokens_per_step=prompt, max_requests=batch + 2, seed=0)
                gen = torch.Generator().manual_seed(1)
                times = []
                for attempt in range(args.warmup + 3):
                    tokens = torch.randint(0, vocab, (prompt,), generator=gen).tolist()
                    torch.cuda.synchronize()
                    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record()
                    engine.runner.step([StepEntry(("p", attempt), tokens, [prompt - 1])])
                    end.record()
                    torch.cuda.synchronize()
                    engine.runner.end(("p", attempt))
                    if attempt >= args.warmup:
                        times.append(start.elapsed_time(end))
                prefill_ms = statistics.median(times)
                ids = fill_cache(engine, batch, context, name)
                decode_ms, launches = time_decode(engine, ids, args.steps, args.warmup, vocab)
                params = sum(int(t.numel()) for part in engine.model.parts() for t in vars(part).values()
                             if isinstance(t, torch.Tensor))
                results[f"{name}_w{width}_l{layers}"] = {
                    "parameters": params, "prefill_ms": prefill_ms, "prefill_tok_s": prompt / (prefill_ms / 1e3),
                    "decode_ms": decode_ms, "decode_tok_s": batch / (decode_ms / 1e3),
                    "decode_launches_per_step": launches // max(1, args.steps),
                    "graphs": bool(engine.cuda_graphs)}
                del engine
                gc.collect()
                torch.cuda.empty_cache()
        kernels = {"bunosun": bunosun_kernels, "rerilorn": design_kernels, "simetar": simetar_kernels,
                   "puvirax": puvirax_kernels}[args.design](2048, pk)
    summary = clocks.summary()
    return {"metric": f"prefill and decode tok/s of the {args.design.capitalize()} design beside the Llama decoder at "
                      f"equal sizes",
            "design": args.design, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "dtype": "bf16", "data": "synthetic: random weights drawn on the device, uniform random token ids",
            "config": {"prompt": prompt, "decode_batch": batch, "decode_context": context, "page_size": PAGE_SIZE,
                       "peaks": pk["source"], "l2": "kernels alone: a 256 MB buffer is rewritten between calls"},
            "models": results, "kernels": kernels,
            "clocks": {"sm_mhz": summary["sm_mhz"], "sm_max_mhz": summary["sm_max_mhz"], "reasons": summary["reasons"]}}


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--design", default="llama", choices=["llama", "rerilorn", "bunosun", "simetar", "puvirax"],
                   help="llama: the headline workload (the default); rerilorn, bunosun, simetar, puvirax: that design's prefill and "
                        "decode throughput at a few sizes beside the Llama decoder at equal sizes, and its kernels alone")
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=128)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--layers", type=int, default=32, help="fewer layers than the model's 32 (named in config)")
    p.add_argument("--prefill_tokens", type=int, default=PROMPT_LEN,
                   help="length of the prompt of the prefill phase (the contract's figure is the default's)")
    p.add_argument("--phases", default="prefill,e2e,decode,points,ctx4096,mixed_1b,serve_13b",
                   help="which measurements to run (a profiler run wants one): "
                        "prefill,e2e,decode,points,ctx4096,mixed_1b,serve_13b")
    args = p.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "cosmonomic/pulsarlm does not install offline here: its build needs hatchling, Python >= 3.13, "
                          "torch 2.15, xmake, CUDA 13.2 and gcc 15, none of which this image has"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    args.warmup = max(3, args.warmup)
    if args.design in ("rerilorn", "bunosun", "simetar", "puvirax"):
        args.steps = min(args.steps, 64)
        print(json.dumps(run_design(args)))
        return 0
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
