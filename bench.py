#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B shape with random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests whose contexts start at 2,048 tokens (the
context length of the benchmark is 4,096). `value` is decoded tokens per second with the steps
enqueued back to back (sampled tokens fed back on the device) and timed with CUDA events; `e2e` is the
same through the Python entry point (`Engine.submit` / `Engine.step`), every step taking its inputs
from pinned host memory and handing its tokens back to the host. One JSON line is printed.
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

# Qwen3-8B layer sizes: the third configuration the baseline names.
QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096, intermediate_size=12288,
    num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
    tie_word_embeddings=False, max_position_embeddings=40960, hidden_act="silu", attention_bias=False, torch_dtype="bfloat16")
# The two larger shapes the baseline names (same architecture; --shape 14b / 32b): not the default run.
SHAPES = {
    "8b": QWEN3_8B,
    "14b": dict(QWEN3_8B, hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40),
    "32b": dict(QWEN3_8B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64),
    # the one size the reference published numbers for (on other hardware)
    "0.6b": dict(QWEN3_8B, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16, tie_word_embeddings=True),
}
CONTEXT = 4096          # benchmark context length
PROMPT = 2048           # prefill length, and the context each decode request starts from
PAGE = 16           # keys per cache page of the benchmark configuration
PAGE_ENGINE = 64    # the engine's own default (one TMA box of 64 rows per page, plane and half head): measured too, as extra points
SETTLE_MS = 250     # idle time between building the requests' contexts (prefill at full power) and a decode measurement's warm-up steps:
                    # the power limiter's clock reduction after the prefill would otherwise be charged to the decode steps
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows: list[list[str]] = []      # each with the time it arrived at
        self.proc = None
        self.begin = self.end = None         # the timed region, by time.perf_counter()

    def mark_begin(self):
        self.begin = time.perf_counter()

    def mark_end(self):
        self.end = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")] + [time.perf_counter()])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for r in self.rows if len(r) >= 8]
        if self.begin is not None:   # the samples of the timed region; if it was too short to catch one, the first ones after its start
            inside = [r for r in rows if self.begin <= r[-1] <= (self.end or float("inf")) + 0.03]
            rows = inside or [r for r in rows if r[-1] >= self.begin][:3]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        num = lambda s: float(s) if s.replace(".", "", 1).isdigit() else None
        sm = [num(r[0]) for r in rows if num(r[0]) is not None]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": num(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def weight_bytes(cfg: dict, layers: int) -> int:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * H + H * q + 2 * I * H + H * I
    return 2 * (layers * per_layer + V * H)      # bfloat16; the lm_head is read once per step, the embedding rows are negligible


def kv_bytes_per_token(cfg: dict, layers: int) -> int:
    return 2 * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * layers


def prefill_flops(cfg: dict, layers: int, T: int) -> float:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = 2.0 * T * layers * ((q + 2 * kv) * H + H * q + 2 * I * H + H * I)
    attention = layers * 4.0 * (T * (T + 1) / 2) * q     # QK^T and PV over the causal half
    return linear + attention + 2.0 * V * H


def _prompt(seed: int, n: int, vocab: int) -> list[int]:
    import numpy as np
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def measure_prefill(engine, steps: int, warmup: int, after: int = 0) -> float:
    """Milliseconds for one step that prefills a PROMPT-token prompt portion and returns its last logits; with
    `after`, the portion follows that many tokens of the same request already in the cache (not timed)."""
    import torch
    from inference_bench_b200.engine.step import StepEntry
    vocab = engine.decoder.plan.vocab_size
    times = []
    for i in range(warmup + steps):
        rid = ("prefill", i)
        toks = _prompt(1000 + i, PROMPT, vocab)
        engine.cache.admit(rid)
        for a in range(0, after, PROMPT):
            engine.runner.step([StepEntry(rid, _prompt(2000 + i + a, min(PROMPT, after - a), vocab), [])], check=False)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.runner.step([StepEntry(rid, toks, [PROMPT - 1])], check=False)
        e1.record()
        torch.cuda.synchronize()
        engine.cache.release(rid)
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    engine.rt.check_status()
    return statistics.median(times)


def measure_decode_device(engine, batch: int, steps: int, warmup: int, clocks=None, start: int = PROMPT) -> tuple[float, int]:
    """Milliseconds per decode step of `batch` requests whose contexts start at PROMPT tokens, steps
    enqueued back to back with tokens fed back on the device; and kernel launches per step."""
    import torch
    from inference_bench_b200.engine.executor import RUN_AHEAD_MAX
    from inference_bench_b200.engine.step import StepEntry
    from inference_bench_b200.sampling.params import GREEDY
    vocab = engine.decoder.plan.vocab_size
    ids = [("decode", batch, i) for i in range(batch)]
    last = []
    for i, rid in enumerate(ids):
        engine.cache.admit(rid)
        toks = _prompt(2000 + i, start, vocab)
        for a in range(0, start, PROMPT):   # the context, in portions of the benchmark's prefill length
            part = toks[a:a + PROMPT]
            logits = engine.runner.step([StepEntry(rid, part, [len(part) - 1] if a + PROMPT >= start else [])], check=False)
        last.append(int(engine.executor.sampler.sample(logits, [GREEDY], [0]).item()))
    generated = 1
    torch.cuda.synchronize()
    time.sleep(SETTLE_MS / 1e3)

    def run(n):
        nonlocal last, generated
        done = 0
        while done < n:
            k = min(RUN_AHEAD_MAX, n - done)
            entries = [StepEntry(rid, [tok], [0]) for rid, tok in zip(ids, last)]
            hist = engine.executor.decode_ahead(entries, [(GREEDY, generated)] * batch, k)
            last = hist[-1]
            generated += k
            done += k

    run(max(warmup, 1))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.mark_begin()
    e0.record()
    run(steps)
    e1.record()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.mark_end()
    ms = e0.elapsed_time(e1) / steps
    launches = engine.executor.graph_for(batch).launches
    for rid in ids:
        engine.cache.release(rid)
    engine.rt.check_status()
    return ms, launches


LEAVE_OUT = {   # kinds of kernel by the library entry points that launch them
    "attention": ["ib_attention_decode", "ib_attention_decode_stream", "ib_attention_decode_fused", "ib_attention_prefill_ws", "ib_attention_prefill_tc"],
    "head": ["ib_embed", "ib_sample_rows"],
    "qkv": ["ib_gemm_qkv_tcgen05_2cta"],
    "norm": ["ib_add_rmsnorm"], "silu_mul": ["ib_silu_mul"], "qk": ["ib_qk_norm_rope_kv"], "sampling": ["ib_sample_rows"],
    "gemm": ["ib_gemm_tcgen05", "ib_gemm_swiglu_tcgen05", "ib_gemm_swiglu_tcgen05_2cta", "ib_gemm_tcgen05_2cta", "ib_gemm_tcgen05_2cta_add"],
    "small": ["ib_add_rmsnorm", "ib_silu_mul", "ib_qk_norm_rope_kv", "ib_rope_table", "ib_sample_rows", "ib_embed"],
}


def leave_out_costs(engine, batch: int, steps: int, warmup: int, kinds: str) -> dict:
    """Milliseconds per decode step with one kind of kernel left out of the captured step at a time (the results of such a
    step are void; only its time means something). The difference from the whole step is what that kind costs inside
    the graph, where kernels overlap their neighbours' tails: the figure a launch list cannot give."""
    from inference_bench_b200.kernels import lib as L
    real, out = L.call, {}
    try:
        for kind in kinds.split(","):
            names = set(sum((LEAVE_OUT[k] for k in kind.split("+")), []))
            L.call = lambda name, *a, _n=names: None if name in _n else real(name, *a)
            engine.executor._graphs.clear()
            out[kind] = measure_decode_device(engine, batch, steps, warmup)[0]
    finally:
        L.call = real
        engine.executor._graphs.clear()
    return out


def measure_mixed_step(engine, steps: int, cfg: dict, layers: int) -> tuple[float, int, float, float]:
    """Milliseconds for one step that holds 8 prompt portions of 512 tokens (starting 0, 512, ... 3,584 tokens into
    their prompts) beside 56 decoded tokens of requests at contexts drawn uniformly from 1,024 to 4,096: the
    mixed batch the baseline names for the 14B shape. Returns (median ms, rows in the step, the step's FLOPs, the
    bytes it has to read: every weight once and the cache of the live requests)."""
    import numpy as np
    import torch
    from inference_bench_b200.engine.step import StepEntry
    vocab = engine.decoder.plan.vocab_size
    rng = np.random.default_rng(0)
    contexts = rng.integers(1024, CONTEXT + 1, 56).tolist()

    def fill(rid, n):   # bring a request to n tokens in the cache
        engine.cache.admit(rid)
        toks = _prompt(abs(hash(rid)) % 1000, n, vocab)
        for a in range(0, n, PROMPT):
            engine.runner.step([StepEntry(rid, toks[a:a + PROMPT], [])], check=False)

    for i, c in enumerate(contexts):
        fill(("mixed-d", i), c - 1)
    for i in range(8):
        fill(("mixed-p", i), 512 * i)
    entries = [StepEntry(("mixed-d", i), [int(rng.integers(0, vocab))], [0]) for i in range(56)]
    entries += [StepEntry(("mixed-p", i), _prompt(50 + i, 512, vocab), [511]) for i in range(8)]
    times = []
    for _ in range(steps + 2):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.runner.step(entries, check=False)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        for e in entries:   # the same work again: forget the step's tokens
            engine.cache.commit(e.request, engine.cache.length(e.request) - len(e.tokens))
    for e in entries:
        engine.cache.release(e.request)
    engine.rt.check_status()
    rows = sum(len(e.tokens) for e in entries)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    keys_seen = sum(contexts) + sum(512 * (512 * i) + 512 * 513 // 2 for i in range(8))       # (query, key) pairs of the step
    flops = 2.0 * rows * layers * ((q + 2 * kv) * H + H * q + 3 * I * H) + layers * 4.0 * keys_seen * q + 2.0 * 64 * V * H
    cached = sum(contexts) + sum(512 * (i + 1) for i in range(8))
    return statistics.median(times[2:]), rows, flops, weight_bytes(cfg, layers) + cached * kv_bytes_per_token(cfg, layers)


def measure_decode_e2e(engine, batch: int, steps: int, warmup: int) -> tuple[float, float, float]:
    """Milliseconds per decode step through Engine.submit / Engine.step: host token ids in (pinned
    staging, copied every step) and sampled token ids back on the host every step."""
    import torch
    vocab = engine.decoder.plan.vocab_size
    for i in range(batch):
        engine.submit(_prompt(3000 + i, PROMPT, vocab), max_tokens=warmup + steps + 8)
    while engine.scheduler.waiting or any(not s.decoding for s in engine.scheduler.running):
        engine.step()
    torch.cuda.synchronize()
    time.sleep(SETTLE_MS / 1e3)
    for _ in range(max(warmup, 1)):
        engine.step()
    ex = engine.executor
    h0, d0 = ex.h2d_bytes, ex.d2h_bytes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    emitted = 0
    for _ in range(steps):
        emitted += len(engine.step().emitted)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    assert emitted == batch * steps, f"{emitted} tokens emitted in {steps} steps of {batch} requests"
    h2d, d2h = (ex.h2d_bytes - h0) / steps, (ex.d2h_bytes - d0) / steps
    for s in list(engine.scheduler.running):
        engine.cancel(s.req.id)
    engine.rt.check_status()
    return (t1 - t0) * 1e3 / steps, h2d, d2h


def make_engine(cfg: dict, page: int, big: int, ctx: int = CONTEXT):
    from inference_bench_b200 import Engine
    return Engine(cfg, dtype="bfloat16", max_ctx=ctx, page_size=page, num_pages=big * (ctx // page) + 64, max_num_seqs=big,
                  max_batched_tokens=8192, prefill_chunk=PROMPT, random_weights_seed=0)


def run_ours(args) -> dict:
    import gc

    import torch
    pk, pk_src = peaks()
    cfg = dict(SHAPES[args.shape])
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers = args.layers or full_layers
    big = max(args.batch, 64)
    page = args.page_size
    start = args.context_start
    after = args.prefill_after if args.only == "prefill" else 0
    if after:   # a portion deep in a long context: a cache for one such request
        engine = make_engine(cfg, page, 1, after + PROMPT)
    elif args.only == "decode" and start != PROMPT:   # another context length: a cache for just these requests
        engine = make_engine(cfg, page, max(args.batch, 8), start + CONTEXT - PROMPT)
    else:
        engine = make_engine(cfg, page, big)
    steps, warmup = args.steps, max(args.warmup, 3)
    if args.only == "prefill":   # one part alone, for profiling: a short report, not the benchmark line
        warm = 1 if after else 2
        report = {"only": "prefill", "layers": layers, "page_size": page, **({"after": after} if after else {}),
                  "ms": measure_prefill(engine, args.steps, warm, after)}
        if args.leave_out:
            from inference_bench_b200.kernels import lib as L
            real, report["without"] = L.call, {}
            try:
                for kind in args.leave_out.split(","):
                    names = set(sum((LEAVE_OUT[k] for k in kind.split("+")), []))
                    L.call = lambda name, *a, _n=names: None if name in _n else real(name, *a)
                    report["without"][kind] = measure_prefill(engine, args.steps, warm, after)
            finally:
                L.call = real
        return report
    if args.only == "mixed":
        clocks = ClockSampler()
        clocks.start()
        ms, rows, flops, step_bytes = measure_mixed_step(engine, max(args.steps, 3) if args.steps < 16 else 5, cfg, layers)
        return {"only": "mixed", "shape": args.shape, "layers": layers, "layers_full": full_layers, "page_size": page, "rows": rows, "ms": ms,
                "tok_s": rows * 1e3 / ms, "prefill": {"tokens": 8 * 512, "frac": flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), "peak_tflops": pk["bf16_tflops"]},
                "roofline": {"bound": "hbm", "achieved": step_bytes / (ms * 1e-3) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]}, "peaks": pk_src, "clocks": clocks.stop()}
    if args.only == "decode":
        ms, launches = measure_decode_device(engine, args.batch, steps, warmup, start=start)
        step_bytes = weight_bytes(cfg, layers) + args.batch * (start + 1 + warmup + steps / 2) * kv_bytes_per_token(cfg, layers)
        report = {"only": "decode", "shape": args.shape, "layers": layers, "batch": args.batch, "context_start": start, "page_size": page, "ms_per_step": ms,
                  "tok_s": args.batch * 1e3 / ms, "launches_per_step": launches, "hbm_frac": step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]}
        if args.leave_out:
            report["without"] = leave_out_costs(engine, args.batch, steps, warmup, args.leave_out)
        return report

    # the headline first (device-timed, then through the entry point), then the other points
    clocks = ClockSampler()
    clocks.start()      # nvidia-smi takes a while to start reporting: it runs from here on, and the samples of the timed region are kept
    ms, launches = measure_decode_device(engine, args.batch, steps, warmup, clocks)
    clock_report = clocks.stop()
    e2e_ms, h2d, d2h = measure_decode_e2e(engine, args.batch, steps, warmup)
    b1_ms, _ = measure_decode_device(engine, 1, steps, warmup)
    b64_ms, _ = measure_decode_device(engine, 64, min(steps, 64), warmup)
    prefill_ms = measure_prefill(engine, 5, 3)
    extra = {}
    if page != PAGE_ENGINE:   # the same measurements at the engine's default page size
        del engine
        gc.collect()   # the engine's parts refer to one another: without this its weights outlive the name
        torch.cuda.empty_cache()
        engine = make_engine(cfg, PAGE_ENGINE, big)
        tag = f"_page{PAGE_ENGINE}"
        extra["prefill" + tag] = PROMPT * 1e3 / measure_prefill(engine, 5, 3)
        extra["decode_b1" + tag] = 1e3 / measure_decode_device(engine, 1, steps, warmup)[0]
        extra["decode_b64" + tag] = 64e3 / measure_decode_device(engine, 64, min(steps, 64), warmup)[0]
        extra[f"decode_b{args.batch}" + tag] = args.batch * 1e3 / measure_decode_device(engine, args.batch, steps, warmup)[0]

    B = args.batch
    avg_ctx = PROMPT + 1 + warmup + steps / 2
    step_bytes = weight_bytes(cfg, layers) + B * avg_ctx * kv_bytes_per_token(cfg, layers)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = prefill_flops(cfg, layers, PROMPT)
    return {
        "metric": f"decode tok/s at batch {B} (Qwen3-{args.shape.upper()} shape, random bf16 weights, context 2048 growing toward 4096)",
        "value": B * 1e3 / ms, "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": layers, "layers_full": full_layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "global_batch": B, "seq_len": CONTEXT, "decode_context_start": PROMPT, "prefill_tokens": PROMPT,
                   "page_size": page, "weights": "random N(0,0.02) bf16 seed 0", "parallelism": "single_gpu",
                   "l2": "inputs larger than L2 (weights read every step)", "peaks": pk_src, "settle_ms": SETTLE_MS},
        "e2e": {"value": B * 1e3 / e2e_ms, "unit": "tok/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * steps,
        "prefill": {"value": PROMPT * 1e3 / prefill_ms, "tokens": PROMPT, "ms": prefill_ms, "frac": flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]},
        "points": {"decode_b1": 1e3 / b1_ms, "decode_b64": 64e3 / b64_ms, **extra},
        "clocks": clock_report,
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: the benchmark's Qwen3-8B, or the larger shapes the baseline names")
    ap.add_argument("--page-size", type=int, default=PAGE, help="keys per cache page (the benchmark configuration names 16)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (both numbers are reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prefill-after", type=int, default=0, help="with --only prefill: the 2,048-token portion follows this many cached tokens of the same request")
    ap.add_argument("--context-start", type=int, default=PROMPT, help="with --only decode: the context each request starts from (default: the benchmark's 2,048)")
    ap.add_argument("--leave-out", default="", help="with --only decode or prefill: also time the step without each of these kinds of kernel (comma separated; "
                    "a+b leaves both out): " + ", ".join(sorted(LEAVE_OUT)))
    ap.add_argument("--only", default="", choices=["", "prefill", "decode", "mixed"], help="run one part alone (for profiling); prints a short report")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust workspace (no setup.py/pyproject.toml): pip cannot install it and no Rust toolchain is present"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    if args.steps + max(args.warmup, 3) + 8 > CONTEXT - PROMPT:
        print(f"--steps + --warmup must stay below {CONTEXT - PROMPT - 8}: contexts start at {PROMPT} and end at {CONTEXT}")
        return 2
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
