"""Trace replay: feed given token ids through a model step by step and write the logits.

It samples nothing and has no model code of its own: it drives the engine's decoder, step function,
cache manager and kernels, the ones generation uses. The reference's counterparts are `logit-diff`
(crates/core/src/logitdiff.rs:16-93), `Runtime::prompt_logits` (crates/specrt/src/runtime.rs:2147)
and the teacher-forced `prefill_then_decode` (crates/specrt/src/runtime.rs:2506-2517).

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input: one JSON object a line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` are the step's batch (each request's next tokens and the places whose logits are wanted),
`end` the requests that are finished after the step. For a step that wants something the logits are
written to OUT/<step>.f32 as little-endian float32 [wanted, vocab]; after every step a line
`done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PAGE_SIZE = 16
MAX_LIVE = 8


def build_runner(model_dir, dtype: str, max_tokens: int, page_size: int = PAGE_SIZE, max_requests: int = MAX_LIVE, device: str = "cuda:0"):
    from .cache.manager import CacheManager
    from .engine.model import load_model
    from .engine.runtime import Runtime
    from .engine.step import ModelRunner

    rt = Runtime(device, dtype)
    _, decoder = load_model(model_dir, rt)
    num_pages = max(1, -(-max_tokens // page_size))
    cache = CacheManager(decoder.cache_needs(), page_size, num_pages, max_requests, max(max_tokens, page_size), device=rt.device,
                         dtype=rt.act_dtype, sources=decoder.cache_sources())
    return ModelRunner(decoder, cache, rt)


def replay(runner, lines, out_dir: Path, say=print) -> None:
    from .engine.step import StepEntry

    out_dir.mkdir(parents=True, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            if not runner.cache.has(e["id"]):
                runner.cache.admit(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        logits = runner.step(entries)
        if logits is not None:
            logits.detach().to("cpu").numpy().astype("<f4").tofile(out_dir / f"{step}.f32")
        for rid in rec.get("end", []):
            if runner.cache.has(rid):
                runner.cache.release(rid)
        say(f"done {step}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="Replay a token trace through the engine and write logits.")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"], help="bfloat16: the kernels serving uses; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    runner = build_runner(args.model, args.dtype, args.max_tokens, args.page_size, device=args.device)

    def say(msg):
        sys.stdout.write(msg + "\n")
        sys.stdout.flush()

    replay(runner, sys.stdin, Path(args.out), say)
    return 0


if __name__ == "__main__":
    sys.exit(main())
