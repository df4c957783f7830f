"""Trace replay: feed given token ids through a model step by step and write the logits.

It samples nothing and has no model code of its own: it drives the engine's decoder, step function,
cache manager and kernels, the ones generation uses. The reference's counterparts are `logit-diff`
(crates/core/src/logitdiff.rs:16-93), `Runtime::prompt_logits` (crates/specrt/src/runtime.rs:2147),
the teacher-forced `prefill_then_decode` (crates/specrt/src/runtime.rs:2506-2517), the per-layer
trace of `trace_prefill` / `trace_decode` (crates/specrt/src/runtime.rs:2480-2504) and the logit
hashes of `logitdump` (crates/specrt/src/bin/logitdump.rs:20-49).

    trace_run --model DIR|SPEC.toml --dtype bfloat16|float32 --out DIR --max-tokens N [--trace-layers] [--hashes]

Standard input: one JSON object a line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` are the step's batch (each request's next tokens and the places whose logits are wanted),
`end` the requests that are finished after the step. For a step that wants something the logits are
written to OUT/<step>.f32 as little-endian float32 [wanted, vocab]; after every step a line
`done <step>` is printed and flushed.

--trace-layers also writes OUT/<step>.layers.f32, float32 [1 + schedule entries, wanted, hidden]: the
residual stream at the wanted places after the embedding and after every entry of the layer schedule,
so that a wrong logit can be followed back to the first layer that differs. --hashes appends
"<step> <hash of the step's logits>" to OUT/hashes.txt (64-bit FNV-1a over the float bit patterns, the
reference's logitdump hash): two runs can then be compared without keeping the logits.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PAGE_SIZE = 16
MAX_LIVE = 8


def build_runner(model, dtype: str, max_tokens: int, page_size: int = PAGE_SIZE, max_requests: int = MAX_LIVE, device: str = "cuda:0", options=None):
    """`model`: a folder, a hub id or a TOML model spec; `options`: runtime options laid over the spec's own."""
    from .cache.manager import CacheManager
    from .config.spec import resolve_model
    from .engine.model import load_model
    from .engine.runtime import Runtime
    from .engine.step import ModelRunner

    spec = resolve_model(model)
    opts = spec.runtime.merged(options or {}, "trace_run options").merged(dtype=dtype, page_size=page_size)
    rt = Runtime(device, options=opts)
    _, decoder = load_model(spec, rt)
    num_pages = max(1, -(-max_tokens // page_size))
    cache = CacheManager(decoder.cache_needs(), page_size, num_pages, max_requests, max(max_tokens, page_size), device=rt.device,
                         dtype=rt.act_dtype, sources=decoder.cache_sources())
    return ModelRunner(decoder, cache, rt)


def logit_hash(values) -> int:
    """64-bit FNV-1a over the bit patterns of float32 values, one word at a time (crates/specrt/src/bin/logitdump.rs:20-22)."""
    import numpy as np
    h = 0xcbf29ce484222325
    for w in np.ascontiguousarray(values, dtype="<f4").view("<u4").ravel().tolist():
        h = ((h ^ w) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return h


def replay(runner, lines, out_dir: Path, say=print, trace_layers: bool = False, hashes: bool = False) -> None:
    import torch

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
        layers = [] if trace_layers else None
        logits = runner.step(entries, trace=layers)
        if logits is not None:
            host = logits.detach().to("cpu").numpy().astype("<f4")
            host.tofile(out_dir / f"{step}.f32")
            if layers:
                torch.stack(layers).to("cpu").numpy().astype("<f4").tofile(out_dir / f"{step}.layers.f32")
            if hashes:
                with open(out_dir / "hashes.txt", "a") as fh:
                    fh.write(f"{step} {logit_hash(host):016x}\n")
        for rid in rec.get("end", []):
            if runner.cache.has(rid):
                runner.cache.release(rid)
        say(f"done {step}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="Replay a token trace through the engine and write logits.")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors, or a TOML model spec")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"], help="bfloat16: the kernels serving uses; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--trace-layers", action="store_true", help="also write <step>.layers.f32: the residual stream at the wanted places after every layer")
    ap.add_argument("--hashes", action="store_true", help="append a hash of every step's logits to OUT/hashes.txt")
    args = ap.parse_args(argv)
    runner = build_runner(args.model, args.dtype, args.max_tokens, args.page_size, device=args.device)

    def say(msg):
        sys.stdout.write(msg + "\n")
        sys.stdout.flush()

    replay(runner, sys.stdin, Path(args.out), say, args.trace_layers, args.hashes)
    return 0


if __name__ == "__main__":
    sys.exit(main())
