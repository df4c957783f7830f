"""Command line of the engine, in the manner of the reference's `inference-bench` tool
(crates/cli/src/main.rs:87-104, 190-222): the same command names and option names where it has them.

    python -m inference_bench_b200 run        --model DIR [--prompt TEXT | --prompt-file F | --prompt-len N] [--max-tokens 64] [--json] [--max-ctx N]
    python -m inference_bench_b200 batch      --model DIR [--prompt-len 128] [--max-tokens 128] [--sizes 1,4,16] [--json]
    python -m inference_bench_b200 logit-diff --model DIR --reference NAME.ref.json [--quantised]
    python -m inference_bench_b200 spec       --model DIR|SPEC.toml
    python -m inference_bench_b200 random-model --config CONFIG.json --seed N --out DIR

Added here: --temperature, --seed, --top-k, --top-p, --min-p, --dtype bfloat16|float32, --runtime NAME=VALUE, --random-weights SEED
(weights made on the device: --model is then a config.json), and the random-model command.
Prompts are token ids unless the model folder has a tokenizer.json; --prompt-len makes a synthetic
prompt of that many token ids, 1000 + (i*7) % 5000 clipped to the vocabulary, like the reference's
bench tool (crates/specrt/src/bin/bench.rs:320-343).
"""
from __future__ import annotations

import argparse
import json
import statistics
import struct
import sys
import time
from pathlib import Path


def _synthetic_prompt(n: int, vocab: int, seed: int = 0) -> list[int]:
    return [(1000 + (i * 7 + seed * 131) % 5000) % vocab for i in range(n)]


def _read_prompt(args, engine) -> list[int]:
    vocab = engine.decoder.plan.vocab_size
    if args.prompt_file:
        text = Path(args.prompt_file).read_text()
        try:
            ids = json.loads(text)
            if isinstance(ids, list) and all(isinstance(t, int) for t in ids):
                return ids
        except json.JSONDecodeError:
            pass
        return engine.tokens(text)
    if args.prompt is not None:
        return engine.tokens(args.prompt)
    return _synthetic_prompt(args.prompt_len or 128, vocab)


def _runtime_overrides(args) -> dict:
    """--runtime name=value pairs, typed like a TOML value (true/false, integers, numbers, strings)."""
    out = {}
    for item in getattr(args, "runtime", None) or []:
        name, eq, text = item.partition("=")
        if not eq:
            raise SystemExit(f"--runtime takes name=value, got {item!r}")
        low = text.strip().lower()
        if low in ("true", "false"):
            value = low == "true"
        else:
            try:
                value = int(text)
            except ValueError:
                try:
                    value = float(text)
                except ValueError:
                    value = text.strip().strip('"')
        out[name.strip()] = value
    return out


def _engine(args, **kw):
    from .engine.engine import Engine
    model = args.model
    seed = getattr(args, "random_weights", None)
    if seed is not None:   # weights made on the device from a seed: --model is then a config.json (or a folder that has one)
        path = Path(model)
        model = json.loads((path / "config.json" if path.is_dir() else path).read_text())
    return Engine(model, dtype=args.dtype, max_ctx=args.max_ctx, options=_runtime_overrides(args) or None, random_weights_seed=seed, **kw)


def _sampling(args):
    from .sampling.params import SamplingParams
    return SamplingParams(temperature=args.temperature, seed=args.seed, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p)


def cmd_run(args) -> int:
    engine = _engine(args, max_num_seqs=1)
    prompt = _read_prompt(args, engine)
    t0 = time.perf_counter()
    reply = engine.generate(prompt, max_tokens=args.max_tokens, sampling=_sampling(args))
    wall = time.perf_counter() - t0
    result = {
        "model": str(args.model), "prompt_tokens": reply.prompt_tokens, "completion_tokens": reply.completion_tokens, "finish": reply.finish,
        "ttft_secs": reply.prefill_secs, "prefill_secs": reply.prefill_secs, "decode_secs": reply.decode_secs, "wall_secs": wall,
        "prefill_tok_s": reply.prompt_tokens / reply.prefill_secs if reply.prefill_secs > 0 else None,
        "decode_tok_s": (reply.completion_tokens - 1) / reply.decode_secs if reply.decode_secs > 0 and reply.completion_tokens > 1 else None,
        "peak_device_bytes": reply.peak_device_bytes, "tokens": reply.tokens,
    }
    if engine.model_dir and (engine.model_dir / "tokenizer.json").is_file():
        try:
            result["text"] = engine.text(reply.tokens)
        except RuntimeError:
            pass
    if args.json:
        print(json.dumps(result, indent=2))
    else:
        print(result.get("text", " ".join(map(str, reply.tokens))))
        print(f"{reply.prompt_tokens} prompt tokens in {reply.prefill_secs:.3f} s, {reply.completion_tokens} new tokens"
              + (f" at {result['decode_tok_s']:.1f} tok/s" if result["decode_tok_s"] else ""), file=sys.stderr)
    return 0


def cmd_batch(args) -> int:
    sizes = [int(s) for s in args.sizes.split(",") if s]
    engine = _engine(args, max_num_seqs=max(sizes))
    vocab = engine.decoder.plan.vocab_size
    results = []
    for n in sizes:
        prompts = [_synthetic_prompt(args.prompt_len, vocab, seed=i) for i in range(n)]
        engine.generate(prompts, max_tokens=3)    # untimed: captures this batch size's decode graph and warms the kernels' one-time set-up
        t0 = time.perf_counter()
        replies = engine.generate(prompts, max_tokens=args.max_tokens, sampling=_sampling(args))
        wall = time.perf_counter() - t0
        completion = sum(r.completion_tokens for r in replies)
        # aggregate decode tok/s = sum over requests of (tokens after the first) / (its decode time), crates/core/src/batch.rs:52-57
        decode = sum((r.completion_tokens - 1) / r.decode_secs for r in replies if r.decode_secs > 0 and r.completion_tokens > 1)
        results.append({"model": str(args.model), "batch": n, "prompt_tokens": sum(r.prompt_tokens for r in replies), "completion_tokens": completion,
                        "wall_secs": wall, "throughput_tok_s": completion / wall, "decode_tok_s": decode,
                        "median_ttft_secs": statistics.median_high([r.prefill_secs for r in replies])})
    if args.json:
        print(json.dumps(results, indent=2))
    else:
        for r in results:
            print(f"batch {r['batch']:4d}: decode {r['decode_tok_s']:10.1f} tok/s  throughput {r['throughput_tok_s']:10.1f} tok/s  median ttft {r['median_ttft_secs'] * 1e3:8.1f} ms")
    return 0


def cmd_logit_diff(args) -> int:
    """Compare the engine's logits at every prompt position with a reference file pair:
    NAME.ref.json {tokens, vocab, ...} and NAME.ref.bin, raw little-endian float32 [tokens, vocab]
    (crates/core/src/logitdiff.rs:76-93). Exit code 2 outside the tolerance."""
    import numpy as np
    meta = json.loads(Path(args.reference).read_text())
    tokens, vocab = meta["tokens"], meta["vocab"]
    ref = np.fromfile(str(args.reference).replace(".ref.json", ".ref.bin"), dtype="<f4").reshape(len(tokens), vocab)
    engine = _engine(args, max_num_seqs=1)
    ours = engine.logits(tokens).numpy()
    if ours.shape != ref.shape:
        print(f"logit shapes differ: {ours.shape} against {ref.shape}", file=sys.stderr)
        return 1
    diff = np.abs(ours - ref)
    report = {"max_abs": float(diff.max()), "mean_abs": float(diff.mean()), "top1_agreement": float((ours.argmax(1) == ref.argmax(1)).mean()),
              "positions": len(tokens), "vocab": vocab}
    # crates/core/src/logitdiff.rs:23-26
    tol = {"max_abs": float("inf"), "mean_abs": 0.1, "top1": 0.95} if args.quantised else {"max_abs": 1e-3, "mean_abs": 1e-4, "top1": 1.0}
    ok = report["max_abs"] <= tol["max_abs"] and report["mean_abs"] <= tol["mean_abs"] and report["top1_agreement"] >= tol["top1"]
    report["within_tolerance"] = ok
    print(json.dumps(report, indent=2))
    return 0 if ok else 2


def cmd_spec(args) -> int:
    """The typed configuration the model resolves to, what the plan derives from it and the runtime options it would
    run with. Works for every registered architecture: derived sizes are whatever integer properties its
    configuration class offers."""
    from .config.spec import resolve_model
    from .engine.model import plan_from_config
    from .registry import resolve
    spec = resolve_model(args.model)
    cfg, plan = plan_from_config(spec.raw_config)
    out = resolve(spec.raw_config).config_to_dict(cfg)
    derived = {}
    for name in dir(type(cfg)):
        if isinstance(getattr(type(cfg), name, None), property):
            value = getattr(cfg, name)
            if isinstance(value, (int, float, str, bool)):
                derived[name] = value
    derived.update(layers=len(plan.layers), schedule=[e.layer for e in plan.schedule],
                   cache_of=[e.cache_of for e in plan.schedule] if any(e.cache_of is not None for e in plan.schedule) else None)
    out["derived"] = {k: v for k, v in derived.items() if v is not None}
    out["name"] = spec.name
    out["weights"] = str(spec.model_dir) if spec.model_dir else None
    out["tensors"] = dict(spec.tensors)
    out["runtime"] = spec.runtime.merged(_runtime_overrides(args), "--runtime").to_dict()
    print(json.dumps(out, indent=2))
    return 0


def cmd_random_model(args) -> int:
    from .weights.random_init import write_random_model
    out = write_random_model(json.loads(Path(args.config).read_text()), args.seed, args.out)
    print(out)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="inference_bench_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p, prompt=True):
        p.add_argument("--model", required=True, help="folder with config.json and model.safetensors, a hub id in the hub cache, or a TOML model spec")
        p.add_argument("--runtime", action="append", metavar="NAME=VALUE", help="a runtime option laid over the model spec's [runtime] table (may be repeated)")
        p.add_argument("--random-weights", type=int, default=None, metavar="SEED", help="make random weights on the device from this seed; --model is then a config.json")
        p.add_argument("--max-ctx", type=int, default=None, help="context limit (default 2048, capped by max_position_embeddings)")
        p.add_argument("--dtype", default=None, choices=["bfloat16", "float32"], help="default: the model spec's [runtime] dtype, else bfloat16")
        if prompt:
            p.add_argument("--max-tokens", type=int, default=64)
            p.add_argument("--temperature", type=float, default=0.0)
            p.add_argument("--seed", type=int, default=0)
            p.add_argument("--top-k", type=int, default=0)
            p.add_argument("--top-p", type=float, default=1.0)
            p.add_argument("--min-p", type=float, default=0.0)
            p.add_argument("--json", action="store_true")

    p = sub.add_parser("run", help="generate from one prompt")
    common(p)
    g = p.add_mutually_exclusive_group()
    g.add_argument("--prompt")
    g.add_argument("--prompt-file")
    g.add_argument("--prompt-len", type=int)
    p.add_argument("--no-save", action="store_true", help="accepted for compatibility; results are never stored")
    p.set_defaults(fn=cmd_run)

    p = sub.add_parser("batch", help="N concurrent requests: aggregate decode tok/s, throughput, median time to first token")
    common(p)
    p.add_argument("--prompt-len", type=int, default=128)
    p.add_argument("--sizes", default="1,4,16")
    p.set_defaults(fn=cmd_batch, max_tokens=128)

    p = sub.add_parser("logit-diff", help="compare prompt logits with a reference file")
    common(p, prompt=False)
    p.add_argument("--reference", required=True)
    p.add_argument("--quantised", action="store_true")
    p.set_defaults(fn=cmd_logit_diff)

    p = sub.add_parser("spec", help="print the typed configuration and runtime options of a model folder or model spec")
    p.add_argument("--model", required=True)
    p.add_argument("--runtime", action="append", metavar="NAME=VALUE")
    p.set_defaults(fn=cmd_spec)

    p = sub.add_parser("random-model", help="write a model folder with random weights")
    p.add_argument("--config", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--out", required=True)
    p.set_defaults(fn=cmd_random_model)

    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
