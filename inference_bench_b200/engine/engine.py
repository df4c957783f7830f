"""The Python entry point: load a model, generate from token ids, read logits.

Names and meanings follow the reference's `Engine` (crates/specrt/src/engine.rs:436-603):
`Engine.load(model, max_ctx)`, `generate(prompt, max_tokens, sampling)`, `logits(prompt)`, and a
`Reply` with prompt_tokens, completion_tokens, prefill_secs, decode_secs and peak_device_bytes
(engine.rs:178-186). Prompts are token ids; text goes through `tokens()` when the model folder has
a tokenizer.json and the `tokenizers` package is importable.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Hashable, Mapping, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager
from ..config.runtime_options import RuntimeOptions
from ..config.spec import ModelSpec, resolve_model
from ..sampling.params import GREEDY, SamplingParams
from .executor import GpuExecutor
from .model import load_model, random_model
from .runtime import Runtime
from .scheduler import Finished, Request, Scheduler, SchedulerConfig
from .step import ModelRunner, StepEntry

DEFAULT_MAX_CTX = 2048   # crates/specrt/src/engine.rs:10


@dataclass
class Reply:
    tokens: list[int]
    finish: str
    prompt_tokens: int
    completion_tokens: int
    prefill_secs: float = 0.0
    decode_secs: float = 0.0
    peak_device_bytes: int = 0
    text: Optional[str] = None


class Engine:
    def __init__(self, model: Union[str, Path, Mapping[str, Any], ModelSpec], dtype: Optional[str] = None, max_ctx: Optional[int] = None,
                 page_size: Optional[int] = None, num_pages: Optional[int] = None, kv_gb: Optional[float] = None, max_num_seqs: Optional[int] = None,
                 max_batched_tokens: Optional[int] = None, prefill_chunk: Union[int, str, None] = None, random_weights_seed: Optional[int] = None,
                 device: str = "cuda:0", use_graphs: Optional[bool] = None, pipeline: Optional[bool] = None,
                 options: Union[RuntimeOptions, Mapping[str, Any], None] = None):
        """model: a folder with config.json and model.safetensors, a hub id whose snapshot lies in the hub cache, a TOML
        model spec (config/spec.py), or a raw config.json mapping; with random_weights_seed the weights are made on the
        device instead of read. How the model is run is a `RuntimeOptions`: the defaults, then the `[runtime]` table of
        a model spec, then `options` (a RuntimeOptions or a mapping of its fields), then the keyword arguments given
        here (dtype, page_size, num_pages, kv_gb, max_num_seqs, max_batched_tokens, prefill_chunk, use_graphs, pipeline).
        num_pages / kv_gb size the cache pool; by default it holds max_num_seqs requests of max_ctx tokens, capped by
        free memory. pipeline: keep decode steps one ahead of the host (engine/scheduler.py). prefill_chunk: the longest
        portion of one prompt in a step (crates/specrt/src/runtime.rs:801), or "auto" for the size near 2,048 whose
        matrix-product tiles fill whole rounds of the GPU best at this model's layer sizes."""
        spec = resolve_model(model)
        opts = spec.runtime
        if isinstance(options, RuntimeOptions):
            opts = opts.merged(options.non_default())
        elif options is not None:
            opts = opts.merged(options, "Engine(options=...)")
        opts = opts.merged(dtype=dtype, page_size=page_size, num_pages=num_pages, kv_gb=kv_gb, max_num_seqs=max_num_seqs,
                           max_batched_tokens=max_batched_tokens, prefill_chunk=prefill_chunk, graphs=use_graphs, pipeline=pipeline)
        self.spec, self.options = spec, opts
        self.rt = Runtime(device, options=opts)
        if random_weights_seed is not None:
            self.config, self.decoder = random_model(spec.raw_config, random_weights_seed, self.rt)
            self.model_dir = None
        else:
            if isinstance(model, Mapping):
                raise ValueError("a raw configuration needs random_weights_seed")
            self.config, self.decoder = load_model(spec, self.rt)
            self.model_dir = spec.model_dir
        page_size, max_num_seqs, num_pages = opts.page_size, opts.max_num_seqs, opts.num_pages
        limit = self.decoder.plan.max_positions
        self.max_ctx = min(max_ctx or DEFAULT_MAX_CTX, limit)   # crates/specrt/src/engine.rs:53-60
        needs = self.decoder.cache_needs()
        if num_pages is None:
            per_page = sum(2 * n.kv_heads * n.head_dim * page_size for n in needs if hasattr(n, "kv_heads")) * torch.empty(0, dtype=self.rt.act_dtype).element_size()
            want = max_num_seqs * -(-self.max_ctx // page_size)
            if opts.kv_gb is not None:
                want = int(opts.kv_gb * 2**30 // max(per_page, 1))
            free, _ = torch.cuda.mem_get_info(self.rt.device)
            room = int(free * 0.85 // max(per_page, 1))     # keep headroom for activations (crates/specrt/src/runtime.rs:1164-1182)
            num_pages = max(1, min(want, room))
        self.cache = CacheManager(needs, page_size, num_pages, max_num_seqs, self.max_ctx, device=self.rt.device, dtype=self.rt.act_dtype,
                                  sources=self.decoder.cache_sources())
        prefill_chunk = self._balanced_portion() if opts.prefill_chunk == "auto" else opts.prefill_chunk
        self.runner = ModelRunner(self.decoder, self.cache, self.rt)
        self.executor = GpuExecutor(self.runner, use_graphs=opts.graphs)
        self.scheduler = Scheduler(self.cache, SchedulerConfig(max_num_seqs, opts.max_batched_tokens, prefill_chunk, self.max_ctx, opts.pipeline))
        self._tokenizer = None
        self._next_id = 0

    def _balanced_portion(self) -> int:
        """The portion size for prefill_chunk="auto": from the matrices of the blocks' parts (bfloat16 mode; 2,048 otherwise)."""
        from ..kernels import gemm_tcgen05
        from .runtime import LinearWeights
        if self.rt.mode != "bfloat16":
            return 2048
        seen, matrices = set(), []
        for block in self.decoder.blocks:
            for part in block.parts():
                for v in vars(part).values():
                    if isinstance(v, LinearWeights) and id(v) not in seen:
                        seen.add(id(v))
                        matrices.append((v.n, v.k))
        return gemm_tcgen05.balanced_portion(matrices, sm_count=self.rt.sm_count) if matrices else 2048

    @classmethod
    def load(cls, model, max_ctx: Optional[int] = None, **kw) -> "Engine":
        return cls(model, max_ctx=max_ctx, **kw)

    # ------------------------------------------------------------------ text (optional)
    def tokens(self, text: str) -> list[int]:
        if self._tokenizer is None:
            path = self.model_dir / "tokenizer.json" if self.model_dir else None
            if path is None or not path.is_file():
                raise RuntimeError("this model folder has no tokenizer.json: pass token ids")
            try:
                from tokenizers import Tokenizer
            except ImportError as e:
                raise RuntimeError("the `tokenizers` package is not installed: pass token ids") from e
            self._tokenizer = Tokenizer.from_file(str(path))
        return self._tokenizer.encode(text).ids

    def text(self, ids: Sequence[int]) -> str:
        self.tokens("")
        return self._tokenizer.decode(list(ids))

    # ------------------------------------------------------------------ streaming interface
    def submit(self, prompt: Sequence[int], max_tokens: int = 64, sampling: SamplingParams = GREEDY, stop_ids: Sequence[int] = ()) -> int:
        """Queue one request; returns its id. Raises `Refused` for a request that can never run."""
        rid = self._next_id
        self._next_id += 1
        self.scheduler.submit(Request(rid, list(prompt), max_tokens, sampling, tuple(stop_ids)))
        return rid

    def step(self):
        """One scheduler step on the device; returns its StepReport (tokens emitted, requests finished)."""
        return self.scheduler.step(self.executor)

    def cancel(self, rid: int):
        return self.scheduler.cancel(rid)

    # ------------------------------------------------------------------ generation
    def generate(self, prompt, max_tokens: int = 64, sampling: Union[SamplingParams, Sequence[SamplingParams]] = GREEDY,
                 stop_ids: Sequence[int] = ()) -> Union[Reply, list[Reply]]:
        """prompt: token ids (or text) of one request, or a list of them; all run together through the
        scheduler. Returns one Reply, or a list in the order of the prompts."""
        single = isinstance(prompt, str) or (len(prompt) > 0 and isinstance(prompt[0], int)) or len(prompt) == 0
        prompts = [prompt] if single else list(prompt)
        samplings = [sampling] * len(prompts) if isinstance(sampling, SamplingParams) else list(sampling)
        ids = []
        texts = []
        for p, sp in zip(prompts, samplings):
            texts.append(isinstance(p, str))
            toks = self.tokens(p) if isinstance(p, str) else list(p)
            rid = self._next_id
            self._next_id += 1
            self.scheduler.submit(Request(rid, toks, max_tokens, sp, tuple(stop_ids)))
            ids.append(rid)
        torch.cuda.reset_peak_memory_stats(self.rt.device)
        done: dict[Hashable, Finished] = {}
        first_token_at: dict[Hashable, float] = {}
        t0 = time.perf_counter()
        while len(done) < len(ids):
            report = self.scheduler.step(self.executor)
            now = time.perf_counter()
            for rid, _ in report.emitted:
                first_token_at.setdefault(rid, now)
            for f in report.finished:
                done[f.id] = f
                first_token_at.setdefault(f.id, now)
            if not report.emitted and not report.finished and self.scheduler.idle():
                break
        t1 = time.perf_counter()
        self.rt.check_status()
        peak = torch.cuda.max_memory_allocated(self.rt.device)
        replies = []
        for rid, is_text in zip(ids, texts):
            f = done[rid]
            r = Reply(f.tokens, f.finish, f.prompt_tokens, f.completion_tokens, first_token_at[rid] - t0, t1 - first_token_at[rid], peak)
            if is_text:
                r.text = self.text(f.tokens)
            replies.append(r)
        return replies[0] if single else replies

    def logits(self, prompt: Sequence[int]) -> torch.Tensor:
        """Logits at every position of the prompt, float32 [n, vocab] on the host
        (crates/specrt/src/runtime.rs:2147-2151)."""
        toks = self.tokens(prompt) if isinstance(prompt, str) else list(prompt)
        rid = ("logits", self._next_id)
        self._next_id += 1
        self.cache.admit(rid)
        try:
            rows = []
            chunk = self.scheduler.cfg.prefill_chunk
            for a in range(0, len(toks), chunk):
                part = toks[a:a + chunk]
                rows.append(self.runner.step([StepEntry(rid, part, list(range(len(part))))]).cpu())
            return torch.cat(rows, dim=0)
        finally:
            self.cache.release(rid)
