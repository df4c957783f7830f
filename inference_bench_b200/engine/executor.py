"""Runs the scheduler's steps on the device: the step function, then sampling, tokens back to the host.

Steps that hold only decoded tokens are the launch-bound inner loop of generation, so they are
replayed as CUDA graphs, one per padded batch size (1, 2, 4, ... rows), like the reference's
`Stepper` (crates/specrt/src/runtime/step.rs:8-20, 197-228): all inputs of such a step live in one
static device buffer that a single copy fills, padded rows write to a scratch page and a scratch
slot, and the graph holds the whole model, the sampling kernel included.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .context import Segment, StepContext
from .step import ModelRunner, StepEntry


RUN_AHEAD_MAX = 64


class _DecodeGraph:
    """The captured decode step for `rows` rows and the static buffers it reads and writes."""

    def __init__(self, runner: ModelRunner, rows: int):
        self.runner, self.rows = runner, rows
        cache, rt = runner.cache, runner.rt
        B, W = rows, cache.table_width
        n_groups = len(cache.groups)
        # layout of the int32 input block: tokens | positions | seg_pos0 | seg_slot | params[B,6] | tables[g][B,W] | count
        self.n_ints = 4 * B + 6 * B + n_groups * B * W + 1
        self.host = torch.zeros(self.n_ints, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(self.n_ints, dtype=torch.int32, device=rt.device)
        h = self.host.numpy()
        self.h_tokens, self.h_pos, self.h_pos0, self.h_slot = h[0:B], h[B:2 * B], h[2 * B:3 * B], h[3 * B:4 * B]
        self.h_params = h[4 * B:10 * B].reshape(B, 6)
        self.h_tables = [h[10 * B + g * B * W:10 * B + (g + 1) * B * W].reshape(B, W) for g in range(n_groups)]
        d = self.dev
        self.d_tables = [d[10 * B + g * B * W:10 * B + (g + 1) * B * W].view(B, W) for g in range(n_groups)]
        const = torch.arange(B + 1, dtype=torch.int32, device=rt.device)
        segs = [Segment(None, cache.scratch_slot, 0, [0], [0]) for _ in range(B)]
        ar = np.arange(B, dtype=np.int32)
        self.ctx = StepContext(
            rt, segs, B, self.h_tokens, self.h_pos, ar, np.arange(B + 1, dtype=np.int32), self.h_pos0, self.h_slot, ar,
            token_ids=d[0:B], positions=d[B:2 * B], seg_of_token=const[:B], seg_start=const, seg_pos0=d[2 * B:3 * B], seg_slot=d[3 * B:4 * B],
            logit_rows=const[:B], caches=cache.views(self.d_tables))
        self.ctx.fixed_shape = True
        self.d_params = d[4 * B:10 * B].view(B, 6)
        self.d_count = d[self.n_ints - 1:self.n_ints]
        self.history = torch.zeros((RUN_AHEAD_MAX, B), dtype=torch.int32, device=rt.device)
        self.h_history = torch.zeros((RUN_AHEAD_MAX, B), dtype=torch.int32).pin_memory()
        self.result = torch.zeros(B + 1, dtype=torch.int32, device=rt.device)   # the step's tokens, then the status word after the step
        self.tokens = self.result[:B]
        self.h_out = torch.zeros(B + 1, dtype=torch.int32).pin_memory()
        # for steps launched without waiting (two may be in flight): a staging copy of the inputs, a place for the tokens and an event each
        self.stages = [torch.zeros(self.n_ints, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.h_outs = [torch.zeros(B + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.events = [torch.cuda.Event() for _ in range(2)]
        self.pending = [False, False]
        self.turn = 0
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._pad_all()

    def _pad_all(self) -> None:
        cache = self.runner.cache
        self.h_tokens[:] = 0
        self.h_pos[:] = 0
        self.h_pos0[:] = 0
        self.h_slot[:] = cache.scratch_slot
        self.h_params[:] = 0
        for g, t in enumerate(self.h_tables):
            t[:] = cache.scratch_page(g)

    def _forward(self) -> None:
        from ..kernels import ops
        self.ctx.memo = {}
        self.logits = self.runner.decoder.forward(self.ctx)
        ops.sample_rows(self.logits, self.d_params, self.result, self.runner.rt.status)
        c = self.ctx
        ops.advance_rows(self.tokens, c.token_ids, c.positions, c.seg_pos0, self.d_params, self.history, self.d_count)

    def capture(self) -> None:
        self.runner.rt.activate()
        self.dev.copy_(self.host, non_blocking=True)
        stream = torch.cuda.Stream(device=self.runner.rt.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):   # warm-up outside the capture: lazy kernel attributes, allocator
                self._forward()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        from ..kernels import lib
        before = lib.launches
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._forward()
        self.launches = lib.launches - before    # kernels in one replay

    def run_ahead(self, entries: list[StepEntry], sampling: list[tuple[SamplingParams, int]], steps: int) -> list[list[int]]:
        """`steps` decode steps with no host work in between: every step's sampled tokens are the next
        step's inputs on the device. The requests' pages for all `steps` positions must be allocated.
        Returns the tokens of every step, [steps][rows]."""
        if not 1 <= steps <= RUN_AHEAD_MAX:
            raise ValueError(f"run_ahead takes 1 to {RUN_AHEAD_MAX} steps, got {steps}")
        self._fill(entries, sampling)
        self.dev.copy_(self.host, non_blocking=True)
        for _ in range(steps):
            self.graph.replay()
        self.h_history.copy_(self.history, non_blocking=True)
        self.h_out.copy_(self.result, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.runner.rt.raise_for(int(self.h_out[self.rows]))
        return self.h_history[:steps, :len(entries)].tolist()

    def run(self, entries: list[StepEntry], sampling: list[tuple[SamplingParams, int]]) -> list[int]:
        n = len(entries)
        self._fill(entries, sampling)
        self.dev.copy_(self.host, non_blocking=True)
        self.graph.replay()
        self.h_out.copy_(self.result, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.runner.rt.raise_for(int(self.h_out[self.rows]))
        return self.h_out[:n].tolist()

    def launch(self, entries: list[StepEntry], sampling: list[tuple[SamplingParams, int]], feed: bool) -> tuple[int, int]:
        """Enqueue one step and return at once. With `feed` the input tokens stay what the step before
        left on the device (its sampled tokens, row by row): everything but the tokens is copied."""
        slot = self.turn
        if self.pending[slot]:
            raise RuntimeError("two decode steps are already in flight")
        self.turn ^= 1
        self._fill(entries, sampling, tokens=not feed)
        stage = self.stages[slot]
        stage.copy_(self.host)
        if feed:
            self.dev[self.rows:].copy_(stage[self.rows:], non_blocking=True)
        else:
            self.dev.copy_(stage, non_blocking=True)
        self.graph.replay()
        self.h_outs[slot].copy_(self.result, non_blocking=True)
        self.events[slot].record()
        self.pending[slot] = True
        return slot, len(entries)

    def collect(self, handle: tuple[int, int]) -> list[int]:
        slot, n = handle
        self.events[slot].synchronize()
        self.pending[slot] = False
        self.runner.rt.raise_for(int(self.h_outs[slot][self.rows]))
        return self.h_outs[slot][:n].tolist()

    def _fill(self, entries: list[StepEntry], sampling: list[tuple[SamplingParams, int]], tokens: bool = True) -> None:
        cache = self.runner.cache
        n = len(entries)
        if n < self.rows:
            self._pad_all()
        slots = cache.fill_rows([e.request for e in entries], self.h_pos, self.h_tables)   # positions and block tables, straight into the pinned block
        if tokens:
            self.h_tokens[:n] = [e.tokens[0] for e in entries]
        self.h_pos0[:n] = self.h_pos[:n]
        self.h_slot[:n] = slots
        self.h_params[:n] = [p.row(step) for p, step in sampling]


class GpuExecutor:
    def __init__(self, runner: ModelRunner, use_graphs: bool = True, max_graph_rows: int = 256):
        self.runner = runner
        self.sampler = Sampler(runner.rt.device)
        self.use_graphs, self.max_graph_rows = use_graphs, max_graph_rows
        self._graphs: dict[int, _DecodeGraph] = {}
        self.last_logits: Optional[torch.Tensor] = None
        self.steps = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def graph_for(self, n_rows: int) -> _DecodeGraph:
        rows = 1
        while rows < n_rows:
            rows *= 2
        g = self._graphs.get(rows)
        if g is None:
            g = self._graphs[rows] = _DecodeGraph(self.runner, rows)
            g.capture()
        return g

    def decode_ahead(self, entries: list[StepEntry], sampling: list[tuple[SamplingParams, int]], steps: int) -> list[list[int]]:
        """Several decode steps of the same requests in a row, tokens fed back on the device."""
        cache = self.runner.cache
        g = self.graph_for(len(entries))
        for e in entries:
            cache.extend(e.request, cache.length(e.request) + steps)
        out = g.run_ahead(entries, sampling, steps)
        for e in entries:
            cache.commit(e.request, cache.length(e.request) + steps)
        self.steps += steps
        self.h2d_bytes += g.n_ints * 4
        self.d2h_bytes += steps * g.rows * 4 + 4
        return out

    def launch_decode(self, entries: list[StepEntry], sampling: list[tuple[SamplingParams, int]], feed: bool = False):
        """Enqueue a step of single decoded tokens without waiting for it; `collect` returns its tokens.
        With `feed`, every row's input token is the one the step before sampled for it, taken on the
        device. None when such a step cannot run as a graph. Raises OutOfPages with nothing changed."""
        if not self.use_graphs or len(entries) > self.max_graph_rows:
            return None
        cache = self.runner.cache
        if not feed:
            for e in entries:
                if not 0 <= e.tokens[0] < self.runner.vocab:
                    raise ValueError(f"request {e.request!r}: token id {e.tokens[0]} is outside the vocabulary of {self.runner.vocab}")
        g = self.graph_for(len(entries))
        try:
            for e in entries:
                cache.extend(e.request, cache.length(e.request) + 1)
        except Exception:
            for e in entries:
                cache.shrink_to_committed(e.request)
            raise
        handle = g.launch(entries, sampling, feed)
        for e in entries:
            cache.commit(e.request, cache.length(e.request) + 1)
        self.steps += 1
        self.h2d_bytes += (g.n_ints - (g.rows if feed else 0)) * 4
        self.d2h_bytes += g.rows * 4 + 4
        return g, handle

    def collect(self, handle) -> list[int]:
        g, h = handle
        return g.collect(h)

    def execute(self, entries: list[StepEntry], sampling: list[tuple[SamplingParams, int]]) -> list[int]:
        self.steps += 1
        cache = self.runner.cache
        if self.use_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries) and len(entries) <= self.max_graph_rows:
            g = self.graph_for(len(entries))
            for e in entries:
                tok = e.tokens[0]
                if not 0 <= tok < self.runner.vocab:
                    raise ValueError(f"request {e.request!r}: token id {tok} is outside the vocabulary of {self.runner.vocab}")
                cache.extend(e.request, cache.length(e.request) + 1)
            out = g.run(entries, sampling)
            for e in entries:
                cache.commit(e.request, cache.length(e.request) + 1)
            self.last_logits = g.logits
            self.h2d_bytes += g.n_ints * 4
            self.d2h_bytes += g.rows * 4 + 4
            return out
        logits = self.runner.step(entries, check=False)
        if logits is None:   # nothing to sample: no transfer comes back, so the status word is read when a later step's tokens are
            return []
        tokens = self.sampler.sample(logits, [p for p, _ in sampling], [s for _, s in sampling], self.runner.rt.status)
        self.last_logits = logits
        self.h2d_bytes += sum(len(e.tokens) for e in entries) * 12 + len(entries) * (12 + 4 * cache.table_width * len(cache.groups)) + len(sampling) * 28
        self.d2h_bytes += len(sampling) * 4 + 4
        host = tokens.cpu().tolist()
        self.runner.rt.raise_for(host[-1])
        return host[:-1]
