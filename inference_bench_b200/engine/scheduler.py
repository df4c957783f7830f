"""The scheduler: admits requests, cuts prompts into portions under a token budget, keeps every
decoding request decoding, finishes and frees. It knows the cache manager's bookkeeping but nothing
about the device: what runs a step is an `Executor`.

Policy, after the reference's scheduler (crates/specrt/src/sched.rs; docs/specrt-scheduler.md):
  * submit refuses what can never run: an empty prompt, max_tokens 0, prompt + max_tokens beyond the
    context limit, or more pages than the pool has (sched.rs:967-981);
  * every step, each decoding request gets one row (sched.rs:1403-1418); if one of them needs a new
    page and none is free, the most recently admitted request is preempted: its pages and slot are
    given back and it returns to the front of the waiting queue with its prompt and what it has
    generated so far, to be recomputed later (sched.rs:1090-1130);
  * the rest of the budget (max_batched_tokens minus the decode rows) goes to prompts: waiting
    requests are admitted first come first served while a slot is free and all pages for their
    tokens plus one are free beyond a small reserve (sched.rs:1132-1230), then running prompts get
    portions, shortest remaining first, each at most prefill_chunk tokens (sched.rs:1457-1530);
  * the last portion of a prompt samples the first token (sched.rs:1496-1497);
  * a request finishes on a stop token (not emitted), at max_tokens, or at the context limit
    (sched.rs:1577-1589), and gives back its pages and slot at once.

While every running request decodes and none waits, steps are kept one ahead (`pipeline`): an executor
that can enqueue a decode step without waiting for it (`launch_decode` / `collect`) is given the next
step, whose input tokens it takes from the step before on the device, before the tokens of the
current step are read back; the host's share of a step then runs while the device computes. A
request that stops on a token the host had not seen yet has computed one token too many, which is
dropped. Every call of `step` still reports exactly one step.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any, Hashable, Optional, Protocol, Sequence

from ..cache.manager import CacheManager, OutOfPages
from ..sampling.params import GREEDY, SamplingParams
from .step import StepEntry


class Refused(ValueError):
    """A request that can never run was submitted."""


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 64            # requests running at once (also bounded by the cache manager's slots)
    max_batched_tokens: int = 8192    # tokens in one step, decode rows included (sched.rs:503-538)
    prefill_chunk: int = 2048         # longest portion of one prompt in one step (runtime.rs:801)
    max_ctx: int = 2048               # context limit: prompt + generated tokens (engine.rs:10)
    pipeline: bool = True             # keep decode steps one ahead when the executor can launch without waiting


@dataclass
class Request:
    id: Hashable
    prompt: Sequence[int]
    max_tokens: int = 64
    sampling: SamplingParams = GREEDY
    stop_ids: Sequence[int] = ()


@dataclass
class Sequence_:
    req: Request
    tokens: list[int]                  # prompt + generated
    generated: int = 0                 # tokens generated so far (also the sampling step number)
    computed: int = 0                  # positions whose state is in the cache
    order: int = 0                     # admission order, for preemption
    preemptions: int = 0

    @property
    def decoding(self) -> bool:
        return self.generated > 0 and self.computed == len(self.tokens) - 1

    @property
    def remaining_prefill(self) -> int:
        return len(self.tokens) - self.computed


@dataclass
class Finished:
    id: Hashable
    tokens: list[int]                  # generated tokens (a stop token is not among them)
    finish: str                        # "stop" | "length" | "cancelled"
    prompt_tokens: int
    completion_tokens: int


@dataclass
class StepReport:
    """What a step did (crates/specrt/src/sched.rs:573-583)."""
    decode_rows: int = 0
    prefill_tokens: int = 0
    preemptions: int = 0
    emitted: list[tuple[Hashable, int]] = field(default_factory=list)   # (request, token) in batch order
    finished: list[Finished] = field(default_factory=list)


class Executor(Protocol):
    def execute(self, entries: list[StepEntry], sampling: list[tuple[SamplingParams, int]]) -> list[int]:
        """Run one step; `sampling[i]` belongs to the i-th wanted row. Returns one token per wanted row."""

    # Optional, for steps kept one ahead:
    #   launch_decode(entries, sampling, feed) -> handle or None: enqueue a step of single decoded tokens
    #     (cache extended and committed as `execute` does) without waiting; with `feed` the input tokens are
    #     the tokens the step before sampled for the same rows, and entries[i].tokens is ignored. None: cannot.
    #   collect(handle) -> list[int]: wait for that step and return its tokens. Handles are collected in order.


@dataclass
class _InFlight:
    handle: Any
    owners: list["Sequence_"]


class Scheduler:
    def __init__(self, cache: CacheManager, config: SchedulerConfig):
        self.cache, self.cfg = cache, config
        self.waiting: deque[Sequence_] = deque()
        self.running: list[Sequence_] = []
        self._order = 0
        self.total_preemptions = 0
        self._inflight: Optional[_InFlight] = None   # a launched decode step whose tokens have not been read

    # ------------------------------------------------------------------ submit / cancel
    def submit(self, req: Request) -> None:
        n = len(req.prompt)
        if n == 0:
            raise Refused(f"request {req.id!r}: the prompt is empty")
        if req.max_tokens <= 0:
            raise Refused(f"request {req.id!r}: max_tokens must be positive")
        limit = min(self.cfg.max_ctx, self.cache.max_tokens_per_request)
        if n + req.max_tokens > limit:
            raise Refused(f"request {req.id!r}: prompt ({n}) + max_tokens ({req.max_tokens}) exceeds the context limit {limit}")
        need = max(self.cache.pages_missing(None, n + req.max_tokens, 0), default=0)
        most = min((g.pool.num_pages for g in self.cache.groups), default=need)
        if need > most:
            raise Refused(f"request {req.id!r}: needs {need} cache pages but the pool has {most}")
        if any(s.req.id == req.id for s in list(self.waiting) + self.running):
            raise Refused(f"request {req.id!r} is already known")
        self.waiting.append(Sequence_(req, list(req.prompt)))

    def cancel(self, req_id: Hashable) -> Optional[Finished]:
        for s in list(self.waiting):
            if s.req.id == req_id:
                self.waiting.remove(s)
                return self._finished(s, "cancelled")
        for s in self.running:
            if s.req.id == req_id:
                self._release(s)
                return self._finished(s, "cancelled")
        return None

    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ------------------------------------------------------------------ one step
    def step(self, executor: Executor) -> StepReport:
        if self._inflight is not None or (self.cfg.pipeline and hasattr(executor, "launch_decode")):
            ahead = self._step_ahead(executor)
            if ahead is not None:
                return ahead
        report = StepReport()
        self._grow_decoders(report)
        decoders = [s for s in self.running if s.decoding]
        budget = max(0, self.cfg.max_batched_tokens - len(decoders))
        budget = self._admit(budget)
        entries: list[StepEntry] = []
        sampling: list[tuple[SamplingParams, int]] = []
        owners: list[Sequence_] = []
        plan: list[tuple[Sequence_, int]] = []
        for s in decoders:
            entries.append(StepEntry(s.req.id, [s.tokens[-1]], [0]))
            sampling.append((s.req.sampling, s.generated))
            owners.append(s)
            plan.append((s, 1))
        left = self.cfg.max_batched_tokens - len(decoders)
        for s in sorted((s for s in self.running if not s.decoding), key=lambda s: (s.remaining_prefill, s.order)):
            if left <= 0:
                break
            n = min(s.remaining_prefill, self.cfg.prefill_chunk, left)
            last = n == s.remaining_prefill
            entries.append(StepEntry(s.req.id, s.tokens[s.computed:s.computed + n], [n - 1] if last else []))
            if last:
                sampling.append((s.req.sampling, s.generated))
                owners.append(s)
            plan.append((s, n))
            left -= n
            report.prefill_tokens += n
        report.decode_rows = len(decoders)
        if not entries:
            return report
        tokens = executor.execute(entries, sampling)
        if len(tokens) != len(owners):
            raise RuntimeError(f"the executor returned {len(tokens)} tokens for {len(owners)} sampled rows")
        for s, n in plan:
            s.computed += n
        for s, tok in zip(owners, tokens):
            self._accept(s, int(tok), report)
        return report

    # ------------------------------------------------------------------ steps kept one ahead
    def _step_ahead(self, executor) -> Optional[StepReport]:
        """One step's report while decode steps are kept one ahead; None when this step has to run the ordinary way."""
        fl = self._inflight
        steady = bool(self.running) and not self.waiting and all(s.decoding for s in self.running)
        same = fl is not None and len(fl.owners) == len(self.running) and all(a is b for a, b in zip(fl.owners, self.running))
        if fl is not None and not (steady and same):    # the batch changes: read what is in flight, start afresh next time
            self._inflight = None
            return self._collect(executor, fl)
        if not steady:
            return None
        if fl is None:
            fl = self._launch(executor, feed=False, ahead=0)
            if fl is None:
                return None
        limit = min(self.cfg.max_ctx, self.cache.max_tokens_per_request)
        goes_on = all(s.generated + 1 < s.req.max_tokens and len(s.tokens) + 1 < limit for s in fl.owners)
        self._inflight = self._launch(executor, feed=True, ahead=1) if goes_on else None
        return self._collect(executor, fl)

    def _launch(self, executor, feed: bool, ahead: int) -> Optional[_InFlight]:
        owners = list(self.running)
        entries = [StepEntry(s.req.id, [0 if feed else s.tokens[-1]], [0]) for s in owners]
        sampling = [(s.req.sampling, s.generated + ahead) for s in owners]
        try:
            handle = executor.launch_decode(entries, sampling, feed)
        except OutOfPages:
            return None
        return None if handle is None else _InFlight(handle, owners)

    def _collect(self, executor, fl: _InFlight) -> StepReport:
        report = StepReport(decode_rows=len(fl.owners))
        tokens = executor.collect(fl.handle)
        if len(tokens) != len(fl.owners):
            raise RuntimeError(f"the executor returned {len(tokens)} tokens for {len(fl.owners)} rows")
        for s, tok in zip(fl.owners, tokens):
            if any(s is r for r in self.running):       # else it stopped or was cancelled after the launch: the token is dropped
                s.computed += 1
                self._accept(s, int(tok), report)
        return report

    # ------------------------------------------------------------------ pieces of the policy
    def _grow_decoders(self, report: StepReport) -> None:
        """Every decoder needs room for one more position; preempt the newest request until it has."""
        for s in sorted((s for s in self.running if s.decoding), key=lambda s: s.order):
            while s in self.running:
                try:
                    self.cache.extend(s.req.id, s.computed + 1)
                    break
                except OutOfPages:
                    victim = max(self.running, key=lambda r: r.order)
                    self._preempt(victim)
                    report.preemptions += 1

    def _preempt(self, s: Sequence_) -> None:
        """Recompute later: everything the request holds is freed; tokens it has emitted stay emitted."""
        self._release(s)
        s.computed = 0
        s.preemptions += 1
        self.total_preemptions += 1
        self.waiting.appendleft(s)

    def _admit(self, budget: int) -> int:
        planned = sum(min(s.remaining_prefill, self.cfg.prefill_chunk) for s in self.running if not s.decoding)
        while self.waiting and planned < budget:
            s = self.waiting[0]
            if len(self.running) >= self.cfg.max_num_seqs or self.cache.free_slots() == 0:
                break
            pool = min((g.pool.num_pages for g in self.cache.groups), default=0)
            reserve = max(1, pool // 100) if self.running else 0    # sched.rs:959-961
            if not self.cache.can_extend(None, len(s.tokens) + 1, 0, reserve):
                break
            self.waiting.popleft()
            self.cache.admit(s.req.id)
            self.cache.extend(s.req.id, len(s.tokens) + 1)
            s.order = self._order
            self._order += 1
            self.running.append(s)
            planned += min(s.remaining_prefill, self.cfg.prefill_chunk)
        return budget

    def _accept(self, s: Sequence_, token: int, report: StepReport) -> None:
        """A sampled token arrives (sched.rs:1577-1589)."""
        if token in s.req.stop_ids:
            self._release(s)
            report.finished.append(self._finished(s, "stop"))
            return
        s.tokens.append(token)
        s.generated += 1
        report.emitted.append((s.req.id, token))
        limit = min(self.cfg.max_ctx, self.cache.max_tokens_per_request)
        if s.generated >= s.req.max_tokens or len(s.tokens) >= limit:
            self._release(s)
            report.finished.append(self._finished(s, "length"))

    def _release(self, s: Sequence_) -> None:
        if s in self.running:
            self.running.remove(s)
        if self.cache.has(s.req.id):
            self.cache.release(s.req.id)

    def _finished(self, s: Sequence_, why: str) -> Finished:
        n = len(s.req.prompt)
        return Finished(s.req.id, s.tokens[n:], why, n, len(s.tokens) - n)
