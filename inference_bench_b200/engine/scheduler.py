"""The scheduler: admits requests, cuts prompts into portions under a token budget, keeps every
decoding request decoding, finishes and frees. It knows the cache manager's bookkeeping but nothing
about the device: what runs a step is an `Executor`. The decisions themselves (admission, preemption,
the rows of a step, finishing) are made by the C++ core (csrc/host/sched_core.cpp) on integer
handles; this class holds what the core does not need (token values, sampling parameters, request
ids), drives the executor and keeps the cache manager's map of request ids in step.

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

import ctypes as C
from dataclasses import dataclass, field
from typing import Any, Hashable, Optional, Protocol, Sequence

from ..cache import native
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


class Sequence_:
    """A request the scheduler knows: its tokens live here, its counters in the core."""
    __slots__ = ("req", "tokens", "_h", "_sched")

    def __init__(self, req: Request, tokens: list[int], handle: int, sched: "Scheduler"):
        self.req, self.tokens, self._h, self._sched = req, tokens, handle, sched   # tokens: prompt + generated

    def _get(self, i: int) -> int:
        out = (C.c_longlong * 7)()
        self._sched._lib.ibh_sched_get(self._sched._core, self._h, out)
        return int(out[i])

    @property
    def generated(self) -> int:       # tokens generated so far (also the sampling step number)
        return self._get(1)

    @property
    def computed(self) -> int:        # positions whose state is in the cache
        return self._get(2)

    @property
    def order(self) -> int:           # admission order, for preemption
        return self._get(3)

    @property
    def preemptions(self) -> int:
        return self._get(4)

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
        self._lib = native.load()
        self._limit = min(config.max_ctx, cache.max_tokens_per_request)
        self._core = self._lib.ibh_sched_new(cache._core, len(cache.groups), config.max_num_seqs, config.max_batched_tokens, config.prefill_chunk,
                                             self._limit)
        self._seqs: dict[int, Sequence_] = {}        # handle -> request, for everything waiting or running
        self._inflight: Optional[_InFlight] = None   # a launched decode step whose tokens have not been read

    def __del__(self):
        core, self._core = getattr(self, "_core", None), None
        if core:
            self._lib.ibh_sched_free(core)

    def _handles(self, count_fn, fill_fn) -> list[int]:
        n = int(count_fn(self._core))
        out = (C.c_int * max(1, n))()
        fill_fn(self._core, out)
        return list(out[:n])

    @property
    def waiting(self) -> list[Sequence_]:
        return [self._seqs[h] for h in self._handles(self._lib.ibh_sched_n_waiting, self._lib.ibh_sched_waiting)]

    @property
    def running(self) -> list[Sequence_]:
        return [self._seqs[h] for h in self._handles(self._lib.ibh_sched_n_running, self._lib.ibh_sched_running)]

    @property
    def total_preemptions(self) -> int:
        return int(self._lib.ibh_sched_total_preemptions(self._core))

    # ------------------------------------------------------------------ submit / cancel
    def submit(self, req: Request) -> None:
        n = len(req.prompt)
        if n == 0:
            raise Refused(f"request {req.id!r}: the prompt is empty")
        if req.max_tokens <= 0:
            raise Refused(f"request {req.id!r}: max_tokens must be positive")
        limit = self._limit
        if n + req.max_tokens > limit:
            raise Refused(f"request {req.id!r}: prompt ({n}) + max_tokens ({req.max_tokens}) exceeds the context limit {limit}")
        need = max(self.cache.pages_missing(None, n + req.max_tokens, 0), default=0)
        most = min((g.pool.num_pages for g in self.cache.groups), default=need)
        if need > most:
            raise Refused(f"request {req.id!r}: needs {need} cache pages but the pool has {most}")
        if any(s.req.id == req.id for s in self._seqs.values()):
            raise Refused(f"request {req.id!r} is already known")
        h = int(self._lib.ibh_sched_submit(self._core, n, int(req.max_tokens)))
        self._seqs[h] = Sequence_(req, list(req.prompt), h, self)

    def cancel(self, req_id: Hashable) -> Optional[Finished]:
        for h, s in self._seqs.items():
            if s.req.id == req_id:
                was = int(self._lib.ibh_sched_cancel(self._core, h))
                if was == 2:
                    self.cache._forget(req_id)   # the core has given its pages and slot back
                del self._seqs[h]
                return self._finished(s, "cancelled") if was else None
        return None

    def idle(self) -> bool:
        return not self._seqs

    # ------------------------------------------------------------------ one step
    def step(self, executor: Executor) -> StepReport:
        if self._inflight is not None or (self.cfg.pipeline and hasattr(executor, "launch_decode")):
            ahead = self._step_ahead(executor)
            if ahead is not None:
                return ahead
        report = StepReport()
        cap = len(self._seqs) + 1
        preempted, admitted, rows, counts = (C.c_int * cap)(), (C.c_int * (2 * cap))(), (C.c_int * (4 * cap))(), (C.c_int * 5)()
        self._lib.ibh_sched_plan(self._core, preempted, admitted, rows, counts)
        n_pre, n_adm, n_rows, report.decode_rows, report.prefill_tokens = (int(c) for c in counts)
        report.preemptions = n_pre
        for i in range(n_pre):                        # the core has freed what they held: the cache manager forgets them
            self.cache._forget(self._seqs[preempted[i]].req.id)
        for i in range(n_adm):                        # and has given these a slot and their pages
            self.cache._adopt(self._seqs[admitted[2 * i]].req.id, int(admitted[2 * i + 1]))
        entries: list[StepEntry] = []
        sampling: list[tuple[SamplingParams, int]] = []
        owners: list[Sequence_] = []
        plan: list[tuple[Sequence_, int]] = []
        for i in range(n_rows):
            s, start, n, samples = self._seqs[rows[4 * i]], int(rows[4 * i + 1]), int(rows[4 * i + 2]), bool(rows[4 * i + 3])
            entries.append(StepEntry(s.req.id, s.tokens[start:start + n], [n - 1] if samples else []))
            if samples:
                sampling.append((s.req.sampling, s.generated))
                owners.append(s)
            plan.append((s, n))
        if not entries:
            return report
        tokens = executor.execute(entries, sampling)
        if len(tokens) != len(owners):
            raise RuntimeError(f"the executor returned {len(tokens)} tokens for {len(owners)} sampled rows")
        for s, n in plan:
            self._lib.ibh_sched_computed(self._core, s._h, n)
        for s, tok in zip(owners, tokens):
            self._accept(s, int(tok), report)
        return report

    # ------------------------------------------------------------------ steps kept one ahead
    def _step_ahead(self, executor) -> Optional[StepReport]:
        """One step's report while decode steps are kept one ahead; None when this step has to run the ordinary way."""
        fl = self._inflight
        steady = bool(self._lib.ibh_sched_steady(self._core))
        running = self.running if fl is not None else None
        same = fl is not None and len(fl.owners) == len(running) and all(a is b for a, b in zip(fl.owners, running))
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
            if self._seqs.get(s._h) is s:                # else it stopped or was cancelled after the launch: the token is dropped
                self._lib.ibh_sched_computed(self._core, s._h, 1)
                self._accept(s, int(tok), report)
        return report

    # ------------------------------------------------------------------ a sampled token arrives
    def _accept(self, s: Sequence_, token: int, report: StepReport) -> None:
        """The core counts the token and says whether the request goes on (sched.rs:1577-1589)."""
        stop = token in s.req.stop_ids
        verdict = int(self._lib.ibh_sched_accept(self._core, s._h, 1 if stop else 0))
        if not stop:
            s.tokens.append(token)
            report.emitted.append((s.req.id, token))
        if verdict:
            self.cache._forget(s.req.id)             # the core has given its pages and slot back
            del self._seqs[s._h]
            report.finished.append(self._finished(s, "stop" if verdict == 1 else "length"))

    def _finished(self, s: Sequence_, why: str) -> Finished:
        n = len(s.req.prompt)
        return Finished(s.req.id, s.tokens[n:], why, n, len(s.tokens) - n)
