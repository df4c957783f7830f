"""The scheduler's decisions on the CPU, with a fake executor in place of the device.

The fake keeps a paged "memory" of its own: every token of a step is written to the page and slot
the request's block table names, and before a request's next token is computed its whole history is
read back through the table and compared with what the request really holds. A page handed to two
requests, a stale table, or a portion that starts at the wrong position fails that check. The next
token is a hash of the history, so outputs are comparable with a request run alone
(the reference tests its scheduler the same way: crates/specrt/src/sched.rs:1591-1760)."""
import numpy as np
import pytest

from inference_bench_b200.cache.manager import CacheManager
from inference_bench_b200.engine.scheduler import Refused, Request, Scheduler, SchedulerConfig
from inference_bench_b200.parts.base import PagedKV
from inference_bench_b200.sampling.params import SamplingParams

VOCAB = 1000


def next_token(history) -> int:
    h = 1469598103
    for t in history:
        h = (h * 1099511 + int(t) + 7) % 2147483647
    return h % VOCAB


def alone(prompt, n, stop=()):
    seq = list(prompt)
    out = []
    for _ in range(n):
        t = next_token(seq)
        if t in stop:
            break
        seq.append(t)
        out.append(t)
    return out


class FakeExecutor:
    def __init__(self, cache: CacheManager, truth: dict):
        self.cache, self.truth = cache, truth
        self.memory = np.full((cache.groups[0].pool.num_pages, cache.page_size), -1, dtype=np.int64)
        self.steps = []

    def execute(self, entries, sampling):
        out = []
        self.steps.append([(e.request, len(e.tokens)) for e in entries])
        for e in entries:
            self.cache.extend(e.request, self.cache.length(e.request) + len(e.tokens))
        for e in entries:
            start = self.cache.length(e.request)
            table = self.cache.table(0, e.request)
            for i, tok in enumerate(e.tokens):
                p = start + i
                assert table[p // self.cache.page_size] >= 0
                self.memory[table[p // self.cache.page_size], p % self.cache.page_size] = tok
            n = start + len(e.tokens)
            seen = [self.memory[table[p // self.cache.page_size], p % self.cache.page_size] for p in range(n)]
            assert seen == list(self.truth[e.request].tokens[:n]), f"request {e.request}: the cache does not hold its history"
            self.cache.commit(e.request, n)
            if e.want:
                out.append(next_token(seen))
        assert len(out) == len(sampling)
        return out


class AheadExecutor(FakeExecutor):
    """A fake that can also take a decode step without answering at once. The cache is extended and
    committed at the launch, as on the device; the "memory" is written and read when the step is
    collected, in launch order, so a step fed from the one before sees that step's tokens."""

    def __init__(self, cache, truth):
        super().__init__(cache, truth)
        self.queue = []
        self.fed = {}            # request -> the token its last launched step sampled (what the device would feed)
        self.launched = 0
        self.wasted = 0

    def launch_decode(self, entries, sampling, feed):
        for e in entries:
            self.cache.extend(e.request, self.cache.length(e.request) + 1)
        rows = []
        for e in entries:
            start = self.cache.length(e.request)
            rows.append((e.request, start, self.cache.table(0, e.request).copy(), None if feed else e.tokens[0]))
            self.cache.commit(e.request, start + 1)
        self.queue.append(rows)
        self.launched += 1
        self.steps.append([(e.request, 1) for e in entries])
        return len(self.queue) - 1

    def collect(self, handle):
        assert handle == len(self.queue) - len([q for q in self.queue if q is not None]), "steps are collected in launch order"
        rows, self.queue[handle] = self.queue[handle], None
        out = []
        for rid, start, table, tok in rows:
            tok = self.fed[rid] if tok is None else tok
            self.memory[table[start // self.cache.page_size], start % self.cache.page_size] = tok
            seen = [self.memory[table[p // self.cache.page_size], p % self.cache.page_size] for p in range(start + 1)]
            if self.cache.has(rid) and len(self.truth[rid].tokens) > start:
                assert seen == list(self.truth[rid].tokens[:start + 1]), f"request {rid}: the cache does not hold its history"
            else:
                self.wasted += 1          # the request ended after this step was launched
            self.fed[rid] = next_token(seen)
            out.append(self.fed[rid])
        return out


def make(pages=64, page=4, slots=8, executor=FakeExecutor, **cfg):
    cache = CacheManager([PagedKV(1, 8, None)], page, pages, slots, cfg.get("max_ctx", 256))
    sched = Scheduler(cache, SchedulerConfig(**{"max_num_seqs": slots, "max_batched_tokens": 64, "prefill_chunk": 16, "max_ctx": 256, **cfg}))
    truth = {}
    ex = executor(cache, truth)

    def submit(rid, prompt, n, **kw):
        sched.submit(Request(rid, prompt, n, **kw))
        truth[rid] = next(s for s in sched.waiting if s.req.id == rid)
    return cache, sched, ex, submit


def run(sched, ex, limit=10000):
    done, reports = {}, []
    for _ in range(limit):
        if sched.idle():
            break
        rep = sched.step(ex)
        reports.append(rep)
        for f in rep.finished:
            done[f.id] = f
        sched.cache.check()
    assert sched.idle()
    return done, reports


def prompt(seed, n):
    return np.random.default_rng(seed).integers(0, VOCAB, n).tolist()


def test_outputs_equal_requests_run_alone_and_everything_is_freed():
    cache, sched, ex, submit = make()
    reqs = {i: (prompt(i, n), k) for i, (n, k) in enumerate([(5, 9), (40, 3), (17, 20), (1, 12), (33, 1)])}
    for i, (p, k) in reqs.items():
        submit(i, p, k)
    done, _ = run(sched, ex)
    for i, (p, k) in reqs.items():
        assert done[i].tokens == alone(p, k) and done[i].finish == "length"
        assert done[i].prompt_tokens == len(p) and done[i].completion_tokens == k
    assert cache.used_pages() == [0] and cache.free_slots() == 8


def test_budget_chunks_and_decoders_never_skipped():
    cache, sched, ex, submit = make(max_batched_tokens=24, prefill_chunk=10)
    submit("short", prompt(1, 3), 30)
    done = {}
    rep = sched.step(ex)                       # prefill of the short prompt samples its first token
    assert rep.prefill_tokens == 3 and len(rep.emitted) == 1
    submit("long", prompt(2, 95), 2)
    while not sched.idle():
        rep = sched.step(ex)
        step = dict(ex.steps[-1])
        assert sum(step.values()) <= 24                                    # the token budget holds, decode rows included
        if "short" in step or any(s.req.id == "short" for s in sched.running):
            assert step.get("short", 1) == 1                               # the decoder gets its row every step
        if "long" in step and step["long"] > 1:
            assert step["long"] <= 10                                      # no portion beyond prefill_chunk
        for f in rep.finished:
            done[f.id] = f
    assert done["short"].tokens == alone(prompt(1, 3), 30) and done["long"].tokens == alone(prompt(2, 95), 2)
    long_portions = [dict(s)["long"] for s in ex.steps if "long" in dict(s) and dict(s)["long"] > 1]
    assert sum(long_portions) == 95 and len(long_portions) == 10


def test_shortest_remaining_prompt_goes_first_and_admission_is_fifo():
    cache, sched, ex, submit = make(max_batched_tokens=40, prefill_chunk=20, slots=2)
    submit("a", prompt(1, 30), 1)
    submit("b", prompt(2, 6), 1)
    submit("c", prompt(3, 2), 1)               # has to wait for a slot although it is the shortest
    sched.step(ex)
    first = dict(ex.steps[0])
    assert first == {"b": 6, "a": 20}          # both admitted in order; the shorter prompt is served first, a gets one full portion
    assert [s.req.id for s in sched.waiting] == ["c"]
    done, _ = run(sched, ex)
    assert set(done) | {"b"} == {"a", "b", "c"}


def test_preemption_recomputes_and_outputs_do_not_change():
    cache, sched, ex, submit = make(pages=10, page=4, slots=4, max_batched_tokens=32, prefill_chunk=8)
    reqs = {i: (prompt(10 + i, n), k) for i, (n, k) in enumerate([(6, 20), (9, 14), (3, 25), (12, 8), (5, 18), (7, 11)])}
    for i, (p, k) in reqs.items():
        submit(i, p, k)
    done, reports = run(sched, ex)
    assert sum(r.preemptions for r in reports) > 0 and sched.total_preemptions > 0
    for i, (p, k) in reqs.items():
        assert done[i].tokens == alone(p, k), f"request {i}"
    emitted = {}
    for r in reports:
        for rid, tok in r.emitted:
            emitted.setdefault(rid, []).append(tok)
    assert all(emitted[i] == done[i].tokens for i in reqs)        # a preempted request never emits a token twice
    assert cache.used_pages() == [0]


def test_preempted_request_is_the_newest_and_returns_to_the_front():
    cache, sched, ex, submit = make(pages=6, page=4, slots=3, max_batched_tokens=64, prefill_chunk=64)
    submit("old", prompt(1, 7), 16)
    submit("new", prompt(2, 7), 16)
    submit("later", prompt(3, 2), 2)
    preempted = None
    for _ in range(40):
        rep = sched.step(ex)
        if rep.preemptions:
            preempted = [s.req.id for s in sched.waiting]
            break
    assert preempted is not None and preempted[0] == "new" and "old" in [s.req.id for s in sched.running]


def test_stop_token_cancel_and_context_limit():
    cache, sched, ex, submit = make(max_ctx=40)
    p = prompt(5, 8)
    full = alone(p, 12)
    stop = full[5]
    submit("s", p, 12, stop_ids=(stop,))
    submit("c", prompt(6, 9), 50 - 19)
    submit("l", prompt(7, 30), 10)             # 30 + 10 = the context limit exactly
    done = {}
    for i in range(200):
        if sched.idle():
            break
        if i == 3:
            f = sched.cancel("c")
            assert f.finish == "cancelled" and cache.has("c") is False
        for f in sched.step(ex).finished:
            done[f.id] = f
    assert done["s"].finish == "stop" and done["s"].tokens == full[:full.index(stop)]
    assert done["l"].finish == "length" and len(done["l"].tokens) == 10
    assert sched.cancel("nobody") is None and cache.used_pages() == [0]


def test_refusals():
    cache, sched, ex, submit = make(pages=8, page=4, max_ctx=64)
    with pytest.raises(Refused, match="empty"):
        sched.submit(Request(1, [], 4))
    with pytest.raises(Refused, match="max_tokens"):
        sched.submit(Request(2, [1], 0))
    with pytest.raises(Refused, match="context limit"):
        sched.submit(Request(3, [1] * 60, 5))
    with pytest.raises(Refused, match="pages"):
        sched.submit(Request(4, [1] * 30, 10))    # 40 tokens need 10 pages, the pool has 8
    sched.submit(Request(5, [1, 2], 2))
    with pytest.raises(Refused, match="already"):
        sched.submit(Request(5, [1, 2], 2))


def test_sampling_rows_carry_the_request_step():
    cache, sched, _, submit = make()
    seen = []

    class Ex(FakeExecutor):
        def execute(self, entries, sampling):
            seen.extend((p.seed, step) for p, step in sampling)
            return super().execute(entries, sampling)
    truth = {}
    ex = Ex(cache, truth)
    sched.submit(Request("a", prompt(1, 4), 3, SamplingParams(temperature=0.5, seed=11)))
    truth["a"] = sched.waiting[0]
    run(sched, ex)
    assert seen == [(11, 0), (11, 1), (11, 2)]


@pytest.mark.parametrize("seed", range(4))
def test_random_load_under_page_pressure(seed):
    """Many requests, few slots and pages (cf. crates/specrt/tests/serving.rs:240-281)."""
    rng = np.random.default_rng(seed)
    cache, sched, ex, submit = make(pages=30, page=4, slots=5, max_batched_tokens=48, prefill_chunk=16, max_ctx=100)
    reqs = {}
    for i in range(24):
        n, k = int(rng.integers(1, 60)), int(rng.integers(1, 40))
        reqs[i] = (prompt(100 * seed + i, n), k)
        submit(i, *reqs[i])
    done, _ = run(sched, ex)
    for i, (p, k) in reqs.items():
        assert done[i].tokens == alone(p, k), f"request {i}"
    assert cache.used_pages() == [0] and cache.free_slots() == 5


# ------------------------------------------------------------------------------------------ steps kept one ahead
def test_steps_one_ahead_give_the_same_tokens_and_waste_nothing_at_max_tokens():
    reqs = {i: (prompt(40 + i, n), k) for i, (n, k) in enumerate([(5, 9), (20, 30), (17, 30), (3, 2), (33, 1)])}
    cache, sched, ex, submit = make(executor=AheadExecutor)
    for i, (p, k) in reqs.items():
        submit(i, p, k)
    done, reports = run(sched, ex)
    for i, (p, k) in reqs.items():
        assert done[i].tokens == alone(p, k) and done[i].finish == "length"
    assert ex.launched > 20 and ex.wasted == 0          # most decode steps went ahead; none ran for a request that had ended by length
    assert all(len(r.emitted) == r.decode_rows for r in reports if r.prefill_tokens == 0)   # every call reports exactly one step
    assert cache.used_pages() == [0] and cache.free_slots() == 8


def test_steps_one_ahead_with_stop_tokens_cancel_and_late_arrivals():
    p0, p1, p2 = prompt(50, 12), prompt(51, 7), prompt(52, 9)
    stop_tok = alone(p0, 8)[5]                          # request 0 stops at its sixth token
    cache, sched, ex, submit = make(executor=AheadExecutor)
    submit(0, p0, 40, stop_ids=(stop_tok,))
    submit(1, p1, 25)
    done = {}
    for step in range(200):
        if sched.idle():
            break
        if step == 9:
            submit(2, p2, 10)                           # arrives while steps are in flight
        if step == 14:
            f = sched.cancel(1)
            assert f is not None and f.finish == "cancelled" and f.tokens == alone(p1, 25)[:len(f.tokens)]
        for f in sched.step(ex).finished:
            done[f.id] = f
        cache.check()
    assert sched.idle()
    assert done[0].finish == "stop" and done[0].tokens == alone(p0, 40, stop=(stop_tok,)) and len(done[0].tokens) == 5
    assert done[2].tokens == alone(p2, 10)
    assert ex.wasted >= 1                               # the step launched before the stop token was seen
    assert cache.used_pages() == [0] and cache.free_slots() == 8


def test_steps_one_ahead_fall_back_when_pages_run_out():
    cache, sched, ex, submit = make(pages=10, page=4, executor=AheadExecutor)
    reqs = {i: (prompt(60 + i, 6), 14) for i in range(3)}      # 3 x 20 tokens = 15 pages > 10: someone is preempted
    for i, (p, k) in reqs.items():
        submit(i, p, k)
    done, reports = run(sched, ex)
    for i, (p, k) in reqs.items():
        assert done[i].tokens == alone(p, k)
    assert sum(r.preemptions for r in reports) >= 1
    assert cache.used_pages() == [0]


def test_pipeline_off_never_launches_ahead():
    cache, sched, ex, submit = make(executor=AheadExecutor, pipeline=False)
    submit(0, prompt(70, 5), 6)
    done, _ = run(sched, ex)
    assert done[0].tokens == alone(prompt(70, 5), 6) and ex.launched == 0


@pytest.mark.parametrize("executor", [FakeExecutor, AheadExecutor])
@pytest.mark.parametrize("seed", range(12))
def test_random_traffic_gives_every_request_its_own_tokens(executor, seed):
    """Requests of random lengths arriving at random steps, some with stop tokens, some cancelled, in a pool small
    enough that requests are preempted: whatever the scheduler does (portions, preemption, steps kept one ahead),
    every request ends with the tokens it would have had alone, and nothing is left held."""
    rng = np.random.default_rng(1000 + seed)
    pages = int(rng.integers(14, 40))
    cache, sched, ex, submit = make(pages=pages, page=4, slots=int(rng.integers(2, 7)), executor=executor,
                                    max_batched_tokens=int(rng.integers(8, 40)), prefill_chunk=int(rng.integers(3, 20)), max_ctx=pages * 4)
    plans, arrivals, cancels = {}, {}, {}
    for rid in range(int(rng.integers(6, 14))):
        n, k = int(rng.integers(1, 30)), int(rng.integers(1, 25))
        if -(-(n + k) // 4) > pages:
            continue
        p = prompt(seed * 100 + rid, n)
        full = alone(p, k)
        stop = (full[int(rng.integers(0, len(full)))],) if rng.random() < 0.3 else ()
        plans[rid] = (p, k, stop)
        arrivals.setdefault(int(rng.integers(0, 40)), []).append(rid)
        if rng.random() < 0.2:
            cancels[rid] = int(rng.integers(0, 80))
    done, cancelled, step = {}, {}, 0
    while step < 5000:
        for rid in arrivals.pop(step, []):
            p, k, stop = plans[rid]
            submit(rid, p, k, stop_ids=stop)
        for rid, at in list(cancels.items()):
            if at == step:
                f = sched.cancel(rid)
                if f is not None:
                    cancelled[rid] = f
                del cancels[rid]
        if sched.idle() and not arrivals:
            break
        for f in sched.step(ex).finished:
            done[f.id] = f
        cache.check()
        step += 1
    assert sched.idle() and not arrivals
    for rid, (p, k, stop) in plans.items():
        want = alone(p, k, stop=stop)
        if rid in cancelled:
            assert cancelled[rid].tokens == alone(p, k)[:len(cancelled[rid].tokens)] and rid not in done
        else:
            assert done[rid].tokens == want, f"request {rid}"
            assert done[rid].finish == ("stop" if len(want) < k else "length")
    assert cache.used_pages() == [0] and cache.free_slots() == cache.max_requests


def test_balanced_portion_fills_whole_rounds_of_tiles():
    """The optional portion size (`Engine(prefill_chunk="auto")`): near 2,048, a multiple of 256, and the one whose
    256 x 256 tiles leave the last round of the 74 CTA pairs fullest (the sizes measured fastest at these shapes)."""
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    shapes = {"8b": [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)], "14b": [(7168, 5120), (5120, 5120), (34816, 5120), (5120, 17408)],
              "32b": [(10240, 5120), (5120, 8192), (51200, 5120), (5120, 25600)]}
    assert {k: G.balanced_portion(v) for k, v in shapes.items()} == {"8b": 2304, "14b": 1792, "32b": 1792}
    for m in shapes.values():
        for nominal in (1024, 2048, 4096):
            T = G.balanced_portion(m, nominal)
            assert T % 256 == 0 and nominal * 3 // 4 <= T <= nominal * 5 // 4
    assert G.balanced_portion([], 2048) == 2048          # nothing to balance: the nominal size
    assert G.balanced_portion([(256, 64)], 2048) == 2560  # one round whatever the size: the most tokens a round


def test_a_product_that_wants_one_sum_is_never_planned_with_a_cut_k_range():
    """The head asks for one finished product (it hands logits on, nobody adds partial sums after it). For a small vocabulary
    and a few hundred tokens the cost model's favourite cuts the k-range; with allow_split=False it must not."""
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    cut = [(T, N, K) for T in (130, 150, 300, 513, 1000) for N, K in ((1500, 1024), (500, 128), (4096, 4096), (151936, 1024))
           if G.plan(T, N, K)[0] == "single" and G.plan(T, N, K)[2] > 1]
    assert (150, 1500, 1024) in cut                       # the case that showed it: 150 tokens, a vocabulary of 1,500
    for T, N, K in cut:
        how = G.plan(T, N, K, allow_split=False)
        assert how[0] == "pair" or how[2] == 1, (T, N, K, how)
