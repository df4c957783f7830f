"""Schedules and entry points beyond the plain step: decode steps replayed with no host work in between, logits of a
prompt longer than a portion, the status word on the serving path, generation with test-defined parts (state of fixed
size, routing) under CUDA graphs, steps kept one ahead and preemption, and the four ways of cutting the work at sizes
that reach the kernels serving uses (CTA-pair products, the q/k/v epilogue, wide and split forms) against the plain model."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import traces
from plain_qwen3 import PlainModel
from tiny_configs import CONFIGS

pytestmark = pytest.mark.gpu


def _engine(model_dirs, name, dtype, **kw):
    from inference_bench_b200 import Engine
    c = CONFIGS[name]
    kw.setdefault("max_ctx", c["config"]["max_position_embeddings"])
    kw.setdefault("page_size", c["page_size"])
    return Engine(model_dirs[name], dtype=dtype, **kw)


# ------------------------------------------------------------------------------------------ decode steps with no host work between
def _prefill(eng, prompts, sampling):
    """Each prompt whole through the step function; returns the requests' ids and their first tokens."""
    from inference_bench_b200.engine.step import StepEntry
    ids, first = [], []
    for i, (p, sp) in enumerate(zip(prompts, sampling)):
        rid = ("ahead", i)
        eng.cache.admit(rid)
        logits = eng.runner.step([StepEntry(rid, p, [len(p) - 1])])
        first.append(int(eng.executor.sampler.sample(logits, [sp], [0])[0].item()))
        ids.append(rid)
    return ids, first


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("rows,k", [(1, 64), (3, 17), (8, 64), (3, 1)])
@pytest.mark.parametrize("sampled", [False, True])
def test_decode_ahead_matches_plain_and_step_by_step(model_dirs, name, rows, k, sampled):
    """`decode_ahead` (a captured decode step replayed k times, tokens, positions and sampling steps advanced on the
    device) against the plain model's own generation in float32, against the same engine decoding step by step through
    `execute`, in float32 and bfloat16; and what the cache holds afterwards."""
    from inference_bench_b200 import SamplingParams
    from inference_bench_b200.engine.step import StepEntry
    vocab = CONFIGS[name]["config"]["vocab_size"]
    page = CONFIGS[name]["page_size"]
    plain = PlainModel(model_dirs[name])
    prompts = [traces.prompt(800 + i, n, vocab) for i, n in zip(range(rows), (11, 3, 37, 1, 20, 8, 29, 16))]
    sampling = [SamplingParams(temperature=0.9, seed=50 + i, top_k=12) if sampled else SamplingParams() for i in range(rows)]
    for dtype in ("float32", "bfloat16"):
        got = {}
        for how in ("ahead", "steps"):
            eng = _engine(model_dirs, name, dtype)
            ids, first = _prefill(eng, prompts, sampling)
            if how == "ahead":
                out = eng.executor.decode_ahead([StepEntry(r, [t], [0]) for r, t in zip(ids, first)], [(sp, 1) for sp in sampling], k)
            else:
                out, last = [], first
                for j in range(k):
                    last = eng.executor.execute([StepEntry(r, [t], [0]) for r, t in zip(ids, last)], [(sp, 1 + j) for sp in sampling])
                    out.append(list(last))
            got[how] = [[first[i]] + [row[i] for row in out] for i in range(rows)]
            for i, rid in enumerate(ids):
                n = len(prompts[i]) + k
                assert eng.cache.length(rid) == n
                table = eng.cache.table(0, rid)
                assert (table[:-(-n // page)] >= 0).all() and (table[-(-n // page):] < 0).all()
                eng.cache.release(rid)
            eng.cache.check()
            assert eng.cache.used_pages() == [0] * len(eng.cache.groups)
            eng.rt.check_status()
        assert got["ahead"] == got["steps"], f"{dtype}: replaying the captured step differs from decoding step by step"
        if dtype == "float32":
            for i, (p, sp) in enumerate(zip(prompts, sampling)):
                want = plain.sample(p, k + 1, sp.temperature, sp.seed, sp.top_k) if sampled else plain.greedy(p, k + 1)
                assert got["ahead"][i] == want, f"request {i}"


# ------------------------------------------------------------------------------------------ Engine.logits
@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16"), ("C", "float32")])
def test_engine_logits_cuts_a_long_prompt_itself(model_dirs, name, dtype):
    vocab = CONFIGS[name]["config"]["vocab_size"]
    eng = _engine(model_dirs, name, dtype, prefill_chunk=7)
    p = traces.prompt(61, 45, vocab)
    got = eng.logits(p)
    want = PlainModel(model_dirs[name]).logits(p)
    assert got.shape == want.shape and got.dtype == torch.float32
    tol = {"float32": 1e-4, "bfloat16": 3e-2}[dtype]
    assert (got - want).abs().max() <= tol * want.abs().max()
    eng.cache.check()
    assert eng.cache.used_pages() == [0] * len(eng.cache.groups) and eng.cache.free_slots() == eng.cache.max_requests
    # and generation still works beside it
    assert len(eng.generate(p[:9], max_tokens=3).tokens) == 3


# ------------------------------------------------------------------------------------------ the status word on the serving path
@pytest.mark.parametrize("graphs,pipeline", [(True, True), (True, False), (False, False)])
def test_engine_step_raises_when_a_kernel_reports_a_fault(model_dirs, graphs, pipeline):
    """A block table entry that goes bad under a running request (made from the host here): the kernels skip the page
    and set the status word, and the caller of Engine.step gets an error with the step's tokens, not garbage tokens."""
    from inference_bench_b200.engine.runtime import DeviceStatusError
    name = "D"
    vocab = CONFIGS[name]["config"]["vocab_size"]
    eng = _engine(model_dirs, name, "bfloat16", use_graphs=graphs, pipeline=pipeline)
    rid = eng.submit(traces.prompt(5, 40, vocab), max_tokens=30)
    for _ in range(4):
        eng.step()
    slot = eng.cache.slot(rid)
    saved = [int(t[slot, 0]) for t in eng.cache._tables]
    for t in eng.cache._tables:
        t[slot, 0] = 10 ** 6       # (an entry of -1 would be filled with a fresh page by the cache manager's next extend)
    try:
        with pytest.raises(DeviceStatusError, match="block table"):
            for _ in range(4):
                eng.step()
    finally:
        for t, page in zip(eng.cache._tables, saved):
            t[slot, 0] = page
    assert int(eng.rt.status.item()) == 0      # the word is cleared when it is reported


# ------------------------------------------------------------------------------------------ test-defined parts through generation
def _greedy_by(logits_fn, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        row = logits_fn(seq)[-1]
        seq.append(int(np.flatnonzero(row == row.max())[0]))
    return seq[len(prompt):]


@pytest.mark.parametrize("toy", ["state", "routed"])
def test_toy_architectures_generate_under_graphs_pipelining_and_preemption(tmp_path, toy):
    """The two architectures that tests/test_parts_gpu.py registers (a mixer with per-request state of fixed size, a layer
    run twice, a layer reading another's cache; a routed feed-forward and a position encoding of its own) through
    Engine.generate: CUDA graphs, steps kept one ahead, several requests, and a pool so small that requests are
    preempted and recomputed, which must restart their state from zero. Float32, so tokens equal the plain toy's."""
    import test_parts_gpu as T
    from inference_bench_b200 import Engine
    from inference_bench_b200.weights.random_init import write_random_model
    if toy == "state":
        T._register_toy()
        folder = write_random_model(T.TOY, 5, tmp_path / "toy", std=0.08)
        vocab, plain = 130, lambda seq: T._toy_plain_logits(folder, seq)
    else:
        T._register_routed_toy()
        folder = write_random_model(T.ROUTED, 17, tmp_path / "routed", std=0.12)
        vocab, plain = 97, lambda seq: T._routed_plain_logits(folder, seq)[0]
    lens, news = [3, 30, 12, 45, 8, 26], [20, 9, 25, 12, 30, 15]
    prompts = [traces.prompt(900 + i, n, vocab) for i, n in enumerate(lens)]
    want = [_greedy_by(plain, p, n) for p, n in zip(prompts, news)]
    for graphs, pipeline, pages in ((True, True, 64), (True, True, 9), (False, False, 9)):
        eng = Engine(folder, dtype="float32", max_ctx=128, page_size=8, num_pages=pages, max_num_seqs=3, prefill_chunk=16, use_graphs=graphs,
                     pipeline=pipeline)
        from inference_bench_b200.engine.scheduler import Request
        for i, (p, n) in enumerate(zip(prompts, news)):
            eng.scheduler.submit(Request(i, p, n))
        done, preempted = {}, 0
        while not eng.scheduler.idle():
            rep = eng.scheduler.step(eng.executor)
            preempted += rep.preemptions
            for f in rep.finished:
                done[f.id] = f.tokens
        eng.rt.check_status()
        eng.cache.check()
        assert (preempted > 0) == (pages == 9), f"{preempted} preemptions with {pages} pages"
        for i in range(len(prompts)):
            assert done[i] == want[i], f"graphs={graphs} pipeline={pipeline} pages={pages}: request {i}"
        assert eng.cache.used_pages() == [0] * len(eng.cache.groups) and eng.cache.free_slots() == 3


# ------------------------------------------------------------------------------------------ the four cuts at serving sizes
SERVING = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1500, hidden_size=1024, intermediate_size=2816,
               num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
               tie_word_embeddings=False, max_position_embeddings=4096, hidden_act="silu", attention_bias=False, torch_dtype="bfloat16")
SERVING_LENGTHS = {"a": 150, "b": 300, "c": 2100, "d": 513, "e": 40}
# Largest |engine - plain| / max|logit| allowed in bfloat16 at these sizes, per cut: about twice the worst value seen on a B200
# (whole 9.1e-3, tail 8.7e-3, portions 9.1e-3, mixed 8.5e-3; float32: 1.2e-5 in every cut).
SERVING_BF16 = {"whole": 2e-2, "tail": 2e-2, "portions": 2e-2, "mixed": 2e-2}


@pytest.fixture(scope="module")
def serving(tmp_path_factory):
    from inference_bench_b200.weights.random_init import write_random_model
    folder = write_random_model(SERVING, 11, tmp_path_factory.mktemp("serving"))      # N(0, 0.02), norms 1 + U(-0.1, 0.1): the benchmark's distributions
    reqs = {r: traces.prompt(700 + i, n, SERVING["vocab_size"]) for i, (r, n) in enumerate(SERVING_LENGTHS.items())}
    plain = PlainModel(folder)
    return folder, reqs, {r: plain.logits(t).numpy() for r, t in reqs.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_cuts_at_serving_sizes_match_plain(serving, dtype, cut):
    """Width 1,024, head size 128, prompts up to 2,100 tokens: whole prompts reach the CTA-pair products with the residual
    add and the q/k/v epilogue (2,048 tokens and more), portions of 257, 129, 64 and 2 tokens the forms the cost model picks
    between, the register form of the norm (256 rows and more) and the fused gate/up product on pairs; the mixed trace puts
    portions of 129 to 300 tokens beside decoded tokens in a pool sized to the live peak, so pages are used again."""
    from inference_bench_b200.trace import build_runner
    folder, reqs, want = serving
    steps = {"whole": lambda r: traces.whole(r), "tail": lambda r: traces.tail_one_by_one(r),
             "portions": lambda r: traces.portions(r, sizes=(257, 129, 64, 2)),
             "mixed": lambda r: traces.mixed(r, seed=2, decode_tail=20, sizes=(129, 300, 257, 2, 64))}[cut](reqs)
    max_tokens = traces.max_live_tokens(steps)
    runner = build_runner(folder, dtype, max_tokens, page_size=16)
    got = traces.run_steps(runner, steps)
    tol = 1e-4 if dtype == "float32" else SERVING_BF16[cut]
    worst = 0.0
    for (r, pos), row in got.items():
        err = np.abs(row - want[r][pos]).max() / np.abs(want[r]).max()
        assert err <= tol, f"{cut}/{dtype}: request {r} position {pos}: |diff| = {err:.3e} of max|logit| (allowed {tol:.1e})"
        worst = max(worst, err)
    assert len(got) == sum(len(t) for t in reqs.values())
    runner.cache.check()
    assert runner.cache.used_pages() == [0]
    print(f"serving/{dtype}/{cut}: worst {worst:.3e} of max|logit|, pool {max_tokens} tokens, {len(steps)} steps")


def test_serving_sizes_reach_the_serving_kernels(serving, monkeypatch):
    """The cuts above are only worth something if they run the kernels they are meant for: count the entry points."""
    from inference_bench_b200.kernels import lib as L
    from inference_bench_b200.trace import build_runner
    folder, reqs, _ = serving
    called: dict = {}
    real = L.call
    monkeypatch.setattr(L, "call", lambda name, *a: (called.__setitem__(name, called.get(name, 0) + 1), real(name, *a))[1])
    steps = traces.whole({"c": reqs["c"]}) + traces.portions({"b": reqs["b"]}, sizes=(257, 43)) + traces.tail_one_by_one({"e": reqs["e"]}, tail=2)
    for s in steps:
        s["step"] = 0
    runner = build_runner(folder, "bfloat16", 4096, page_size=16)
    traces.run_steps(runner, steps)
    for name in ("ib_gemm_qkv_tcgen05_2cta", "ib_gemm_tcgen05_2cta_add", "ib_gemm_swiglu_tcgen05_2cta", "ib_gemm_tcgen05", "ib_attention_prefill_ws",
                 "ib_attention_decode_fused", "ib_add_rmsnorm"):
        assert called.get(name, 0) > 0, f"{name} never ran: {sorted(called)}"


def test_runtime_options_reach_the_engine(model_dirs):
    """Options given to the entry point are the ones the runtime carries, and an engine with everything optional switched off
    (no graphs, no pipeline, no early launches, no fused forms, NVTX ranges on) generates the plain model's tokens."""
    from inference_bench_b200.config.runtime_options import RuntimeOptions
    name = "D"
    vocab = CONFIGS[name]["config"]["vocab_size"]
    p = traces.prompt(12, 70, vocab)
    want = PlainModel(model_dirs[name]).greedy(p, 6)
    off = RuntimeOptions(graphs=False, pipeline=False, pdl=False, fuse=False, nvtx=True, decode_attention="split", prefill_attention="tcgen05")
    eng = _engine(model_dirs, name, "float32", options=off)
    assert eng.rt.options.pdl is False and eng.rt.options.dtype == "float32" and eng.rt.options.page_size == CONFIGS[name]["page_size"]
    assert eng.executor.use_graphs is False and eng.scheduler.cfg.pipeline is False
    assert eng.generate(p, max_tokens=6).tokens == want
    eng16 = _engine(model_dirs, name, "bfloat16", options={"fuse": False, "decode_attention": "split", "prefill_attention": "tcgen05", "nvtx": True})
    on16 = _engine(model_dirs, name, "bfloat16")
    a, b = eng16.logits(p), on16.logits(p)
    assert (a - b).abs().max() <= 2e-2 * b.abs().max() and not torch.equal(a, b)      # other kernels, the same model


@pytest.mark.parametrize("name,seed", [("B", 0), ("C", 1)])
def test_random_traffic_matches_plain(model_dirs, name, seed):
    """Requests that arrive at random steps with random lengths, greedy and seeded sampling, stop tokens, a few cancelled in
    flight, a pool so small that requests are preempted and recomputed; CUDA graphs and steps kept one ahead. Float32: what
    every request generated equals what the plain model generates for it alone (a cancelled one: a prefix of it)."""
    from inference_bench_b200 import SamplingParams
    from inference_bench_b200.engine.scheduler import Request
    rng = np.random.default_rng(seed)
    vocab = CONFIGS[name]["config"]["vocab_size"]
    page = CONFIGS[name]["page_size"]
    plain = PlainModel(model_dirs[name])
    n_req = 18
    reqs = []
    for i in range(n_req):
        p = traces.prompt(1000 + 31 * seed + i, int(rng.integers(1, 12) if rng.random() < 0.6 else rng.integers(12, 60)), vocab)   # short prompts are admitted side by side
        new = int(rng.integers(1, 40))                                                                                          # ... and then outgrow the pool
        sp = SamplingParams() if rng.random() < 0.5 else SamplingParams(temperature=float(rng.choice([0.7, 1.1])), seed=int(rng.integers(0, 10 ** 6)), top_k=int(rng.choice([0, 5, 40])))
        full = plain.greedy(p, new) if sp.temperature == 0 else plain.sample(p, new, sp.temperature, sp.seed, sp.top_k)
        stop = ()
        if len(full) > 4 and rng.random() < 0.4:
            stop = (int(full[int(rng.integers(2, len(full)))]),)
        want = full[:full.index(stop[0])] if stop and stop[0] in full else full
        reqs.append(dict(prompt=p, new=new, sp=sp, stop=stop, want=want, arrive=int(rng.integers(0, 40)), cancel=(int(rng.integers(3, 30)) if rng.random() < 0.2 else None)))
    longest = max(len(r["prompt"]) + r["new"] for r in reqs)
    eng = _engine(model_dirs, name, "float32", max_ctx=128, num_pages=-(-longest // page) + 2, max_num_seqs=4, prefill_chunk=16, max_batched_tokens=40)
    got, finish, born = {i: [] for i in range(n_req)}, {}, {}
    preempted, step = 0, 0
    while len(finish) < n_req and step < 4000:
        for i, r in enumerate(reqs):
            if r["arrive"] == step:
                eng.scheduler.submit(Request(i, r["prompt"], r["new"], r["sp"], r["stop"]))
                born[i] = step
        for i, r in enumerate(reqs):
            if r["cancel"] is not None and i in born and i not in finish and step == born[i] + r["cancel"]:
                f = eng.cancel(i)
                if f is not None:
                    finish[i] = "cancelled"
                    got[i] = list(f.tokens)
        rep = eng.step()
        preempted += rep.preemptions
        for rid, tok in rep.emitted:
            if rid not in finish:
                got[rid].append(tok)
        for f in rep.finished:
            finish[f.id] = f.finish
            assert got[f.id] == list(f.tokens), f"request {f.id}: the emitted tokens and the finished record differ"
        eng.cache.check()
        step += 1
    assert len(finish) == n_req, f"{n_req - len(finish)} requests never finished"
    assert preempted > 0, "the pool was meant to be too small"
    eng.rt.check_status()
    for i, r in enumerate(reqs):
        if finish[i] == "cancelled":
            assert got[i] == r["want"][:len(got[i])], f"request {i} (cancelled)"
        else:
            assert got[i] == r["want"], f"request {i} ({finish[i]}; preemptions so far {preempted})"
            assert finish[i] == ("stop" if r["stop"] and len(r["want"]) < r["new"] else "length")
    assert eng.cache.used_pages() == [0] * len(eng.cache.groups) and eng.cache.free_slots() == 4
