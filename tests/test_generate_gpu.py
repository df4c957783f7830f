"""Generation through the Python entry point against the plain implementation: greedy and seeded
temperature sampling, batches, CUDA-graph decode, and preemption when pages run out."""
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


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_matches_plain_fp32(model_dirs, name, graphs):
    vocab = CONFIGS[name]["config"]["vocab_size"]
    plain = PlainModel(model_dirs[name])
    eng = _engine(model_dirs, name, "float32", use_graphs=graphs)
    prompts = [traces.prompt(7 + i, n, vocab) for i, n in enumerate((7, 19, 33))]
    want = [plain.greedy(p, 8) for p in prompts]
    # one by one
    for p, w in zip(prompts, want):
        r = eng.generate(p, max_tokens=8)
        assert r.tokens == w and r.finish == "length" and r.prompt_tokens == len(p) and r.completion_tokens == 8
    # all together (a batch of decode rows, prompts cut into portions beside them)
    eng2 = _engine(model_dirs, name, "float32", use_graphs=graphs, prefill_chunk=5, max_batched_tokens=12)
    got = eng2.generate(prompts, max_tokens=8)
    assert [r.tokens for r in got] == want
    assert eng2.cache.used_pages() == [0] * len(eng2.cache.groups)
    eng2.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_seeded_sampling_matches_plain_fp32(model_dirs, name):
    from inference_bench_b200 import SamplingParams
    vocab = CONFIGS[name]["config"]["vocab_size"]
    plain = PlainModel(model_dirs[name])
    eng = _engine(model_dirs, name, "float32", prefill_chunk=3)
    prompts = [traces.prompt(40 + i, n, vocab) for i, n in enumerate((1, 12, 40, 65))]
    sp = [SamplingParams(temperature=0.8, seed=100 + i) for i in range(len(prompts))]
    got = eng.generate(prompts, max_tokens=6, sampling=sp)
    for p, s, r in zip(prompts, sp, got):
        assert r.tokens == plain.sample(p, 6, s.temperature, s.seed)
    # the same seed gives the same tokens, another seed other tokens
    again = eng.generate(prompts[2], max_tokens=6, sampling=sp[2])
    other = eng.generate(prompts[2], max_tokens=6, sampling=SamplingParams(temperature=0.8, seed=999))
    assert again.tokens == got[2].tokens and other.tokens != got[2].tokens
    # filters
    f = SamplingParams(temperature=1.3, seed=5, top_k=7, top_p=0.8, min_p=0.02)
    r = eng.generate(prompts[1], max_tokens=6, sampling=f)
    assert r.tokens == plain.sample(prompts[1], 6, f.temperature, f.seed, f.top_k, f.top_p, f.min_p)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_bfloat16_stays_within_rounding_of_plain(model_dirs, name):
    """bfloat16 may pick another token only where the plain logits of the two are within rounding."""
    vocab = CONFIGS[name]["config"]["vocab_size"]
    plain = PlainModel(model_dirs[name])
    eng = _engine(model_dirs, name, "bfloat16")
    for i, n in enumerate((5, 21, 50)):
        p = traces.prompt(70 + i, n, vocab)
        r = eng.generate(p, max_tokens=12)
        seq = p + r.tokens
        lg = plain.logits(seq).numpy()
        for j, tok in enumerate(r.tokens):
            row = lg[len(p) + j - 1]
            assert row.max() - row[tok] <= 2 * 3e-2 * np.abs(lg).max(), f"token {j}: plain prefers another token by {row.max() - row[tok]:.3e}"


def test_long_decoding_fp32_and_first_tokens(model_dirs):
    """A one-token prompt decoded far past several pages, against the plain implementation."""
    name = "B"
    vocab = CONFIGS[name]["config"]["vocab_size"]
    plain = PlainModel(model_dirs[name])
    eng = _engine(model_dirs, name, "float32")
    p = traces.prompt(3, 1, vocab)
    r = eng.generate(p, max_tokens=150)
    assert r.tokens == plain.greedy(p, 150)


def test_preemption_when_pages_run_out_gives_the_same_tokens(model_dirs):
    """So few pages that running requests must be preempted and recomputed; every output still
    equals the request run alone, and no page is left behind."""
    name = "A"
    vocab = CONFIGS[name]["config"]["vocab_size"]
    plain = PlainModel(model_dirs[name])
    lens = [3, 30, 12, 45, 8, 26, 17, 40]
    news = [20, 9, 25, 12, 30, 15, 22, 10]
    prompts = [traces.prompt(200 + i, n, vocab) for i, n in enumerate(lens)]
    eng = _engine(model_dirs, name, "float32", num_pages=9, max_num_seqs=4, prefill_chunk=16)
    from inference_bench_b200.engine.scheduler import Request
    for i, (p, n) in enumerate(zip(prompts, news)):
        eng.scheduler.submit(Request(i, p, n))
    done = {}
    preempted = 0
    while not eng.scheduler.idle():
        rep = eng.scheduler.step(eng.executor)
        preempted += rep.preemptions
        for f in rep.finished:
            done[f.id] = f.tokens
        eng.cache.check()
    eng.rt.check_status()
    assert preempted > 0, "the test must exercise preemption"
    for i, (p, n) in enumerate(zip(prompts, news)):
        assert done[i] == plain.greedy(p, n), f"request {i}"
    assert eng.cache.used_pages() == [0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_kept_one_ahead_change_no_token(model_dirs, dtype):
    """Decode steps launched before the tokens of the step before are read back (the default) against
    the same engine with that off: greedy and seeded sampling, different lengths, a stop token in the
    middle of the run, a request that arrives later."""
    from inference_bench_b200 import SamplingParams
    name = "B"
    vocab = CONFIGS[name]["config"]["vocab_size"]
    prompts = [traces.prompt(90 + i, n, vocab) for i, n in enumerate((9, 21, 4, 30))]
    sp = [SamplingParams(), SamplingParams(temperature=0.9, seed=3), SamplingParams(temperature=1.2, seed=4, top_k=20), SamplingParams()]
    outs = {}
    for pipeline in (False, True):
        eng = _engine(model_dirs, name, dtype, pipeline=pipeline)
        free = eng.generate(prompts, max_tokens=24, sampling=sp)
        stop = free[0].tokens[10]                                # request 0 then stops at its 11th token at the latest
        first = free[0].tokens.index(stop)
        stopped = eng.generate(prompts, max_tokens=24, sampling=sp, stop_ids=[stop])
        assert stopped[0].finish == "stop" and stopped[0].tokens == free[0].tokens[:first]
        # submit / step by hand: a request that arrives while two steps are in flight
        a = eng.submit(prompts[1], max_tokens=12, sampling=sp[1])
        got = {a: []}
        for i in range(60):
            if i == 5:
                b = eng.submit(prompts[3], max_tokens=7)
                got[b] = []
            rep = eng.step()
            for rid, tok in rep.emitted:
                got[rid].append(tok)
            if eng.scheduler.idle():
                break
        if dtype == "float32":                                   # bfloat16 may round differently in another batch
            assert got[a] == free[1].tokens[:12] and got[b] == free[3].tokens[:7]
        assert len(got[a]) == 12 and len(got[b]) == 7
        eng.rt.check_status()
        eng.cache.check()
        assert eng.cache.used_pages() == [0] * len(eng.cache.groups)
        outs[pipeline] = ([r.tokens for r in free], [r.tokens for r in stopped], [r.finish for r in stopped], got[a], got[b])
    assert outs[True] == outs[False]
