"""Two layers at the layer sizes of Qwen3-8B, 14B and 32B (random weights made on the device): the
bfloat16 path with its tensor-core kernels against the true 32-bit path of the same weights, prompt
portions and decode (groups of 4, 5 and 8 query heads per kv head; 32B: heads * head_dim != hidden)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

QWEN3_8B_2L = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096, intermediate_size=12288,
    num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
    tie_word_embeddings=False, max_position_embeddings=40960, hidden_act="silu", attention_bias=False, torch_dtype="bfloat16")


SHAPES = {
    "8b": QWEN3_8B_2L,
    "14b": dict(QWEN3_8B_2L, hidden_size=5120, intermediate_size=17408, num_attention_heads=40),
    "32b": dict(QWEN3_8B_2L, hidden_size=5120, intermediate_size=25600, num_attention_heads=64),
}


@pytest.mark.parametrize("shape,page", [("8b", 16), ("14b", 64), ("32b", 16)])
def test_bfloat16_against_float32_at_large_layer_sizes(shape, page):
    from inference_bench_b200 import Engine
    from inference_bench_b200.engine.step import StepEntry
    QWEN3_8B_2L = SHAPES[shape]
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, 151936, 300).tolist()
    logits = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(QWEN3_8B_2L, dtype=dtype, max_ctx=512, page_size=page, num_pages=64, max_num_seqs=2, random_weights_seed=0)
        eng.cache.admit("r")
        rows = [eng.runner.step([StepEntry("r", prompt[:257], [0, 100, 256])]).cpu()]         # a portion that crosses query tiles
        rows.append(eng.runner.step([StepEntry("r", prompt[257:299], [41])]).cpu())              # a second portion
        rows.append(eng.runner.step([StepEntry("r", prompt[299:], [0])]).cpu())                  # one decoded token
        logits[dtype] = torch.cat(rows)
        eng.cache.release("r")
        del eng
        torch.cuda.empty_cache()
    ref, got = logits["float32"], logits["bfloat16"]
    assert torch.isfinite(got).all()
    err = (got - ref).abs().max().item() / ref.abs().max().item()
    assert err <= 2e-2, f"bfloat16 differs from float32 by {err:.3e} of max|logit| (worst seen on a B200: 9.4e-3)"
    print(f"{shape} layer sizes, 2 layers: bfloat16 vs float32 worst {err:.3e} of max|logit|")


@pytest.mark.parametrize("shape,page", [("8b", 64), ("32b", 16)])
def test_a_long_portion_in_bfloat16_against_float32(shape, page):
    """A portion of 2,100 tokens (the q/k/v projection then finishes norm, rotation and cache write in its epilogue,
    and every matrix product runs on CTA pairs), a second portion and a decoded token that read what it cached."""
    from inference_bench_b200 import Engine
    from inference_bench_b200.engine.step import StepEntry
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    cfg = SHAPES[shape]
    from inference_bench_b200.engine.runtime import Runtime
    assert G.qkv_in_epilogue(Runtime("cuda:0"), 2100, (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * 128, cfg["hidden_size"])
    prompt = np.random.default_rng(2).integers(0, 151936, 2300).tolist()
    logits = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(cfg, dtype=dtype, max_ctx=2560, page_size=page, num_pages=2560 // page + 4, max_num_seqs=2, random_weights_seed=0)
        eng.cache.admit("r")
        rows = [eng.runner.step([StepEntry("r", prompt[:2100], [0, 1000, 2099])]).cpu()]
        rows.append(eng.runner.step([StepEntry("r", prompt[2100:2299], [198])]).cpu())
        rows.append(eng.runner.step([StepEntry("r", prompt[2299:], [0])]).cpu())
        logits[dtype] = torch.cat(rows)
        eng.cache.release("r")
        del eng
        torch.cuda.empty_cache()
    ref, got = logits["float32"], logits["bfloat16"]
    assert torch.isfinite(got).all()
    err = (got - ref).abs().max().item() / ref.abs().max().item()
    assert err <= 2e-2, f"bfloat16 differs from float32 by {err:.3e} of max|logit| (worst seen on a B200: 9.4e-3)"
    print(f"{shape} layer sizes, 2 layers, 2,100-token portion: bfloat16 vs float32 worst {err:.3e} of max|logit|")


@pytest.mark.parametrize("shape,page,tokens", [("8b", 16, 257), ("32b", 16, 257), ("14b", 64, 321), ("8b", 64, 2100)])
def test_a_prompt_portion_gives_the_same_bits_every_time(shape, page, tokens):
    """Kernels that start while the kernel before them is still running (programmatic dependent launch) must give
    what one kernel after the other gives, run after run: with every query tile released at the same moment, copies
    land late, and a wait in the prefill attention kernel that took a barrier's phase for the one before it showed
    here as a few rows of one layer's attention output that changed from run to run."""
    from inference_bench_b200 import Engine
    from inference_bench_b200.engine.step import StepEntry
    from inference_bench_b200.kernels import lib as L
    lib = L.load()
    prompt = np.random.default_rng(1).integers(0, 151936, tokens).tolist()
    eng = Engine(SHAPES[shape], dtype="bfloat16", max_ctx=max(512, tokens + 64), page_size=page, num_pages=max(64, tokens // page + 4), max_num_seqs=2,
                 random_weights_seed=0)

    def once():
        eng.cache.admit("r")
        out = eng.runner.step([StepEntry("r", prompt, [0, tokens // 3, tokens - 1])])
        eng.cache.release("r")
        return out

    early = eng.rt.options
    assert early.pdl
    eng.rt.options = early.merged(pdl=False)   # a step applies its runtime's options to the library when it starts
    try:
        ref = once()
        assert lib.ib_pdl_enabled() == 0
    finally:
        eng.rt.options = early
    different = sum(not torch.equal(once(), ref) for _ in range(60))
    assert different == 0, f"{different} of 60 runs differ from the run with one kernel after the other"


def test_mixed_steps_give_the_same_bits_every_time():
    """One random schedule of mixed steps (portions of 2 to 257 tokens beside decoded tokens, four requests), replayed
    with one kernel after the other and then eight times with kernels starting early: the same logits, bit for bit."""
    from inference_bench_b200 import Engine
    from inference_bench_b200.engine.step import StepEntry
    from inference_bench_b200.kernels import lib as L
    lib = L.load()
    rng = np.random.default_rng(5)
    names = ["r0", "r1", "r2", "r3"]
    prompts = {k: rng.integers(0, 151936, int(rng.integers(40, 420))).tolist() for k in names}
    done = dict.fromkeys(names, 0)
    steps = []
    while any(done[k] < len(prompts[k]) for k in names):
        entries = []
        for k in names:
            left = len(prompts[k]) - done[k]
            if left == 0 or rng.random() < 0.25:
                continue
            n = 1 if (done[k] > 0 and rng.random() < 0.5) else int(min(left, rng.choice([2, 17, 64, 128, 129, 200, 257])))
            entries.append((k, prompts[k][done[k]:done[k] + n], [n - 1]))
            done[k] += n
        if entries:
            steps.append(entries)
    eng = Engine(SHAPES["8b"], dtype="bfloat16", max_ctx=512, page_size=16, num_pages=128, max_num_seqs=4, random_weights_seed=0)

    def replay():
        for k in names:
            eng.cache.admit(k)
        outs = [eng.runner.step([StepEntry(*e) for e in entries]) for entries in steps]
        for k in names:
            eng.cache.release(k)
        return outs

    early = eng.rt.options
    eng.rt.options = early.merged(pdl=False)
    try:
        ref = replay()
        assert lib.ib_pdl_enabled() == 0
    finally:
        eng.rt.options = early
    for i in range(8):
        got = replay()
        diff = [j for j, (a, b) in enumerate(zip(ref, got)) if not torch.equal(a, b)]
        assert not diff, f"replay {i}: the logits of steps {diff} of {len(steps)} differ from the run with one kernel after the other"


def test_portion_size_chosen_for_the_layer_sizes():
    """prefill_chunk="auto" at the 14B layer sizes: portions of 1,792 tokens, and a prompt cut that way gives the tokens of
    the same prompt cut at 2,048 (greedy, a few tokens: the two ways differ by rounding only)."""
    from inference_bench_b200 import Engine
    prompt = np.random.default_rng(4).integers(0, 151936, 2500).tolist()
    got = {}
    for chunk in ("auto", 2048):
        eng = Engine(SHAPES["14b"], dtype="bfloat16", max_ctx=3072, page_size=64, max_num_seqs=2, prefill_chunk=chunk, random_weights_seed=0)
        if chunk == "auto":
            assert eng.scheduler.cfg.prefill_chunk == 1792
        got[chunk] = eng.generate(prompt, max_tokens=4).tokens
        del eng
        torch.cuda.empty_cache()
    assert len(got["auto"]) == 4 and got["auto"][0] == got[2048][0]
