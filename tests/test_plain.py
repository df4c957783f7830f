"""The plain implementation itself: properties that follow from the formulas it cites (no GPU).

The reference's model code cannot be built here (Rust emitting CUDA for NVRTC, no CPU path), so
there is no golden output from it under tests/golden/: these checks and the cited formulas are what
the oracle rests on."""
import math

import numpy as np
import torch

import plain_qwen3 as P
import traces
from tiny_configs import CONFIGS


def test_rmsnorm_and_swiglu_formulas():
    x = torch.tensor([[3.0, -4.0]])
    w = torch.tensor([2.0, 0.5])
    y = P.rmsnorm(x, w, 0.0)
    assert torch.allclose(y, torch.tensor([[2 * 3 / math.sqrt(12.5), 0.5 * -4 / math.sqrt(12.5)]]))
    ws = {"m.gate_proj.weight": torch.eye(2), "m.up_proj.weight": 2 * torch.eye(2), "m.down_proj.weight": torch.eye(2)}
    out = P.swiglu(torch.tensor([[1.0, -2.0]]), ws, "m.")
    assert torch.allclose(out, torch.tensor([[1 / (1 + math.exp(-1)) * 2, -2 / (1 + math.exp(2)) * -4]]))


def test_rope_is_a_rotation_that_depends_on_relative_position():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 24, generator=g, dtype=torch.float64)
    k = torch.randn(1, 1, 24, generator=g, dtype=torch.float64)
    def dot(pq, pk):
        return float((P.rope_neox(q, torch.tensor([pq]), 1e4) * P.rope_neox(k, torch.tensor([pk]), 1e4)).sum())
    assert abs(dot(5, 3) - dot(105, 103)) < 1e-9 and abs(dot(5, 3) - dot(5, 4)) > 1e-6
    assert torch.allclose(P.rope_neox(q, torch.tensor([0]), 1e4), q)
    assert abs(float(P.rope_neox(q, torch.tensor([77]), 1e4).norm() - q.norm())) < 1e-9
    # pair (d, d + half): with only dim 0 set, position 1 moves it into dims 0 and 12 by cos(1), sin(1)
    e = torch.zeros(1, 1, 24, dtype=torch.float64)
    e[..., 0] = 1
    r = P.rope_neox(e, torch.tensor([1]), 1e4)[0, 0]
    assert abs(r[0] - math.cos(1)) < 1e-12 and abs(r[12] - math.sin(1)) < 1e-12


def test_attention_mask_and_groups():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(9, h, 8, generator=g, dtype=torch.float64) for h in (4, 2, 2))
    full = P.attention_scores(q, k, v).reshape(9, 4, 8)
    assert torch.allclose(full[0], v[0].repeat_interleave(2, dim=0))          # the first token sees only itself; heads 0,1 -> kv head 0
    win = P.attention_scores(q, k, v, window=3).reshape(9, 4, 8)
    assert torch.allclose(win[:3], full[:3]) and not torch.allclose(win[5], full[5])
    k2 = k.clone()
    k2[1] += 100.0                                                             # outside the window of the last token: no effect there
    assert torch.allclose(P.attention_scores(q, k2, v, window=3)[-1], win.reshape(9, -1)[-1])


def test_causality_and_window_of_the_whole_model(model_dirs):
    for name in ("A", "C"):
        m = P.PlainModel(model_dirs[name])
        vocab = CONFIGS[name]["config"]["vocab_size"]
        t = traces.prompt(1, 40, vocab)
        a = m.logits(t)
        t2 = list(t)
        t2[30] = (t2[30] + 1) % vocab
        b = m.logits(t2)
        assert torch.equal(a[:30], b[:30]) and not torch.equal(a[30:], b[30:])
        assert m.greedy(t, 3) == m.greedy(t, 3) and len(m.greedy(t, 3)) == 3


def test_sampling_rules():
    row = torch.tensor([0.0, 3.0, 3.0, 1.0, -2.0])
    assert P.sample_token(row, 0.0, 0, 0) == 1                                 # the lowest index wins a tie
    picks = {P.sample_token(row, 1.0, seed, 0, top_k=2) for seed in range(200)}
    assert picks == {1, 2}
    picks = {P.sample_token(row, 1.0, seed, 0, top_p=0.5) for seed in range(200)}
    assert picks <= {1, 2}
    picks = {P.sample_token(row, 1.0, seed, 0, min_p=0.2) for seed in range(300)}
    assert picks == {1, 2}                                                      # exp(1 - 3) = 0.135 < 0.2
    many = [P.sample_token(row, 1.0, 3, step) for step in range(3000)]
    freq = np.bincount(many, minlength=5) / 3000
    want = torch.softmax(row, 0).numpy()
    assert np.abs(freq - want).max() < 0.03                                     # Gumbel-max samples the softmax
    assert P.sample_token(row, 1.0, 3, 7) == P.sample_token(row, 1.0, 3, 7)
