"""The parts the Qwen3 dense decoder is made of, each parametrized by its own sizes and constants.

Formulas follow v0l/inference-bench's `specrt`; the file:line beside each class names where the
reference computes the same thing.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from . import base
from .base import FixedState, PagedKV, WeightSpec


# ------------------------------------------------------------------------------------------ norm
@base.register_norm("rmsnorm")
class RMSNorm(base.Norm):
    """y = w * (x * rsqrt(mean(x^2) + eps)), float32 arithmetic, fused with the residual add that
    precedes it (crates/kir/tests/golden/rmsnorm_sm120.cu:19-29; no unit offset for this family,
    crates/specrt/src/weights.rs:877-880)."""

    def __init__(self, name: str, size: int, eps: float):
        self.name, self.size, self.eps = name, size, eps
        self.w: Optional[torch.Tensor] = None

    def weight_specs(self):
        return [WeightSpec(self.name, (self.size,), role="norm")]

    def bind(self, weights, rt):
        self.w = rt.vector(weights[self.name])

    def forward(self, ctx, x, delta, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.rt.empty((n, self.size))
        ops.add_rmsnorm(x, delta, self.w, out, self.eps, rows)
        return out


# ------------------------------------------------------------------------------------------ position
@base.register_position_encoding("rope")
class RotaryEmbedding(base.PositionEncoding):
    """Half-rotation ("NeoX") rotary encoding over the first `rotary_dim` dims of a head:
    inv_freq_i = theta^(-2i/rotary_dim), angle = float(pos) * inv_freq_i in float32
    (crates/kir/tests/golden/attention/RopeKvWrite_bf16x2_sm120.cu:32-35, 200-206)."""

    def __init__(self, rotary_dim: int, theta: float):
        if rotary_dim % 2:
            raise ValueError(f"rotary_dim {rotary_dim} must be even")
        self.rotary_dim, self.theta = rotary_dim, theta
        self.inv_freq: Optional[torch.Tensor] = None

    def bind(self, weights, rt):
        i = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
        self.inv_freq = rt.upload((1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), i / self.rotary_dim)).to(torch.float32))

    def tables(self, ctx):
        key = ("rope", self.rotary_dim, self.theta)
        if key not in ctx.memo:
            half = self.rotary_dim // 2
            cos = ctx.rt.empty((ctx.n_tokens, half), torch.float32)
            sin = ctx.rt.empty((ctx.n_tokens, half), torch.float32)
            ops.rope_table(ctx.positions, self.inv_freq, cos, sin)
            ctx.memo[key] = (cos, sin)
        return ctx.memo[key]


@base.register_position_encoding("none")
class NoPositionEncoding(base.PositionEncoding):
    def __init__(self):
        pass

    def tables(self, ctx):
        return None, None


# ------------------------------------------------------------------------------------------ mixer
@base.register_mixer("attention")
class Attention(base.Mixer):
    """Causal grouped-query attention over a paged cache, with optional per-head RMSNorm of q and k
    before the rotation and an optional window.

    qkv = Wqkv h (q, k, v rows concatenated at load: crates/specrt/src/weights.rs:886-953);
    per-head norm then RoPE (crates/kir/src/cuda/attention/common.rs:49-96);
    s = q.k / sqrt(head_dim), keys visible when key <= pos and, with a window W, key > pos - W
    (crates/kir/src/cuda/attention/flash_mma.rs:193); out = Wo (softmax(s) v).
    With own_kv=False the layer has only a q projection and reads the cache it is given."""

    def __init__(self, prefix: str, hidden: int, heads: int, kv_heads: int, head_dim: int, qk_norm: bool, norm_eps: float,
                 position: base.PositionEncoding, window: Optional[int] = None, own_kv: bool = True, scale: Optional[float] = None):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        self.prefix, self.hidden, self.heads, self.kv_heads, self.head_dim = prefix, hidden, heads, kv_heads, head_dim
        self.qk_norm, self.norm_eps, self.position, self.window, self.own_kv = qk_norm, norm_eps, position, window, own_kv
        self.scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)  # crates/specrt/src/codegen.rs:147
        self.wqkv = self.wo = self.q_norm = self.k_norm = None

    def cache_need(self):
        return PagedKV(self.kv_heads, self.head_dim, self.window) if self.own_kv else None

    def weight_specs(self):
        p, hd = self.prefix, self.head_dim
        specs = [WeightSpec(f"{p}.q_proj.weight", (self.heads * hd, self.hidden)), WeightSpec(f"{p}.o_proj.weight", (self.hidden, self.heads * hd))]
        if self.own_kv:
            specs += [WeightSpec(f"{p}.k_proj.weight", (self.kv_heads * hd, self.hidden)), WeightSpec(f"{p}.v_proj.weight", (self.kv_heads * hd, self.hidden))]
        if self.qk_norm:
            specs.append(WeightSpec(f"{p}.q_norm.weight", (hd,), role="norm"))
            if self.own_kv:
                specs.append(WeightSpec(f"{p}.k_norm.weight", (hd,), role="norm"))
        return specs

    def bind(self, weights, rt):
        p = self.prefix
        rows = [weights[f"{p}.q_proj.weight"]]
        if self.own_kv:
            rows += [weights[f"{p}.k_proj.weight"], weights[f"{p}.v_proj.weight"]]
        else:  # keep the [q | k | v] row layout the kernels read; the k and v rows are never used
            z = torch.zeros((2 * self.kv_heads * self.head_dim, self.hidden), dtype=rows[0].dtype, device=rows[0].device)
            rows.append(z)
        self.wqkv = rt.matrix(torch.cat(rows, dim=0))
        self.wo = rt.matrix(weights[f"{p}.o_proj.weight"])
        if self.qk_norm:
            self.q_norm = rt.vector(weights[f"{p}.q_norm.weight"])
            if self.own_kv:
                self.k_norm = rt.vector(weights[f"{p}.k_norm.weight"])
        self.position.bind(weights, rt)

    adds_to_residual = True   # the output projection may add to the residual stream in its epilogue

    def forward(self, ctx, h, cache, residual=None):
        rt = ctx.rt
        cos, sin = self.position.tables(ctx)
        from ..kernels import attention
        q = attention.project_qkv(ctx, h, self.wqkv, self.q_norm, self.k_norm, self.norm_eps, cos, sin, cache, self.heads, self.own_kv)
        if q is not None:   # many tokens: norm, rotation and cache write happened in the projection's epilogue
            out = attention.paged_attention(ctx, q, cache, self.heads, self.window, self.scale)
            return rt.linear(out, self.wo, add_to=residual)
        qkv = rt.linear(h, self.wqkv)
        out = attention.decode_fused(ctx, qkv, self.q_norm, self.k_norm, self.norm_eps, cos, sin, cache, self.heads, self.window, self.scale, self.own_kv)
        if out is None:   # not a step of decoded tokens only, or sizes the fused kernel does not have
            q = rt.empty((ctx.n_tokens, self.heads * self.head_dim))
            ops.qk_norm_rope_kv(qkv, self.q_norm, self.k_norm, self.norm_eps, cos, sin, ctx.positions, ctx.seg_of_token, q, cache, self.heads,
                                rt.status, write_kv=self.own_kv)
            out = attention.paged_attention(ctx, q, cache, self.heads, self.window, self.scale)
        return rt.linear(out, self.wo, add_to=residual)


# ------------------------------------------------------------------------------------------ feed-forward
@base.register_feed_forward("swiglu")
class SwiGLU(base.FeedForward):
    """down(silu(gate h) * up h), silu(g) = g / (1 + exp(-g)) in float32
    (crates/kir/src/cuda/prelude.cu:125-133; gate and up fused into one product at load,
    crates/specrt/src/weights.rs:1049-1062)."""

    def __init__(self, prefix: str, hidden: int, intermediate: int):
        self.prefix, self.hidden, self.intermediate = prefix, hidden, intermediate
        self.wgu = self.wd = None

    def weight_specs(self):
        p = self.prefix
        return [WeightSpec(f"{p}.gate_proj.weight", (self.intermediate, self.hidden)), WeightSpec(f"{p}.up_proj.weight", (self.intermediate, self.hidden)),
                WeightSpec(f"{p}.down_proj.weight", (self.hidden, self.intermediate))]

    def bind(self, weights, rt):
        p = self.prefix
        self.wgu = rt.matrix(torch.cat([weights[f"{p}.gate_proj.weight"], weights[f"{p}.up_proj.weight"]], dim=0))
        self.wd = rt.matrix(weights[f"{p}.down_proj.weight"])

    adds_to_residual = True   # the down projection may add to the residual stream in its epilogue

    def forward(self, ctx, h, residual=None):
        rt = ctx.rt
        return rt.linear(rt.gate_up_act(h, self.wgu), self.wd, add_to=residual)


# ------------------------------------------------------------------------------------------ embedding and head
@base.register_embedding("table")
class TokenEmbedding(base.Embedding):
    """x[t] = float32(E[token_t]) * 1 (crates/kir/src/prims.rs:387)."""

    def __init__(self, name: str, vocab: int, hidden: int):
        self.name, self.vocab, self.hidden = name, vocab, hidden
        self.table = None

    def weight_specs(self):
        return [WeightSpec(self.name, (self.vocab, self.hidden))]

    def bind(self, weights, rt):
        self.table = rt.matrix(weights[self.name])

    def forward(self, ctx):
        x = ctx.rt.empty((ctx.n_tokens, self.hidden), torch.float32)
        ops.embed(self.table.weight, ctx.token_ids, x, ctx.rt.status)
        return x


@base.register_head("linear")
class LinearHead(base.Head):
    """logits = W h in float32; `tied_to` names the embedding table to use instead of a matrix of
    its own (a tied model ignores lm_head.weight even when the file has it:
    crates/specrt/src/weights.rs:1396-1405)."""

    def __init__(self, name: str, vocab: int, hidden: int, tied_to: Optional[str] = None):
        self.name, self.vocab, self.hidden, self.tied_to = name, vocab, hidden, tied_to
        self.w = None

    def weight_specs(self):
        return [WeightSpec(self.tied_to or self.name, (self.vocab, self.hidden))]   # tied: the embedding's table, read by both

    def bind(self, weights, rt):
        self.w = rt.matrix(weights[self.tied_to or self.name])

    def forward(self, ctx, h):
        out = ctx.rt.linear(h, self.w, allow_split=False)
        if out.shape[0] != 1:
            raise RuntimeError(f"the head's product came back in {out.shape[0]} partial sums although it asked for one")
        return out[0]


# ------------------------------------------------------------------------------------------ block
@base.register_block("prenorm")
class PreNormBlock(base.Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x)) (crates/specrt/graphs/decoder.toml:168-303).
    Each residual add is fused into the norm that follows it, so the feed-forward's contribution
    is handed to the next block (or the final norm) instead of being added here."""

    def forward(self, ctx, x, pending, cache):
        h = self.mixer_norm.forward(ctx, x, pending)
        a = self.mixer.forward(ctx, h, cache, residual=x) if self.mixer.adds_to_residual else self.mixer.forward(ctx, h, cache)
        h = self.feed_forward_norm.forward(ctx, x, a)
        return self.feed_forward.forward(ctx, h, residual=x) if self.feed_forward.adds_to_residual else self.feed_forward.forward(ctx, h)
