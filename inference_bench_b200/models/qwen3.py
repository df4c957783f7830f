"""Qwen3 dense (`Qwen3ForCausalLM`) as a plan: which parts, with which sizes, under which tensor names.

Tensor names are the ones the reference reads (crates/specrt/src/plan.rs:117-151, 185-193); the
block is pre-norm attention + SwiGLU (crates/specrt/graphs/decoder.toml:168-303) with per-head
q/k norm (crates/specrt/specs/family-qwen3.toml:10-11) and half-rotation RoPE over the whole head.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..parts.plan import LayerPlan, ModelPlan, PartSpec, ScheduleEntry
from ..registry import register_architecture


def qwen3_plan(c: Qwen3Config) -> ModelPlan:
    rope = PartSpec("rope", {"rotary_dim": c.head_dim, "theta": c.rope_theta})
    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}"
        layers.append(LayerPlan(
            prefix=p,
            block="prenorm",
            mixer=PartSpec("attention", {
                "prefix": f"{p}.self_attn", "hidden": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                "head_dim": c.head_dim, "qk_norm": True, "norm_eps": c.rms_norm_eps, "position": rope, "window": c.window_of(i)}),
            feed_forward=PartSpec("swiglu", {"prefix": f"{p}.mlp", "hidden": c.hidden_size, "intermediate": c.intermediate_size}),
            mixer_norm=PartSpec("rmsnorm", {"name": f"{p}.input_layernorm.weight", "size": c.hidden_size, "eps": c.rms_norm_eps}),
            feed_forward_norm=PartSpec("rmsnorm", {"name": f"{p}.post_attention_layernorm.weight", "size": c.hidden_size, "eps": c.rms_norm_eps}),
        ))
    return ModelPlan(
        architecture="Qwen3ForCausalLM",
        vocab_size=c.vocab_size,
        hidden_size=c.hidden_size,
        max_positions=c.max_position_embeddings,
        embedding=PartSpec("table", {"name": "model.embed_tokens.weight", "vocab": c.vocab_size, "hidden": c.hidden_size}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(c.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"name": "model.norm.weight", "size": c.hidden_size, "eps": c.rms_norm_eps}),
        head=PartSpec("linear", {"name": "lm_head.weight", "vocab": c.vocab_size, "hidden": c.hidden_size,
                                 "tied_to": "model.embed_tokens.weight" if c.tie_word_embeddings else None}),
        ignored_tensors=("lm_head.weight",) if c.tie_word_embeddings else (),
    )


# `Qwen3MoeForCausalLM` / `qwen3_moe` are deliberately not registered: this engine has the dense decoder only.
register_architecture(["Qwen3ForCausalLM", "qwen3"], Qwen3Config.from_dict, qwen3_plan,
                      traits={"attention": "gqa", "qk_norm": True, "norm": "rmsnorm", "norm_unit_offset": False, "rope_style": "neox", "activation": "swiglu"})
