"""Tiny Qwen3 configurations for the tests. They differ in every size and option: layers, width,
head counts and group size, head size (coupled to the width or not), feed-forward width,
vocabulary, rotation base, norm eps, tied or untied head, window and which layers have one, page
size. Sizes are deliberately no powers of two where the architecture allows it."""
from __future__ import annotations

from pathlib import Path

CONFIGS = {
    # 2 layers, group 2, head 16 (4*16 == 64), tied, no window
    "A": dict(seed=0, page_size=16, std=0.05, config=dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64, intermediate_size=192,
        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0,
        tie_word_embeddings=True, max_position_embeddings=128, hidden_act="silu", attention_bias=False, torch_dtype="bfloat16")),
    # 3 layers, group 2, head 24 (6*24 != 96), untied, no window, small pages
    "B": dict(seed=1, page_size=8, std=0.04, config=dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=384, hidden_size=96, intermediate_size=160,
        num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3, head_dim=24, rms_norm_eps=1e-5, rope_theta=1000000.0,
        tie_word_embeddings=False, max_position_embeddings=256, hidden_act="silu", attention_bias=False, torch_dtype="bfloat16")),
    # 4 layers, group 5 on one kv head, head 32, odd vocabulary, windows on layers 0 and 2
    "C": dict(seed=2, page_size=16, std=0.06, config=dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=301, hidden_size=80, intermediate_size=112,
        num_hidden_layers=4, num_attention_heads=5, num_key_value_heads=1, head_dim=32, rms_norm_eps=3e-6, rope_theta=500000.0,
        tie_word_embeddings=False, max_position_embeddings=512, hidden_act="silu", attention_bias=False, torch_dtype="bfloat16",
        sliding_window=24, layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"])),
    # head 64 with a window on layer 1: the tensor-core attention kernels in bfloat16
    "D": dict(seed=3, page_size=16, std=0.05, config=dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=500, hidden_size=128, intermediate_size=200,
        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0,
        tie_word_embeddings=False, max_position_embeddings=512, hidden_act="silu", attention_bias=False, torch_dtype="bfloat16",
        sliding_window=40, layer_types=["full_attention", "sliding_attention"])),
    # head 128, group 4 on one kv head, larger pages
    "E": dict(seed=4, page_size=32, std=0.05, config=dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=320, hidden_size=72, intermediate_size=136,
        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
        tie_word_embeddings=True, max_position_embeddings=512, hidden_act="silu", attention_bias=False, torch_dtype="bfloat16")),
}


def write_tiny(name: str, out_dir) -> Path:
    from inference_bench_b200.weights.random_init import write_random_model

    c = CONFIGS[name]
    return write_random_model(c["config"], c["seed"], out_dir, std=c["std"])
