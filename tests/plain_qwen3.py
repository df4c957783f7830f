"""Plain, slow implementation of the Qwen3 dense decoder, used as the oracle by the tests.

Whole sequences, no cache, no paging, no batching; one function per part; float32 (or float64)
tensors on the CPU. It shares no code with the engine package: it has its own safetensors
reader and its own config handling, and it is written from the formulas of v0l/inference-bench
(`specrt`), cited per function by the file's path inside that project.

The model code of v0l/inference-bench is Rust that emits CUDA text for NVRTC and has no CPU
execution path, and no Rust toolchain exists where these tests run, so this file could not be
compared with the reference's own model code: it rests on the cited formulas.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2), "I32": (np.int32, 4), "I64": (np.int64, 8)}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Read every tensor of a .safetensors file to float32 (integers stay integers).

    Format: 8-byte little-endian header length, JSON header {name: {dtype, shape, data_offsets}},
    raw little-endian data (crates/specrt/src/weights.rs:181-201 opens the same layout)."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + n])
    base = 8 + n
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        np_dtype, _ = _DTYPES[info["dtype"]]
        lo, hi = info["data_offsets"]
        arr = np.frombuffer(raw[base + lo : base + hi], dtype=np_dtype).reshape(info["shape"])
        if info["dtype"] == "BF16":
            t = torch.from_numpy((arr.astype(np.uint32) << 16).view(np.float32).copy())
        elif info["dtype"] in ("I32", "I64"):
            t = torch.from_numpy(arr.copy())
        else:
            t = torch.from_numpy(arr.astype(np.float32))
        out[name] = t
    return out


def read_config(model_dir) -> dict:
    """config.json keys the Qwen3 family reads (crates/specrt/src/spec.rs:958-1003, 1461-1738)."""
    c = json.loads((Path(model_dir) / "config.json").read_text())
    heads = c["num_attention_heads"]
    theta = c.get("rope_theta")
    if theta is None and isinstance(c.get("rope_parameters"), dict):
        theta = c["rope_parameters"].get("rope_theta")
    types = c.get("layer_types") or ["full_attention"] * c["num_hidden_layers"]
    return {
        "vocab": c["vocab_size"],
        "hidden": c["hidden_size"],
        "inter": c["intermediate_size"],
        "layers": c["num_hidden_layers"],
        "heads": heads,
        "kv_heads": c.get("num_key_value_heads", heads),
        "head_dim": c.get("head_dim") or c["hidden_size"] // heads,
        "eps": c["rms_norm_eps"],
        "theta": float(theta if theta is not None else 10000.0),
        "tied": bool(c.get("tie_word_embeddings", False)),
        "windows": [c.get("sliding_window") if t == "sliding_attention" else None for t in types],
    }


def embedding(table: torch.Tensor, tokens) -> torch.Tensor:
    """x[t, :] = table[token_t, :] with scale 1 (crates/kir/tests/golden/prims/prims_sm120.cu:19-24)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """inv = rsqrt(mean(x^2) + eps); y_i = w_i * (x_i * inv), no unit offset for Qwen3
    (crates/kir/tests/golden/rmsnorm_sm120.cu:19-29; crates/specrt/src/weights.rs:877-880)."""
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return w * (x * inv)


def rope_neox(v: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Half-rotation RoPE over the whole head: pair (d, d + hd/2), inv_freq_i = theta^(-2i/hd),
    angle = pos * inv_freq_i; out_d = v_d cos - v_{d+half} sin (d < half),
    out_d = v_d cos + v_{d-half} sin (d >= half)
    (crates/kir/tests/golden/attention/RopeKvWrite_bf16x2_sm120.cu:32-35, 200-206).
    v: [n, heads, hd], positions: [n]."""
    hd = v.shape[-1]
    half = hd // 2
    i = torch.arange(half, dtype=torch.float64)
    inv_freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), 2.0 * i / hd)
    ang = positions.to(torch.float64)[:, None] * inv_freq[None, :]
    c = torch.cos(ang).to(v.dtype)[:, None, :]
    s = torch.sin(ang).to(v.dtype)[:, None, :]
    a, b = v[..., :half], v[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def attention_scores(q, k, v, window=None, positions=None) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    s = (q . k) / sqrt(hd); key j is visible from query i when j <= i, and with a window W only
    when j > i - W; softmax over visible keys; query head h reads kv head h // (heads / kv_heads)
    (crates/kir/tests/golden/attention/FlashMma_bf16x2_sm120.cu:261-266, 468-520;
    mask: crates/kir/src/cuda/attention/flash_mma.rs:193).
    q: [n, heads, hd], k, v: [n, kv_heads, hd] -> [n, heads*hd]."""
    n, heads, hd = q.shape
    group = heads // k.shape[1]
    pos = torch.arange(n) if positions is None else positions
    visible = pos[None, :] <= pos[:, None]
    if window:
        visible &= pos[None, :] > pos[:, None] - window
    out = torch.empty(n, heads, hd, dtype=q.dtype)
    for h in range(heads):
        s = (q[:, h, :] @ k[:, h // group, :].T) / math.sqrt(hd)
        s = s.masked_fill(~visible, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, h // group, :]
    return out.reshape(n, heads * hd)


def attention_block(x, w, prefix, cfg, window, positions=None) -> torch.Tensor:
    """q/k/v projections, per-head RMSNorm of q and k (same eps), RoPE, attention, o projection
    (crates/specrt/src/weights.rs:886-953; crates/kir/tests/golden/attention/RopeKvWrite_bf16x2_sm120.cu:193-197;
    crates/specrt/graphs/decoder.toml:168-249)."""
    n = x.shape[0]
    hd = cfg["head_dim"]
    pos = torch.arange(n) if positions is None else positions
    q = (x @ w[prefix + "q_proj.weight"].T).reshape(n, cfg["heads"], hd)
    k = (x @ w[prefix + "k_proj.weight"].T).reshape(n, cfg["kv_heads"], hd)
    v = (x @ w[prefix + "v_proj.weight"].T).reshape(n, cfg["kv_heads"], hd)
    q = rope_neox(rmsnorm(q, w[prefix + "q_norm.weight"], cfg["eps"]), pos, cfg["theta"])
    k = rope_neox(rmsnorm(k, w[prefix + "k_norm.weight"], cfg["eps"]), pos, cfg["theta"])
    a = attention_scores(q, k, v, window, pos)
    return a @ w[prefix + "o_proj.weight"].T


def swiglu(x, w, prefix) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), silu(g) = g / (1 + exp(-g))
    (crates/kir/src/cuda/prelude.cu:125-133; crates/kir/tests/golden/swiglu_silu.cu:1-11)."""
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    return ((g / (1.0 + torch.exp(-g))) * u) @ w[prefix + "down_proj.weight"].T


def lm_head(x, w, cfg) -> torch.Tensor:
    """logits = W_lm . rmsnorm(x); a tied model uses the embedding table even when the file
    carries lm_head.weight too (crates/specrt/src/weights.rs:1396-1405)."""
    table = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return rmsnorm(x, w["model.norm.weight"], cfg["eps"]) @ table.T


def hidden_states(w, cfg, tokens, upto_layers=None) -> torch.Tensor:
    """Pre-norm residual stack: x += attn(norm(x)); x += mlp(norm(x))
    (crates/specrt/graphs/decoder.toml:168-303)."""
    x = embedding(w["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["layers"] if upto_layers is None else upto_layers):
        p = f"model.layers.{layer}."
        h = rmsnorm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        x = x + attention_block(h, w, p + "self_attn.", cfg, cfg["windows"][layer])
        h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        x = x + swiglu(h, w, p + "mlp.")
    return x


class PlainModel:
    """A model folder (config.json + model.safetensors) evaluated whole, in float32 or float64."""

    def __init__(self, model_dir, dtype=torch.float32):
        self.cfg = read_config(model_dir)
        self.w = {k: (t.to(dtype) if t.is_floating_point() else t) for k, t in read_safetensors(Path(model_dir) / "model.safetensors").items()}

    @torch.no_grad()
    def logits(self, tokens) -> torch.Tensor:
        """Logits at every position of `tokens`, [n, vocab]."""
        return lm_head(hidden_states(self.w, self.cfg, tokens), self.w, self.cfg)

    @torch.no_grad()
    def greedy(self, tokens, new_tokens: int) -> list[int]:
        """Greedy continuation (argmax, lowest index on ties:
        crates/kir/tests/golden/prims/prims_sm120.cu:165-196), recomputing the whole sequence."""
        seq = list(tokens)
        for _ in range(new_tokens):
            seq.append(argmax_lowest(self.logits(seq)[-1]))
        return seq[len(tokens):]

    @torch.no_grad()
    def sample(self, tokens, new_tokens: int, temperature: float, seed: int, top_k=0, top_p=1.0, min_p=0.0) -> list[int]:
        seq = list(tokens)
        for step in range(new_tokens):
            seq.append(sample_token(self.logits(seq)[-1].float(), temperature, seed, step, top_k, top_p, min_p))
        return seq[len(tokens):]


def argmax_lowest(row: torch.Tensor) -> int:
    m = row.max()
    return int(torch.nonzero(row == m)[0, 0])


def gumbel_noise(seed: int, step: int, n: int) -> torch.Tensor:
    """g_i = -ln(-ln u_i), u_i from an integer hash of (seed, step, i)
    (crates/kir/tests/golden/prims/prims_sm120.cu:34-39)."""
    i = np.arange(n, dtype=np.uint64)
    m = np.uint64(0xFFFFFFFF)
    x = (np.uint64(seed) * np.uint64(747796405) + np.uint64(step) * np.uint64(2891336453) + i * np.uint64(2246822519) + np.uint64(1)) & m
    x ^= x >> np.uint64(16)
    x = (x * np.uint64(2246822507)) & m
    x ^= x >> np.uint64(13)
    x = (x * np.uint64(3266489909)) & m
    x ^= x >> np.uint64(16)
    u = ((x >> np.uint64(8)).astype(np.float32) + np.float32(0.5)) / np.float32(16777216.0)
    return torch.from_numpy(-np.log(-np.log(u.astype(np.float64))).astype(np.float32))


def sample_token(row: torch.Tensor, temperature: float, seed: int, step: int, top_k=0, top_p=1.0, min_p=0.0) -> int:
    """Temperature 0 is argmax. Otherwise Gumbel-max over the candidates that survive top-k
    (value >= k-th largest), top-p (smallest set of largest values with mass >= top_p) and min-p
    (value >= max + ln(min_p)), all on v = logit / T
    (crates/kir/tests/golden/prims/prims_sm120.cu:51-163, 208-250; crates/specrt/src/runtime.rs:602-630)."""
    if temperature <= 0:
        return argmax_lowest(row)
    v = row.float() * np.float32(1.0 / temperature)
    n = v.numel()
    thr = -math.inf
    if 0 < top_k < n:
        thr = float(torch.topk(v, top_k).values[-1])
    if top_p < 1.0:
        kept = v[v >= thr]
        srt = torch.sort(kept.double(), descending=True).values
        p = torch.exp(srt - srt[0])
        cum = torch.cumsum(p, 0)
        idx = int(torch.nonzero(cum >= max(top_p, 1e-9) * cum[-1])[0, 0])
        thr = max(thr, float(srt[idx]))
    if min_p > 0.0:
        thr = max(thr, float(v.max()) + math.log(min_p))
    noisy = torch.where(v >= thr, v + gumbel_noise(seed, step, n), torch.tensor(-math.inf))
    return argmax_lowest(noisy)
