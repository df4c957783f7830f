"""Tensor-level wrappers of the kernel library: argument checks, then one launch on the current stream.

Tensors must be contiguous CUDA tensors; nothing here computes on the CPU or through torch ops.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import lib as L

_CODE = {torch.float32: L.F32, torch.bfloat16: L.BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODE[dtype]
    except KeyError:
        raise L.KernelError(f"dtype {dtype} is not supported by the kernels (float32 and bfloat16 are)") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check(name: str, t: torch.Tensor, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise L.KernelError(f"{name} must be a CUDA tensor: the kernels have no CPU path")
    if not t.is_contiguous():
        raise L.KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise L.KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise L.KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)   # the current stream's handle without building a Stream object
_device_index: Optional[int] = None


def _stream() -> int:
    """The handle of torch's current stream on the engine's device (every kernel is launched on it)."""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


_KV_MAPS: dict = {}   # (pool address, shape) -> (buffer that owns the bytes, aligned address of the 128-byte tensor map) or None


def kv_tensor_map(pool: torch.Tensor):
    """The TMA description of a bfloat16 cache pool, made once per pool; None when the geometry
    cannot be served by TMA (the attention kernels then copy with cp.async)."""
    key = (pool.data_ptr(), tuple(pool.shape), pool.dtype)
    if key not in _KV_MAPS:
        entries, pages, two, kv_heads, page_size, head_dim = pool.shape
        made = None
        if pool.dtype == torch.bfloat16 and head_dim % 64 == 0 and page_size % 8 == 0 and (64 % page_size == 0 or page_size % 64 == 0):
            buf = C.create_string_buffer(128 + 64)
            addr = (C.addressof(buf) + 63) & ~63
            lib = L.load()
            lib.ib_make_kv_map.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int]
            lib.ib_make_kv_map.restype = C.c_int
            if lib.ib_make_kv_map(addr, pool.data_ptr(), pages * entries * two * kv_heads * page_size, head_dim, page_size) == 0:
                made = (buf, addr)
        _KV_MAPS[key] = made
    return _KV_MAPS[key]


@dataclass
class KvLayerView:
    """One layer's keys and values inside a paged pool, plus the block table of the step."""
    pool: torch.Tensor          # [entries, pages, 2, kv_heads, page_size, head_dim]: one layer's pages lie together
    entry: int
    block_table: torch.Tensor   # int32 [segments, table_stride]

    def tma(self) -> tuple[Optional[int], int]:
        """(address of the pool's tensor map or None, pool row where this view's keys of page 0, head 0 start)."""
        m = kv_tensor_map(self.pool)
        _, pages, _, kv_heads, page_size, _ = self.pool.shape
        return (m[1] if m else None), self.entry * pages * 2 * kv_heads * page_size

    def c_view(self) -> L.KvView:
        cv = self.__dict__.get("_cv")   # made once per view: a layer asks for it several times a step
        if cv is None:
            cv = self.__dict__["_cv"] = self._make_c_view()
        return cv

    def _make_c_view(self) -> L.KvView:
        entries, pages, two, kv_heads, page_size, head_dim = self.pool.shape
        if two != 2:
            raise L.KernelError(f"a KV pool must be [entries, pages, 2, kv_heads, page_size, head_dim], got {tuple(self.pool.shape)}")
        _check("kv pool", self.pool)
        _check("block_table", self.block_table, torch.int32)
        per_kv = kv_heads * page_size * head_dim
        esz = self.pool.element_size()
        return L.KvView(
            base=self.pool.data_ptr() + self.entry * pages * 2 * per_kv * esz,
            page_stride=2 * per_kv,
            v_offset=per_kv,
            block_table=self.block_table.data_ptr(),
            table_stride=self.block_table.shape[1],
            page_size=page_size,
            num_pages=pages,
            kv_heads=kv_heads,
            head_dim=head_dim,
            dtype=dtype_code(self.pool.dtype),
        )


def embed(table: torch.Tensor, tokens: torch.Tensor, x: torch.Tensor, status: torch.Tensor) -> None:
    """x[t] = float32(table[tokens[t]])."""
    V, H = table.shape
    T = tokens.shape[0]
    _check("table", table)
    _check("tokens", tokens, torch.int32)
    _check("x", x, torch.float32, (T, H))
    L.call("ib_embed", table.data_ptr(), dtype_code(table.dtype), tokens.data_ptr(), x.data_ptr(), T, H, V, status.data_ptr(), _stream())


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, out: torch.Tensor, eps: float,
                rows: Optional[torch.Tensor] = None) -> None:
    """x += sum_p delta[p] (in place, unless `rows` gathers); out = w * (x * rsqrt(mean(x^2) + eps)).

    delta is None or float32 [P, T, H]; with `rows` (int32 [n]) output row r comes from source row rows[r]."""
    T, H = x.shape
    _check("x", x, torch.float32)
    _check("w", w, torch.float32, (H,))
    n_rows = T if rows is None else rows.shape[0]
    _check("out", out, None, (n_rows, H))
    P, stride = 0, 0
    if delta is not None:
        _check("delta", delta, torch.float32)
        if delta.dim() != 3 or tuple(delta.shape[1:]) != (T, H):
            raise L.KernelError(f"delta must be [P, {T}, {H}], got {tuple(delta.shape)}")
        P, stride = delta.shape[0], T * H
    if rows is not None:
        _check("rows", rows, torch.int32)
    L.call("ib_add_rmsnorm", x.data_ptr(), _ptr(delta), P, stride, w.data_ptr(), out.data_ptr(), dtype_code(out.dtype), _ptr(rows), n_rows, H,
           float(eps), 0 if rows is not None else 1, _stream())


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    T, half = positions.shape[0], inv_freq.shape[0]
    _check("positions", positions, torch.int32)
    _check("inv_freq", inv_freq, torch.float32)
    _check("cos", cos, torch.float32, (T, half))
    _check("sin", sin, torch.float32, (T, half))
    L.call("ib_rope_table", positions.data_ptr(), inv_freq.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, half, _stream())


def silu_mul(gate_up: torch.Tensor, act: torch.Tensor) -> None:
    """act = silu(gate) * up with gate_up float32 [P, T, 2I] = [gate | up], partials summed first."""
    _check("gate_up", gate_up, torch.float32)
    P, T, I2 = gate_up.shape
    _check("act", act, None, (T, I2 // 2))
    L.call("ib_silu_mul", gate_up.data_ptr(), P, T * I2, act.data_ptr(), dtype_code(act.dtype), T, I2 // 2, _stream())


def qk_norm_rope_kv(qkv: torch.Tensor, q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                    cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor, seg_of_token: torch.Tensor,
                    q_out: torch.Tensor, kv: KvLayerView, heads: int, status: torch.Tensor, write_kv: bool = True) -> None:
    """qkv float32 [P, T, (heads + 2 kv_heads) * hd] -> q_out [T, heads*hd] and the paged cache."""
    _check("qkv", qkv, torch.float32)
    P, T, R = qkv.shape
    view = kv.c_view()
    if R != (heads + 2 * view.kv_heads) * view.head_dim:
        raise L.KernelError(f"qkv has {R} columns, expected {(heads + 2 * view.kv_heads) * view.head_dim}")
    _check("q_out", q_out, None, (T, heads * view.head_dim))
    _check("positions", positions, torch.int32, (T,))
    _check("seg_of_token", seg_of_token, torch.int32, (T,))
    rot_half = 0
    if cos is not None:
        rot_half = cos.shape[1]
        _check("cos", cos, torch.float32, (T, rot_half))
        _check("sin", sin, torch.float32, (T, rot_half))
    for name, w in (("q_norm", q_norm_w), ("k_norm", k_norm_w)):
        if w is not None:
            _check(name, w, torch.float32, (view.head_dim,))
    L.call("ib_qk_norm_rope_kv", qkv.data_ptr(), P, T * R, _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(cos), _ptr(sin), rot_half,
           positions.data_ptr(), seg_of_token.data_ptr(), q_out.data_ptr(), dtype_code(q_out.dtype), C.byref(view), 1 if write_kv else 0, T,
           heads, status.data_ptr(), _stream())


def attention_generic(q: torch.Tensor, kv: KvLayerView, positions: torch.Tensor, seg_of_token: torch.Tensor, window: Optional[int],
                      scale: float, out: torch.Tensor, heads: int, status: torch.Tensor) -> None:
    view = kv.c_view()
    T = q.shape[0]
    _check("q", q, None, (T, heads * view.head_dim))
    _check("out", out, q.dtype, (T, heads * view.head_dim))
    _check("positions", positions, torch.int32, (T,))
    _check("seg_of_token", seg_of_token, torch.int32, (T,))
    L.call("ib_attention_generic", q.data_ptr(), dtype_code(q.dtype), C.byref(view), positions.data_ptr(), seg_of_token.data_ptr(),
           int(window or 0), float(scale), out.data_ptr(), T, heads, status.data_ptr(), _stream())


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, n] = sum_k x[t, k] w[n, k], float32 FMA."""
    T, K = x.shape
    N = w.shape[0]
    _check("x", x)
    _check("w", w, None, (N, K))
    _check("out", out, torch.float32, (T, N))
    L.call("ib_gemm_simt", x.data_ptr(), dtype_code(x.dtype), w.data_ptr(), dtype_code(w.dtype), out.data_ptr(), T, N, K, _stream())


def sample_chunks(vocab: int) -> int:
    return int(L.load().ib_sample_chunks(int(vocab)))


def sample_rows(logits: torch.Tensor, params: torch.Tensor, tokens: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """params int32 [rows, 6] = (inv_temp bits, seed, step, top_k, top_p bits, min_p bits). With `status` (the
    device status word) tokens has rows + 1 entries and the last one receives the word's value, so one
    transfer brings the host both the tokens and whether a kernel of the step reported a fault."""
    rows, V = logits.shape
    _check("logits", logits, torch.float32)
    _check("params", params, torch.int32, (rows, 6))
    _check("tokens", tokens, torch.int32, (rows + (1 if status is not None else 0),))
    scratch = torch.empty(rows * (1 + 2 * sample_chunks(V)), dtype=torch.float32, device=logits.device)
    L.call("ib_sample_rows", logits.data_ptr(), rows, V, params.data_ptr(), tokens.data_ptr(), scratch.data_ptr(), _ptr(status), _stream())


def advance_rows(sampled: torch.Tensor, token_in: torch.Tensor, positions: torch.Tensor, pos0: torch.Tensor, params: torch.Tensor,
                 history: torch.Tensor, count: torch.Tensor) -> None:
    """Feed sampled tokens back as the next inputs of a decode batch and log them: history[count, :] = sampled."""
    rows = sampled.shape[0]
    for name, t in (("sampled", sampled), ("token_in", token_in), ("positions", positions), ("pos0", pos0)):
        _check(name, t, torch.int32, (rows,))
    _check("params", params, torch.int32, (rows, 6))
    _check("history", history, torch.int32)
    _check("count", count, torch.int32, (1,))
    L.call("ib_advance_rows", sampled.data_ptr(), token_in.data_ptr(), positions.data_ptr(), pos0.data_ptr(), params.data_ptr(), history.data_ptr(),
           count.data_ptr(), rows, history.shape[0], _stream())
