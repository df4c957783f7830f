"""Chooses the attention kernels for a step. bfloat16 with a head size of 64 or 128 runs on the
tensor-core kernels: decoded tokens (segments of one token) on the split-context kernel, prompt
portions on the flash kernel; everything else (float32, other head sizes, groups above 16) runs on
the generic kernel. All of them read keys and values through the block table and agree up to rounding.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import lib as L
from . import ops

def decode_tile() -> int:
    """Keys per tile of the decode kernel (csrc/attention_decode.cu); a CTA walks a slice of several tiles."""
    return int(L.load().ib_attention_decode_tile())


def decode_tiles_per_slice(n_dec: int, kv_heads: int, max_keys: int) -> int:
    """How many tiles one CTA takes: one while the step has few (token, kv head, tile) items, so
    that every SM gets work; more when there are thousands, so that fewer partial results are
    written and merged. For a given value a token's result does not depend on the batch."""
    items = n_dec * kv_heads * -(-max_keys // decode_tile())
    tps = 2 if max_keys > 2 * decode_tile() else 1      # two tiles: the second is fetched while the first is used
    while tps < 8 and items // tps > 1024:
        tps *= 2
    return tps

def stream_slices(n_dec: int, kv_heads: int, max_keys: int, sm_count: int) -> int:
    """Into how many slices the streaming decode kernel cuts each token's keys. Its CTAs stay (two per
    SM) and take (slice, token, kv head) units in turn: with few tokens, as many slices as give every
    CTA one unit; with more (token, kv head) pairs than CTAs, enough slices for about six units per
    CTA, so that the last round leaves few CTAs idle. A slice has two tiles at least."""
    slots = 2 * sm_count
    pairs = n_dec * kv_heads
    want = slots // pairs if pairs <= slots else -(-6 * slots // pairs)
    tiles = -(-max_keys // decode_tile())
    return max(1, min(want, -(-tiles // 2)))


QTILE = 128   # query rows per CTA of the prefill kernels (csrc/attention_prefill_ws.cu, attention_prefill_tc.cu)

# Which kernel runs is a runtime option (config/runtime_options.py): `prefill_attention` "ws" (tcgen05, one job per warp, keys and
# values by TMA) or "tcgen05" (every thread does everything, cp.async), "auto" = ws where TMA can serve the page size;
# `decode_attention` "stream" (CTAs that stay and a ring that TMA fills: measured inside whole decode steps at the Qwen3-8B shape and
# page size 64 the faster one from 1 to 128 requests, by 1 to 7 %) or "split" (one CTA per slice, cp.async), "auto" = stream where TMA
# can serve the page size; `fuse_decode_qk` with `fuse_decode_max_pairs` (every unit of the fused kernel prepares its queries again,
# which costs more than the saved kernel from about 16 requests of 8 kv heads on).
L.register("ib_attention_decode", [L._p, C.POINTER(L.KvView), L._p, L._i, L._p, L._p, L._i, L._f, L._p, L._p, L._p, L._i, L._i, L._i, L._p, L._p])
L.register("ib_attention_decode_stream", [L._p, C.POINTER(L.KvView), L._p, L._i, L._p, L._p, L._i, L._f, L._p, L._p, L._p, L._i, L._i, L._i, L._p, L._ll, L._p, L._p])
L.register("ib_attention_decode_fused", [L._p, L._i, L._ll, L._p, L._p, L._f, L._p, L._p, L._i, C.POINTER(L.KvView), L._p, L._i, L._p, L._p, L._i, L._f, L._p, L._p,
                                         L._p, L._i, L._i, L._i, L._p, L._ll, L._p, L._p])
L.register("ib_attention_prefill_tc", [L._p, C.POINTER(L.KvView), L._p, L._p, L._i, L._p, L._p, L._i, L._f, L._p, L._i, L._p, L._p])
L.register("ib_attention_prefill_ws", [L._p, C.POINTER(L.KvView), L._p, L._p, L._i, L._p, L._p, L._i, L._f, L._p, L._i, L._p, L._ll, L._p, L._p])


def has_tensor_core_kernel(dtype: torch.dtype, head_dim: int, heads: int, kv_heads: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and heads // kv_heads <= 16


def _work_lists(ctx):
    """Per step, shared by all layers: flat rows of decoded tokens, and 64-row query tiles of portions."""
    qtile = QTILE
    key = ("attention_work", qtile)
    if key in ctx.memo:
        return ctx.memo[key]
    if ctx.fixed_shape:
        work = dict(dec_tokens=ctx.seg_start[:ctx.n_tokens], n_dec=ctx.n_tokens, tile_seg=None, tile_row0=None, n_tiles=0, max_pos=None)
    else:
        lens = np.diff(ctx.h_seg_start)
        dec = ctx.h_seg_start[:-1][lens == 1].astype(np.int32)
        tiles = []   # (last position the tile sees, segment, first row): the tiles with the most keys go first
        for s in np.nonzero(lens > 1)[0]:
            for r in range(0, int(lens[s]), qtile):
                tiles.append((int(ctx.h_seg_pos0[s]) + min(r + qtile, int(lens[s])), int(s), r))
        tiles.sort(key=lambda t: -t[0])
        tile_seg, tile_row0 = [t[1] for t in tiles], [t[2] for t in tiles]
        flat = np.concatenate([dec, np.asarray(tile_seg, np.int32), np.asarray(tile_row0, np.int32)]).astype(np.int32)
        dev = torch.from_numpy(flat).pin_memory().to(ctx.rt.device, non_blocking=True) if flat.size else None
        nd, nt = dec.size, len(tile_seg)
        work = dict(dec_tokens=dev[:nd] if nd else None, n_dec=nd, tile_seg=dev[nd:nd + nt] if nt else None,
                    tile_row0=dev[nd + nt:] if nt else None, n_tiles=nt,
                    max_pos=int(ctx.h_positions[dec].max()) if nd else None)
    ctx.memo[key] = work
    return work


def project_qkv(ctx, h: torch.Tensor, lw, q_norm_w, k_norm_w, eps: float, cos, sin, cache: ops.KvLayerView, heads: int, write_kv: bool) -> Optional[torch.Tensor]:
    """The q/k/v projection of h [T, K] by the fused [q | k | v] matrix with the per-head norms, the rotation and the
    cache write in the matrix product's epilogue: returns the finished queries [T, heads * hd], or None when that
    kernel does not take the step (float32, few tokens, a head size other than 128, a rotation over part of the
    head): the caller then runs the product and `ops.qk_norm_rope_kv`."""
    rt = ctx.rt
    if rt.mode != "bfloat16" or rt.gemm == "simt" or h.dtype != torch.bfloat16:
        return None
    from . import gemm_tcgen05 as G
    view = cache.c_view()
    if view.head_dim != 128 or view.dtype != L.BF16 or not G.supports(lw.k) or lw.n != (heads + 2 * view.kv_heads) * 128:
        return None
    if cos is not None and 2 * cos.shape[1] != 128:
        return None
    if not G.qkv_in_epilogue(rt, h.shape[0], lw.n, lw.k):
        return None
    q = rt.empty((h.shape[0], heads * 128))
    G.gemm_qkv_pair(h, lw.weight, q, cache, heads, q_norm_w, k_norm_w, eps, cos, sin, ctx.positions, ctx.seg_of_token, write_kv, rt.status)
    return q


def decode_fused(ctx, qkv: torch.Tensor, q_norm_w, k_norm_w, eps: float, cos, sin, cache: ops.KvLayerView, heads: int, window: Optional[int],
                 scale: float, write_kv: bool) -> Optional[torch.Tensor]:
    """Attention for a step of decoded tokens only, straight from the q/k/v projection's partial sums
    qkv float32 [P, T, (heads + 2 kv_heads) * hd]: what `ops.qk_norm_rope_kv` and `paged_attention` do
    together, in one kernel (csrc/attention_decode.cu, the fused form). Returns None when that kernel
    cannot take the step (prompt portions in it, float32, a head size or page size it does not have,
    a rotation over part of the head, or a layer that reads another layer's cache: its own position's
    key and value are that layer's, not its own projection's): the caller then runs the two steps."""
    rt = ctx.rt
    view = cache.c_view()
    hd = view.head_dim
    if not write_kv:
        return None
    opt = rt.options
    if not (opt.decode_qk and opt.decode_attention != "split" and rt.act_dtype == torch.bfloat16 and has_tensor_core_kernel(rt.act_dtype, hd, heads, view.kv_heads)):
        return None
    if cos is not None and 2 * cos.shape[1] != hd:
        return None
    work = _work_lists(ctx)
    if work["n_tiles"] or not work["n_dec"]:
        return None
    kv_map, row0 = cache.tma()
    if not kv_map or work["n_dec"] * view.kv_heads > opt.fuse_decode_max_pairs:
        return None
    P, T, R = qkv.shape
    if R != (heads + 2 * view.kv_heads) * hd or T != ctx.n_tokens:
        raise L.KernelError(f"decode_fused: qkv is {tuple(qkv.shape)}, expected [P, {ctx.n_tokens}, {(heads + 2 * view.kv_heads) * hd}]")
    ops._check("qkv", qkv, torch.float32)
    for name, w in (("q_norm", q_norm_w), ("k_norm", k_norm_w)):
        if w is not None:
            ops._check(name, w, torch.float32, (hd,))
    if cos is not None:
        ops._check("cos", cos, torch.float32, (T, hd // 2))
        ops._check("sin", sin, torch.float32, (T, hd // 2))
    out = rt.empty((T, heads * hd), rt.act_dtype)
    limit = view.table_stride * view.page_size
    max_keys = limit if work["max_pos"] is None else work["max_pos"] + 1
    tps = opt.stream_tiles_per_slice
    max_slices = -(-max_keys // (tps * decode_tile())) if tps else stream_slices(work["n_dec"], view.kv_heads, max_keys, rt.sm_count)
    skey = ("decode_scratch", heads, hd, max_slices)
    if skey not in ctx.memo:
        n = work["n_dec"] * heads * max_slices
        ctx.memo[skey] = (rt.empty((n * hd,), torch.float32), rt.empty((n * 2,), torch.float32))
    part_o, part_ml = ctx.memo[skey]
    L.call("ib_attention_decode_fused", qkv.data_ptr(), P, T * R, ops._ptr(q_norm_w), ops._ptr(k_norm_w), float(eps), ops._ptr(cos), ops._ptr(sin),
           1 if write_kv else 0, C.byref(view), work["dec_tokens"].data_ptr(), work["n_dec"], ctx.positions.data_ptr(), ctx.seg_of_token.data_ptr(),
           int(window or 0), float(scale), part_o.data_ptr(), part_ml.data_ptr(), out.data_ptr(), heads, max_slices, tps, kv_map, row0,
           rt.status.data_ptr(), ops._stream())
    return out


def paged_attention(ctx, q: torch.Tensor, cache: ops.KvLayerView, heads: int, window: Optional[int], scale: float) -> torch.Tensor:
    """q [T, heads*hd] (activation dtype) -> attention output of the same shape and dtype."""
    rt = ctx.rt
    out = rt.empty(tuple(q.shape), q.dtype)
    view = cache.c_view()
    if not has_tensor_core_kernel(q.dtype, view.head_dim, heads, view.kv_heads):
        ops.attention_generic(q, cache, ctx.positions, ctx.seg_of_token, window, scale, out, heads, rt.status)
        return out
    work = _work_lists(ctx)
    stream = ops._stream()
    if work["n_dec"]:
        limit = view.table_stride * view.page_size
        max_keys = limit if work["max_pos"] is None else work["max_pos"] + 1
        opt = rt.options
        stream_map, stream_row0 = cache.tma() if opt.decode_attention != "split" else (None, 0)
        if opt.decode_attention == "stream" and not stream_map:
            raise L.KernelError(f"decode_attention = \"stream\" needs a page size that TMA can serve (a multiple of 8 that divides 64, or a multiple of 64), got {view.page_size}")
        if stream_map:
            tps = opt.stream_tiles_per_slice
            max_slices = -(-max_keys // (tps * decode_tile())) if tps else stream_slices(work["n_dec"], view.kv_heads, max_keys, rt.sm_count)
        else:
            tps = opt.split_tiles_per_slice or decode_tiles_per_slice(work["n_dec"], view.kv_heads, max_keys)
            max_slices = -(-max_keys // (tps * decode_tile()))
        skey = ("decode_scratch", heads, view.head_dim, max_slices)
        if skey not in ctx.memo:
            n = work["n_dec"] * heads * max_slices
            ctx.memo[skey] = (rt.empty((n * view.head_dim,), torch.float32), rt.empty((n * 2,), torch.float32))
        part_o, part_ml = ctx.memo[skey]
        args = (q.data_ptr(), C.byref(view), work["dec_tokens"].data_ptr(), work["n_dec"], ctx.positions.data_ptr(), ctx.seg_of_token.data_ptr(),
                int(window or 0), float(scale), part_o.data_ptr(), part_ml.data_ptr(), out.data_ptr(), heads, max_slices, tps)
        if stream_map:
            L.call("ib_attention_decode_stream", *args, stream_map, stream_row0, rt.status.data_ptr(), stream)
        else:
            L.call("ib_attention_decode", *args, rt.status.data_ptr(), stream)
    if work["n_tiles"]:
        args = (q.data_ptr(), C.byref(view), work["tile_seg"].data_ptr(), work["tile_row0"].data_ptr(), work["n_tiles"], ctx.seg_start.data_ptr(),
                ctx.seg_pos0.data_ptr(), int(window or 0), float(scale), out.data_ptr(), heads)
        kv_map, row0 = cache.tma() if rt.options.prefill_attention != "tcgen05" else (None, 0)
        if rt.options.prefill_attention == "ws" and not kv_map:
            raise L.KernelError(f"prefill_attention = \"ws\" needs a page size that TMA can serve (a multiple of 8 that divides 64, or a multiple of 64), got {view.page_size}")
        if kv_map:
            L.call("ib_attention_prefill_ws", *args, kv_map, row0, rt.status.data_ptr(), stream)
        else:
            L.call("ib_attention_prefill_tc", *args, rt.status.data_ptr(), stream)
    return out
