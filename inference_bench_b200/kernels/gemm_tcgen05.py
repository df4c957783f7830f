"""Tile and split choice for the tcgen05 matrix product, and its launch.

The kernel puts 128 weight rows and `bn` tokens in a CTA. Few tokens leave few CTAs, so the k-range
of a tile is then split over several CTAs, each writing its own float32 partial; the consumer kernel
adds the partials in a fixed order, so results are reproducible. The choice depends only on the
sizes of the product (T, N, K), never on which requests make up the batch.
"""
from __future__ import annotations

import torch

from . import lib as L
from . import ops

SM_COUNT = 148
TOKEN_TILES = (16, 32, 64, 128, 256)

L.register("ib_gemm_tcgen05", [L._p, L._p, L._p, L._i, L._i, L._i, L._i, L._i, L._p, L._p])


def supports(k: int) -> bool:
    return k % 8 == 0


def choose(T: int, N: int, K: int, allow_split: bool = True) -> tuple[int, int]:
    """(tokens per CTA, k-splits)."""
    bn = next((b for b in TOKEN_TILES if T <= b), 256)
    tiles = -(-N // 128) * -(-T // bn)
    ktiles = -(-K // 64)
    splits = 1
    slots = SM_COUNT * (2 if bn <= 32 else 1)      # CTAs resident at once (two per SM for the small token tiles)
    if allow_split and tiles < slots:
        splits = max(1, min(slots // tiles, ktiles // 4, 16))
        per = -(-ktiles // splits)
        splits = -(-ktiles // per)  # no empty split
    return bn, splits


def gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bn: int, splits: int, status: torch.Tensor) -> None:
    """out [splits, T, N] float32 = per-split partial products of x [T, K] and w [N, K] (bfloat16)."""
    T, K = x.shape
    N = w.shape[0]
    ops._check("x", x, torch.bfloat16)
    ops._check("w", w, torch.bfloat16, (N, K))
    ops._check("out", out, torch.float32, (splits, T, N))
    L.call("ib_gemm_tcgen05", x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, bn, splits, status.data_ptr(), ops._stream())


def linear(rt, x: torch.Tensor, lw, allow_split: bool = True) -> torch.Tensor:
    T = x.shape[0]
    bn, splits = choose(T, lw.n, lw.k, allow_split)
    out = rt.empty((splits, T, lw.n), torch.float32)
    gemm(x, lw.weight, out, bn, splits, rt.status)
    return out
