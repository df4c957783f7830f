"""Tile and split choice for the tcgen05 matrix product, and its launch.

The kernel puts 128 weight rows and `bn` tokens in a CTA. Few tokens leave few CTAs, so the k-range
of a tile is then split over several CTAs, each writing its own float32 partial; the consumer kernel
adds the partials in a fixed order, so results are reproducible. The choice depends only on the
sizes of the product (T, N, K), never on which requests make up the batch.
"""
from __future__ import annotations

import ctypes as C
import functools
from typing import Optional

import torch

from . import lib as L
from . import ops

FITTED_SM_COUNT = 148   # the part the cost model below was fitted on; every function takes the running device's count as an argument
TOKEN_TILES = (16, 32, 64, 128, 256)

L.register("ib_gemm_tcgen05", [L._p, L._p, L._p, L._i, L._i, L._i, L._i, L._i, L._i, L._p, L._p])
L.register("ib_gemm_swiglu_tcgen05", [L._p, L._p, L._p, L._i, L._i, L._i, L._i, L._i, L._p, L._p])
L.register("ib_gemm_tcgen05_2cta", [L._p, L._p, L._p, L._i, L._i, L._i, L._p, L._p])
L.register("ib_gemm_swiglu_tcgen05_2cta", [L._p, L._p, L._p, L._i, L._i, L._i, L._p, L._p])
L.register("ib_gemm_tcgen05_2cta_add", [L._p, L._p, L._p, L._i, L._i, L._i, L._p, L._p])
L.register("ib_gemm_qkv_tcgen05_2cta", [L._p, L._p, L._i, L._i, L._p, L._p, L._f, L._p, L._p, L._p, L._p, L._p, C.POINTER(L.KvView), L._i, L._i, L._p, L._p])

# Runtime options that steer the choice (config/runtime_options.py): `pair_min_tokens` (129: the fused gate/up product runs on the
# persistent CTA-pair kernel, csrc/gemm_tcgen05_2cta.cu, from here on whatever its size), `pair_always_tokens` (2,048: every
# product from here on; between the two, `plan` decides by its cost model) and `fuse_qkv_epilogue`.


def supports(k: int) -> bool:
    return k % 8 == 0


@functools.lru_cache(maxsize=4096)
def choose(T: int, N: int, K: int, allow_split: bool = True, sm_count: int = FITTED_SM_COUNT) -> tuple[int, int, bool]:
    """(tokens per CTA, k-splits, wide) for up to 128 tokens: the smallest token tile that holds them, and the
    k-range split over CTAs until the GPU is full."""
    if T > 128:
        raise ValueError(f"choose is for up to 128 tokens, got {T}: see plan")
    ktiles = -(-K // 64)
    bn = next(b for b in TOKEN_TILES if T <= b)
    tiles = -(-N // 128)
    slots = sm_count * (2 if bn <= 64 else 1)      # CTAs resident at once (two per SM for the small token tiles)
    splits = 1
    if allow_split and tiles < slots:
        splits = max(1, min(slots // tiles, ktiles // 4, 16))
        per = -(-ktiles // splits)
        splits = -(-ktiles // per)  # no empty split
    return bn, splits, False


# Cost model for 129 to 2,048 tokens, fitted to timings of every variant below on the layer shapes of Qwen3-0.6B, 8B,
# 14B and 32B at 160 to 1,536 tokens (the variant it picks is within 5 % of the fastest on all of them, 0.2 % on
# average). A variant's time is waves of CTAs (or CTA pairs) times the longer of a CTA's MMA time and its copy time,
# plus a fixed cost, plus the traffic of split-K partial sums. Units: FLOP/us, bytes/us, us.
_MID = dict(rate=4.015e6, cap=250e3, t0=4.36, partial_bw=3.455e6, pair_rate=5.446e6, hbm=8.0e6, pair_cap=188e3,
            speed={(256, True): 1.0, (256, False): 0.982, (128, True): 0.895, (128, False): 0.956})


def single_variants(T: int, N: int, K: int, sm_count: int = FITTED_SM_COUNT, allow_split: bool = True):
    """The forms of the single-CTA kernel that `plan` weighs for more than 128 tokens: (tokens per CTA, k-splits, wide)."""
    ktiles = -(-K // 64)
    for bn in (128, 256):
        for wide in (False, True):
            for sp in ((1, 2, 3, 4, 6) if allow_split else (1,)):
                per = -(-ktiles // sp)
                if sp > max(1, ktiles // 4) or -(-ktiles // per) != sp:   # at least four k-tiles a split, and none empty
                    continue
                ctas = -(-N // (256 if wide else 128)) * -(-T // bn) * sp
                if sp > 1 and ctas > 4 * sm_count:
                    continue
                yield bn, sp, wide


@functools.lru_cache(maxsize=4096)
def plan_costs(T: int, N: int, K: int, sm_count: int = FITTED_SM_COUNT, allow_split: bool = True) -> tuple:
    """(expected us of the CTA-pair kernel, expected us of the best single-CTA form, that form) for 129 <= T < 2048.
    allow_split=False leaves out the forms that cut the k-range (for a caller that wants one finished product)."""
    m = _MID
    tiles = -(-N // 256) * -(-T // 256)
    active = min(tiles, sm_count // 2) * 2
    pair = -(-tiles // (sm_count // 2)) * max(256 * 256 * K * 2 / (2 * m["pair_rate"]), 256 * K * 2 / min(m["pair_cap"], m["hbm"] / active)) + m["t0"]
    best = (float("inf"), None)
    ktiles = -(-K // 64)
    for bn, sp, wide in single_variants(T, N, K, sm_count, allow_split):
        rows = 256 if wide else 128
        ctas = -(-N // rows) * -(-T // bn) * sp
        kc = -(-ktiles // sp) * 64
        mma = rows * bn * kc * 2 / (m["rate"] * m["speed"][(bn, wide)])
        copy = (rows + min(bn, T)) * kc * 2 / min(m["cap"], m["hbm"] / min(ctas, sm_count))
        t = -(-ctas // sm_count) * max(mma, copy) + m["t0"] + (sp * T * N * 4 / m["partial_bw"] if sp > 1 else 0.0)
        if t < best[0]:
            best = (t, (bn, sp, wide))
    return pair, best[0], best[1]


def plan(T: int, N: int, K: int, sm_count: int = FITTED_SM_COUNT, allow_split: bool = True) -> tuple:
    """For 129 <= T < 2048: ("pair",) or ("single", tokens per CTA, k-splits, wide), whichever the cost model
    expects to be faster. Depends on the sizes (and the device's SM count) only."""
    pair, single, form = plan_costs(T, N, K, sm_count, allow_split)
    return ("pair",) if pair <= single else ("single",) + form


def qkv_in_epilogue(rt, T: int, N: int, K: int) -> bool:
    """Whether the q/k/v projection of T tokens runs as the CTA-pair kernel with the q/k norm, the rotation and the
    cache write in its epilogue: from 2,048 tokens always; from 129 when that is expected to take no longer than the
    best plain product followed by the kernel it saves (about 3 us + 20 ns a token inside a step)."""
    if not rt.options.qkv_epilogue or T <= 128:
        return False
    if T >= rt.options.pair_always_tokens:
        return True
    pair, single, _ = plan_costs(T, N, K, rt.sm_count)
    return pair <= single + 3.0 + 0.02 * T


def balanced_portion(matrices, nominal: int = 2048, sm_count: int = FITTED_SM_COUNT) -> int:
    """A prompt-portion size near `nominal` (a multiple of 256 between 3/4 and 5/4 of it) whose 256 x 256 tiles fill
    whole rounds of the CTA pairs best, for the [N, K] matrices of a layer: the time a token costs is taken as the sum
    over the matrices of K x rounds x 74 tiles / tokens. The CTA-pair products work in rounds of 74 tiles, and a portion
    that ends in a nearly empty round pays for it (measured: 14B shape 45.2 k tok/s at 1,792 tokens against 41.3 k at
    2,048; 32B 19.0 against 18.1 k; 8B 80.8 k at 2,304 against 79.9 k). Ties go to the size nearest to `nominal`."""
    pairs = sm_count // 2
    best = None
    for T in range(max(256, nominal * 3 // 4 // 256 * 256), nominal * 5 // 4 + 1, 256):
        cost = sum(k * -(-(-(-n // 256) * -(-T // 256)) // pairs) for n, k in matrices) / T
        key = (cost, abs(T - nominal), -T)
        if best is None or key < best[0]:
            best = (key, T)
    return best[1] if best else nominal


def gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bn: int, splits: int, status: torch.Tensor, wide: bool = False) -> None:
    """out [splits, T, N] float32 = per-split partial products of x [T, K] and w [N, K] (bfloat16).
    wide: 256 rows of w per CTA instead of 128 (token tiles of 128 or 256 only)."""
    T, K = x.shape
    N = w.shape[0]
    ops._check("x", x, torch.bfloat16)
    ops._check("w", w, torch.bfloat16, (N, K))
    ops._check("out", out, torch.float32, (splits, T, N))
    L.call("ib_gemm_tcgen05", x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, bn, splits, 1 if wide else 0, status.data_ptr(), ops._stream())


def gemm_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor, add: bool = False) -> None:
    """out [T, N] float32 = x [T, K] w[N, K]^T on CTA pairs (256 x 256 tiles, persistent); with `add`
    the product is added to what out holds."""
    T, K = x.shape
    N = w.shape[0]
    ops._check("x", x, torch.bfloat16)
    ops._check("w", w, torch.bfloat16, (N, K))
    ops._check("out", out, torch.float32, (T, N))
    L.call("ib_gemm_tcgen05_2cta_add" if add else "ib_gemm_tcgen05_2cta", x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, status.data_ptr(), ops._stream())


def gemm_qkv_pair(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, kv: "ops.KvLayerView", heads: int, q_norm_w: Optional[torch.Tensor],
                  k_norm_w: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                  seg_of_token: torch.Tensor, write_kv: bool, status: torch.Tensor) -> None:
    """q_out [T, heads * 128] bfloat16 and the paged cache from x [T, K] and w [(heads + 2 kv_heads) * 128, K]: the
    projection, the per-head norms, the rotation and the cache write in one kernel (csrc/gemm_tcgen05_2cta.cu)."""
    T, K = x.shape
    view = kv.c_view()
    if view.head_dim != 128 or (cos is not None and cos.shape[1] != 64):
        raise L.KernelError(f"gemm_qkv_pair: head size {view.head_dim} with a rotation over {None if cos is None else 2 * cos.shape[1]} values (128 and 128 or none)")
    N = (heads + 2 * view.kv_heads) * 128
    ops._check("x", x, torch.bfloat16)
    ops._check("w", w, torch.bfloat16, (N, K))
    ops._check("q_out", q_out, torch.bfloat16, (T, heads * 128))
    ops._check("positions", positions, torch.int32, (T,))
    ops._check("seg_of_token", seg_of_token, torch.int32, (T,))
    for name, v in (("q_norm", q_norm_w), ("k_norm", k_norm_w)):
        if v is not None:
            ops._check(name, v, torch.float32, (128,))
    if cos is not None:
        ops._check("cos", cos, torch.float32, (T, 64))
        ops._check("sin", sin, torch.float32, (T, 64))
    L.call("ib_gemm_qkv_tcgen05_2cta", x.data_ptr(), w.data_ptr(), T, K, ops._ptr(q_norm_w), ops._ptr(k_norm_w), float(eps), ops._ptr(cos), ops._ptr(sin),
           positions.data_ptr(), seg_of_token.data_ptr(), q_out.data_ptr(), C.byref(view), 1 if write_kv else 0, heads, status.data_ptr(), ops._stream())


def linear(rt, x: torch.Tensor, lw, allow_split: bool = True, add_to: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    T = x.shape[0]
    how = ("pair",) if T >= rt.options.pair_always_tokens else (plan(T, lw.n, lw.k, rt.sm_count, allow_split) if T > 128 else None)
    if how is not None and how[0] == "single":
        _, bn, splits, wide = how
        out = rt.empty((splits, T, lw.n), torch.float32)
        gemm(x, lw.weight, out, bn, splits, rt.status, wide)
        return out
    if how is not None:
        if add_to is not None:
            gemm_pair(x, lw.weight, add_to, rt.status, add=True)
            return None
        out = rt.empty((1, T, lw.n), torch.float32)
        gemm_pair(x, lw.weight, out[0], rt.status)
        return out
    bn, splits, wide = choose(T, lw.n, lw.k, allow_split, rt.sm_count)
    out = rt.empty((splits, T, lw.n), torch.float32)
    gemm(x, lw.weight, out, bn, splits, rt.status, wide)
    return out


PAIR_SWIGLU_MIN_TILES = 40   # 256-column blocks of the intermediate size from which the CTA-pair kernel takes the fused gate/up product of 33 to 128 tokens


HALF_SWIGLU_MIN_CTAS = 148   # CTAs (intermediate size / 64) from which the form with gate and up rows in one accumulator is used
HALF_SWIGLU_MAX_TOKENS = 64   # ... and up to how many tokens (at 64 tokens 0.7 % of a batch-64 decode step faster than the CTA-pair form, Qwen3-8B shape)


def swiglu_supported(T: int, k: int, inter: int = 0) -> bool:
    """Whether the gate/up product applies the activation in its epilogue: from 65 tokens always; from 33 where the
    intermediate size gives the CTA-pair kernel 40 tiles or more (measured 8 to 10 % faster there than the split-K
    product followed by the SiLU-mul kernel, at the 8B, 14B and 32B shapes; slower at the 0.6B shape); up to 64 tokens
    in the form that puts 64 gate rows and their 64 up rows into one accumulator, where the intermediate size is a
    multiple of 64 and gives every SM a CTA (a smaller one goes through the split-K product and the SiLU-mul kernel,
    which then fill the GPU better)."""
    if not supports(k):
        return False
    if half_swiglu(T, inter):
        return True
    return T > 64 or (T > 32 and -(-inter // 256) >= PAIR_SWIGLU_MIN_TILES)


def half_swiglu(T: int, inter: int) -> bool:
    """Whether the fused gate/up product of T tokens takes the form with 64 gate rows and 64 up rows in one accumulator."""
    return T <= HALF_SWIGLU_MAX_TOKENS and inter % 64 == 0 and inter // 64 >= HALF_SWIGLU_MIN_CTAS


def gemm_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor, status: torch.Tensor, bn: int | None = None, pair_min_tokens: int = 129,
                half: bool | None = None) -> None:
    """act [T, I] bfloat16 = silu(x gate^T) * (x up^T) with w_gate_up [2I, K] = gate rows then up rows."""
    T, K = x.shape
    I = w_gate_up.shape[0] // 2
    ops._check("x", x, torch.bfloat16)
    ops._check("w_gate_up", w_gate_up, torch.bfloat16, (2 * I, K))
    ops._check("act", act, torch.bfloat16, (T, I))
    if bn is None and (half_swiglu(T, I) or (T <= 32 and I % 64 == 0)):
        bn, half = (16 if T <= 16 else 32 if T <= 32 else 64), True
    if half is None:
        half = bn in (16, 32)
    if bn is None and (T >= pair_min_tokens or (T > 32 and -(-I // 256) >= PAIR_SWIGLU_MIN_TILES)):
        L.call("ib_gemm_swiglu_tcgen05_2cta", x.data_ptr(), w_gate_up.data_ptr(), act.data_ptr(), T, I, K, status.data_ptr(), ops._stream())
        return
    if bn is None:
        bn = 64 if T <= 64 else (128 if T <= 128 else 256)
    L.call("ib_gemm_swiglu_tcgen05", x.data_ptr(), w_gate_up.data_ptr(), act.data_ptr(), T, I, K, bn, 1 if half else 0, status.data_ptr(), ops._stream())
