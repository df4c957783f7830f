"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some hosts of this library cannot allocate device memory while they run (they gave the device to
an arena of their own, or their serving loop forbids calls that may synchronise the device), so
`ib_attention_decode_noalloc` keeps the kernel's scratch in a fixed array inside the library. This
test checks it against the ordinary entry point, which takes scratch from the caller (the same
kernels, so the same bits), and against a plain float64 attention, on two calls in a row (the second
call finds the first call's leftovers in the shared array); that the driver's count of free device
memory does not move across a call; that a call too large for the fixed array is refused; and that a
`max_slices` too small for the positions in use is reported through the status word instead of
reading past the array. It sits in a file that pytest collects last."""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_FLOATS = 2 * 1024 * 1024


def _case(seed, heads, kvh, hd, page, lengths):
    """Decoded tokens at the last position of requests with the given context lengths."""
    from inference_bench_b200.kernels.ops import KvLayerView
    g = torch.Generator().manual_seed(seed)
    n = len(lengths)
    need = [-(-L // page) for L in lengths]
    total = sum(need) + 3
    order = np.random.default_rng(seed).permutation(total)
    pool = (torch.randn(1, total, 2, kvh, page, hd, generator=g)).to(torch.bfloat16)
    table = np.full((n, max(need) + 1), -1, dtype=np.int32)
    at = 0
    for s in range(n):
        for p in range(need[s]):
            table[s, p] = order[at]
            at += 1
    q = torch.randn(n, heads * hd, generator=g).to(torch.bfloat16)
    view = KvLayerView(pool.to(DEV), 0, torch.from_numpy(table).to(DEV))
    positions = torch.tensor([L - 1 for L in lengths], dtype=torch.int32, device=DEV)
    seg = torch.arange(n, dtype=torch.int32, device=DEV)
    return q.to(DEV), view, positions, seg


def _plain(q, view, lengths, heads, kvh, hd, page, window):
    """Float64 attention of each decoded token over its request's keys, read back out of the paged pool."""
    import plain_qwen3 as P
    pool, table = view.pool.cpu().float(), view.block_table.cpu().numpy()
    out = []
    for s, L_ in enumerate(lengths):
        pages = [int(table[s, p]) for p in range(-(-L_ // page))]
        k = torch.cat([pool[0, pg, 0] for pg in pages], dim=1)[:, :L_].transpose(0, 1)   # [L, kvh, hd]
        v = torch.cat([pool[0, pg, 1] for pg in pages], dim=1)[:, :L_].transpose(0, 1)
        q_full = torch.zeros(L_, heads, hd, dtype=torch.float64)
        q_full[-1] = q[s].cpu().double().reshape(heads, hd)
        out.append(P.attention_scores(q_full, k.double(), v.double(), window or None)[-1].reshape(-1))
    return torch.stack(out)


def test_no_alloc_entry_point_matches_the_ordinary_one():
    from inference_bench_b200.kernels import lib as L
    lib = L.load()
    fn = lib.ib_attention_decode_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.POINTER(L.KvView), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_int,
                   C.c_int, C.c_void_p, C.c_void_p]
    ref_fn = lib.ib_attention_decode
    ref_fn.restype = C.c_int
    ref_fn.argtypes = [C.c_void_p, C.POINTER(L.KvView), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_void_p,
                       C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    TILE = lib.ib_attention_decode_tile()
    stream = torch.cuda.current_stream().cuda_stream
    first = True
    for seed, (heads, kvh, hd, page, lengths, window, tps) in enumerate([(8, 2, 128, 16, [700, 129, 5, 1024], 0, 1), (4, 1, 64, 32, [300, 64, 2000], 150, 4)]):
        q, view, positions, seg = _case(seed, heads, kvh, hd, page, lengths)
        n = len(lengths)
        max_slices = max(lengths) // (TILE * tps) + 1
        cview = view.c_view()
        scale = 1 / math.sqrt(hd)
        part_o = torch.empty(n * heads * max_slices * hd, device=DEV)
        part_ml = torch.empty(n * heads * max_slices * 2, device=DEV)
        want = torch.empty_like(q)
        rc = ref_fn(q.data_ptr(), C.byref(cview), seg.data_ptr(), n, positions.data_ptr(), seg.data_ptr(), window, scale, part_o.data_ptr(),
                    part_ml.data_ptr(), want.data_ptr(), heads, max_slices, tps, status.data_ptr(), stream)
        assert rc == 0, lib.ib_last_error()
        plain = _plain(q, view, lengths, heads, kvh, hd, page, window)
        for call in range(2):
            got = torch.full_like(q, float("nan"))
            if first:   # the very first call on the device resolves the array's address; allocation is measured on the calls after it
                rc = fn(q.data_ptr(), C.byref(cview), seg.data_ptr(), n, positions.data_ptr(), seg.data_ptr(), window, scale, got.data_ptr(), heads,
                        max_slices, tps, status.data_ptr(), stream)
                assert rc == 0, lib.ib_last_error()
                first = False
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info(DEV)     # the driver's own count of free device memory: sees every cudaMalloc, not only torch's
            torch_before = torch.cuda.memory_allocated(DEV)
            rc = fn(q.data_ptr(), C.byref(cview), seg.data_ptr(), n, positions.data_ptr(), seg.data_ptr(), window, scale, got.data_ptr(), heads,
                    max_slices, tps, status.data_ptr(), stream)
            assert rc == 0, lib.ib_last_error()
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info(DEV)
            assert free_after == free_before and torch.cuda.memory_allocated(DEV) == torch_before
            assert status.item() == 0
            assert torch.equal(got, want), f"case {seed}, call {call}: differs from the ordinary entry point, which runs the same kernels"
            diff = (got.cpu().double() - plain).abs().max().item()
            assert diff <= 1.5e-2 * plain.abs().max().item(), f"case {seed}, call {call}: differs from the plain attention by {diff}"
    # a call beyond the fixed scratch is refused with a message, and nothing runs
    q, view, positions, seg = _case(9, 32, 8, 128, 16, [100] * 8)
    cview = view.c_view()
    out = torch.zeros_like(q)
    too_many = MAX_FLOATS // (8 * 32 * 130) + 1
    rc = fn(q.data_ptr(), C.byref(cview), seg.data_ptr(), 8, positions.data_ptr(), seg.data_ptr(), 0, 0.1, out.data_ptr(), 32, too_many,
            1, status.data_ptr(), stream)
    torch.cuda.synchronize()
    assert rc != 0 and b"more than the fixed scratch" in lib.ib_last_error()
    assert out.abs().max().item() == 0
    # max_slices that does not cover the positions in use (only a foreign host can get this wrong: positions live on the
    # device, so the entry point cannot check it): the status word says so and nothing beyond the scratch is read
    q, view, positions, seg = _case(10, 8, 2, 128, 16, [700, 129])
    cview = view.c_view()
    out = torch.zeros_like(q)
    rc = fn(q.data_ptr(), C.byref(cview), seg.data_ptr(), 2, positions.data_ptr(), seg.data_ptr(), 0, 0.1, out.data_ptr(), 8, 3, 1,
            status.data_ptr(), stream)
    torch.cuda.synchronize()
    assert rc == 0 and status.item() == L.ERR_INTERNAL
    assert torch.isfinite(out.float()).all()
    status.zero_()
