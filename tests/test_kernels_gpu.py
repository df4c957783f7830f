"""Each CUDA kernel alone against its plain float32/float64 reference, at sizes other than the
engine's tiny models: widths and vocabularies that are no powers of two, odd token counts, several
head sizes and group sizes, shuffled pages, windows, and inputs built so that a fault shows."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def status():
    from inference_bench_b200.kernels import lib
    lib.load()
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def _g(seed):
    return torch.Generator().manual_seed(seed)


# ------------------------------------------------------------------------------------------ matrix products
@pytest.mark.parametrize("T,N,K", [(1, 7, 5), (3, 70, 33), (65, 129, 100), (130, 64, 257)])
def test_gemm_simt_float32(T, N, K):
    from inference_bench_b200.kernels import ops
    x = torch.randn(T, K, generator=_g(1)).to(DEV)
    w = torch.randn(N, K, generator=_g(2)).to(DEV)
    out = torch.empty(T, N, device=DEV)
    ops.gemm_simt(x, w, out)
    ref = (x.double() @ w.double().T)
    assert (out.double() - ref).abs().max() <= 1e-5 * ref.abs().max()


@pytest.mark.parametrize("T,N,K,bn,splits", [
    (1, 128, 64, 16, 1), (5, 100, 96, 16, 1), (16, 136, 72, 16, 2), (17, 384, 1024, 32, 4), (33, 130, 520, 64, 3),
    (100, 1000, 264, 128, 1), (300, 257, 2048, 256, 2), (513, 640, 4096, 256, 1), (8, 4096, 4096, None, None), (128, 1536, 1024, None, None),
    (2048, 1536, 1024, 256, 1)])
def test_gemm_tcgen05_bfloat16(status, T, N, K, bn, splits):
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    x = (torch.randn(T, K, generator=_g(3)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=_g(4)) * 0.5).to(torch.bfloat16).to(DEV)
    wide = False
    if bn is None:
        bn, splits, wide = G.choose(T, N, K)
    out = torch.full((splits, T, N), float("nan"), device=DEV)
    G.gemm(x, w, out, bn, splits, status, wide)
    ref = x.double() @ w.double().T
    got = out.double().sum(0)
    assert status.item() == 0
    assert (got - ref).abs().max() <= 2e-5 * ref.abs().max() + 1e-6
    # and it agrees with the plain-loop kernel on the same bfloat16 inputs
    from inference_bench_b200.kernels import ops
    simt = torch.empty(T, N, device=DEV)
    ops.gemm_simt(x, w, simt)
    assert (got - simt.double()).abs().max() <= 2e-5 * ref.abs().max() + 1e-6


@pytest.mark.parametrize("T,N,K", [(257, 1100, 1544), (300, 264, 4096), (129, 2000, 520), (700, 520, 1024)])
def test_gemm_tcgen05_every_form_above_128_tokens(status, T, N, K):
    """Every (token tile, k-split, wide) that `plan` may choose between 129 and 2,047 tokens, the CTA-pair kernel and
    what `plan` picks: all against the float64 product, and each the same bits when run twice."""
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    x = (torch.randn(T, K, generator=_g(5)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=_g(6)) * 0.5).to(torch.bfloat16).to(DEV)
    ref = x.double() @ w.double().T
    tol = 2e-5 * ref.abs().max() + 1e-6
    forms = list(G.single_variants(T, N, K))
    assert len(forms) >= 6
    for bn, sp, wide in forms:
        outs = []
        for _ in range(2):
            out = torch.full((sp, T, N), float("nan"), device=DEV)
            G.gemm(x, w, out, bn, sp, status, wide)
            outs.append(out)
        assert status.item() == 0
        assert torch.equal(outs[0], outs[1]), (bn, sp, wide)
        assert (outs[0].double().sum(0) - ref).abs().max() <= tol, (bn, sp, wide)
    out = torch.full((T, N), float("nan"), device=DEV)
    G.gemm_pair(x, w, out, status)
    assert status.item() == 0 and (out.double() - ref).abs().max() <= tol
    how = G.plan(T, N, K)
    assert how == ("pair",) or tuple(how[1:]) in forms


@pytest.mark.parametrize("T,N,K,bn", [(130, 300, 72, 128), (300, 520, 264, 256), (700, 1000, 1024, 256)])
def test_gemm_tcgen05_wide_tile(status, T, N, K, bn):
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    x = (torch.randn(T, K, generator=_g(3)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=_g(4)) * 0.5).to(torch.bfloat16).to(DEV)
    out = torch.full((1, T, N), float("nan"), device=DEV)
    G.gemm(x, w, out, bn, 1, status, wide=True)
    ref = x.double() @ w.double().T
    assert status.item() == 0 and (out[0].double() - ref).abs().max() <= 2e-5 * ref.abs().max() + 1e-6


@pytest.mark.parametrize("T,I,K,bn", [(65, 200, 136, 64), (70, 136, 72, 128), (300, 520, 264, 128), (513, 1000, 1024, 256), (2048, 384, 512, None)])
def test_gemm_swiglu_tcgen05(status, T, I, K, bn):
    """Gate and up products with the activation in the epilogue, against float64."""
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    x = (torch.randn(T, K, generator=_g(5)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, K, generator=_g(6)) * 0.2).to(torch.bfloat16).to(DEV)
    act = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    G.gemm_swiglu(x, w, act, status, bn)
    gu = x.double() @ w.double().T
    g, u = gu[:, :I], gu[:, I:]
    ref = g / (1 + torch.exp(-g)) * u
    assert status.item() == 0
    assert ((act.double() - ref).abs() <= 2.0 ** -8 * ref.abs() + 1e-5 * ref.abs().max()).all()


@pytest.mark.parametrize("T,I,K", [(1, 64, 64), (8, 12288, 4096), (5, 192, 72), (16, 640, 136), (17, 1344, 264), (32, 9536, 520), (3, 17408, 5120)])
def test_gemm_swiglu_few_tokens(status, T, I, K):
    """Up to 32 tokens: 64 gate rows and their 64 up rows in one accumulator, the halves meeting in the epilogue. Intermediate
    sizes that are no multiple of 128 (but of 64), k-ranges that end inside a k-tile, one token."""
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    from inference_bench_b200.kernels import lib as L
    x = (torch.randn(T, K, generator=_g(5)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, K, generator=_g(6)) * (3.0 / math.sqrt(K))).to(torch.bfloat16).to(DEV)
    act = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    called = []
    real = L.call
    L.call = lambda name, *a: (called.append((name, a[6] if name == "ib_gemm_swiglu_tcgen05" else None)), real(name, *a))[1]
    try:
        G.gemm_swiglu(x, w, act, status)
    finally:
        L.call = real
    assert called == [("ib_gemm_swiglu_tcgen05", 16 if T <= 16 else 32)]
    act64 = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=DEV)      # the same form with 64 tokens per CTA
    G.gemm_swiglu(x, w, act64, status, bn=64, half=True)
    assert torch.equal(act64, act)
    gu = x.double() @ w.double().T
    g, u = gu[:, :I], gu[:, I:]
    ref = g / (1 + torch.exp(-g)) * u
    assert status.item() == 0
    assert ((act.double() - ref).abs() <= 2.0 ** -8 * ref.abs() + 1e-5 * ref.abs().max()).all()
    with pytest.raises(L.KernelError, match="multiple of 64"):
        G.gemm_swiglu(x, torch.zeros(2 * 100, K, dtype=torch.bfloat16, device=DEV), torch.empty(T, 100, dtype=torch.bfloat16, device=DEV), status, bn=16)
    assert G.swiglu_supported(8, 4096, 12288) and not G.swiglu_supported(8, 4096, 3072) and not G.swiglu_supported(8, 4096, 12300)


@pytest.mark.parametrize("T,N,K", [(256, 256, 64), (257, 130, 72), (300, 520, 264), (1000, 1000, 1024), (2048, 1536, 512), (4152, 640, 256)])
def test_gemm_tcgen05_cta_pairs(status, T, N, K):
    """The persistent CTA-pair kernel (cta_group::2), more tiles than pairs included."""
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    x = (torch.randn(T, K, generator=_g(3)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=_g(4)) * 0.5).to(torch.bfloat16).to(DEV)
    out = torch.full((T, N), float("nan"), device=DEV)
    G.gemm_pair(x, w, out, status)
    ref = x.double() @ w.double().T
    assert status.item() == 0 and (out.double() - ref).abs().max() <= 2e-5 * ref.abs().max() + 1e-6
    # the same product added to a residual stream in place
    base = torch.randn(T, N, generator=_g(7)).to(DEV) * 3
    acc = base.clone()
    G.gemm_pair(x, w, acc, status, add=True)
    assert status.item() == 0 and torch.equal(acc, base + out)


@pytest.mark.parametrize("T,I,K", [(256, 128, 64), (300, 520, 264), (1000, 1000, 1024), (2048, 20000, 128), (33, 10240, 136), (64, 12288, 200),
                                   (100, 10300, 72)])
def test_gemm_swiglu_cta_pairs(status, T, I, K):
    """The fused gate/up product on CTA pairs: from 129 tokens, and from 33 when the intermediate size gives 40 tiles."""
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    assert T >= 129 or (T > 32 and -(-I // 256) >= G.PAIR_SWIGLU_MIN_TILES)
    x = (torch.randn(T, K, generator=_g(5)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, K, generator=_g(6)) * 0.2).to(torch.bfloat16).to(DEV)
    act = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    G.gemm_swiglu(x, w, act, status)          # no tile given: 256 tokens and more go to the CTA pairs
    gu = x.double() @ w.double().T
    g, u = gu[:, :I], gu[:, I:]
    ref = g / (1 + torch.exp(-g)) * u
    assert status.item() == 0
    assert ((act.double() - ref).abs() <= 2.0 ** -8 * ref.abs() + 1e-5 * ref.abs().max()).all()


def test_gemm_tcgen05_refuses_bad_sizes(status):
    from inference_bench_b200.kernels import gemm_tcgen05 as G, lib
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device=DEV)   # K = 100 is no multiple of 8
    w = torch.zeros(8, 100, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(lib.KernelError, match="multiple of 8"):
        G.gemm(x, w, torch.empty(1, 4, 8, device=DEV), 16, 1, status)
    with pytest.raises(lib.KernelError, match="wide tile"):
        G.gemm(torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV), torch.empty(1, 4, 8, device=DEV), 16, 1, status, wide=True)
    assert not G.supports(100)


# ------------------------------------------------------------------------------------------ row-wise kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,P_", [(1, 10, 0), (7, 100, 1), (33, 1000, 3), (4, 5120, 2), (300, 1000, 0), (257, 4096, 1), (260, 72, 2), (256, 8192, 0)])   # 256 rows and more take the register form
def test_add_rmsnorm(dtype, T, H, P_):
    from inference_bench_b200.kernels import ops
    x = torch.randn(T, H, generator=_g(5)) * 3
    delta = torch.randn(P_, T, H, generator=_g(6)) if P_ else None
    w = 1 + 0.1 * torch.randn(H, generator=_g(7))
    eps = 3e-5
    xd = x.to(DEV)
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(xd, delta.to(DEV) if P_ else None, w.to(DEV), out, eps)
    x_ref = x.double() + (delta.double().sum(0) if P_ else 0)
    ref = P.rmsnorm(x_ref, w.double(), eps)
    assert (xd.cpu().double() - x_ref).abs().max() <= 1e-5
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -8
    assert ((out.cpu().double() - ref).abs() <= tol * ref.abs() + 1e-6).all()
    # gathered rows leave x alone
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    x2 = x.to(DEV)
    out2 = torch.empty(2, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(x2, delta.to(DEV) if P_ else None, w.to(DEV), out2, eps, rows)
    assert torch.equal(x2.cpu(), x)
    assert torch.equal(out2.cpu(), out.cpu()[[T - 1, 0]])


def test_embed_and_bad_token(status):
    from inference_bench_b200.kernels import ops
    table = torch.randn(301, 70, generator=_g(8)).to(torch.bfloat16)
    toks = torch.tensor([0, 300, 17, 17], dtype=torch.int32)
    x = torch.empty(4, 70, device=DEV)
    ops.embed(table.to(DEV), toks.to(DEV), x, status)
    assert torch.equal(x.cpu(), P.embedding(table.float(), toks.tolist()))
    assert status.item() == 0
    ops.embed(table.to(DEV), torch.tensor([301], dtype=torch.int32, device=DEV), torch.empty(1, 70, device=DEV), status)
    assert status.item() == 2   # a token outside the vocabulary is reported, never read
    status.zero_()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(dtype):
    from inference_bench_b200.kernels import ops
    gu = torch.randn(2, 5, 2 * 37, generator=_g(9)) * 4
    act = torch.empty(5, 37, dtype=dtype, device=DEV)
    ops.silu_mul(gu.to(DEV), act)
    s = gu.double().sum(0)
    g, u = s[:, :37], s[:, 37:]
    ref = g / (1 + torch.exp(-g)) * u
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -8
    assert ((act.cpu().double() - ref).abs() <= tol * ref.abs() + 1e-6).all()


def test_rope_table():
    from inference_bench_b200.kernels import ops
    pos = torch.tensor([0, 1, 77, 4095, 40000], dtype=torch.int32)
    inv = (1.0 / torch.pow(torch.tensor(1e6, dtype=torch.float64), torch.arange(0, 48, 2, dtype=torch.float64) / 48)).float()
    cos = torch.empty(5, 24, device=DEV)
    sin = torch.empty(5, 24, device=DEV)
    ops.rope_table(pos.to(DEV), inv.to(DEV), cos, sin)
    ang = pos.float()[:, None] * inv[None, :]     # float32 angles, as the reference computes them
    assert (cos.cpu() - torch.cos(ang.double()).float()).abs().max() <= 2e-6
    assert (sin.cpu() - torch.sin(ang.double()).float()).abs().max() <= 2e-6


def test_a_wait_that_runs_out_is_reported_and_the_kernel_returns(status):
    """Every wait inside the tensor-core kernels has a limit. Here the limit is set to a millisecond and the matrix
    product is launched through the entry point whose copying warp sends nothing, so no barrier is ever completed: the
    kernel must set the wait-timeout bit, store nothing, give its tensor memory back and return; and the next ordinary
    product on the same device must be right (tensor memory that was not given back would make it wait for ever)."""
    import ctypes as C
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    from inference_bench_b200.kernels import lib as L
    lib = L.load()
    fn = lib.ib_test_gemm_tcgen05_starved
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    lib.ib_set_wait_limit_ms.argtypes = [C.c_int]
    T, N, K = 8, 256, 512
    x = (torch.randn(T, K, generator=_g(71)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=_g(72)) * 0.5).to(torch.bfloat16).to(DEV)
    out = torch.full((1, T, N), float("nan"), device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, status.data_ptr(), stream) != 0      # refused while the limit is the ordinary two seconds
    assert b"wait limit" in lib.ib_last_error()
    lib.ib_set_wait_limit_ms(1)
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        assert fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, status.data_ptr(), stream) == 0, lib.ib_last_error()
        t1.record()
        torch.cuda.synchronize()
    finally:
        lib.ib_set_wait_limit_ms(2000)
    assert status.item() == L.ERR_WAIT_TIMEOUT
    assert 0.9 <= t0.elapsed_time(t1) < 50.0, f"the starved kernel took {t0.elapsed_time(t1):.2f} ms with a limit of 1 ms"
    assert torch.isnan(out).all()                      # nothing was stored
    status.zero_()
    for _ in range(3):                                 # the ordinary kernel, three times: it allocates tensor memory again
        G.gemm(x, w, out, 16, 1, status)
    ref = x.double() @ w.double().T
    assert status.item() == 0
    assert (out[0].double() - ref).abs().max() <= 2e-5 * ref.abs().max() + 1e-6


# ------------------------------------------------------------------------------------------ paged attention
def _paged(contexts, page_size, dtype, seed, entries=2, entry=1):
    """Scatter dense K, V ([L, kv_heads, hd] per request) into a pool with shuffled pages."""
    from inference_bench_b200.kernels.ops import KvLayerView
    kvh, hd = contexts[0][0].shape[1:]
    need = [-(-k.shape[0] // page_size) for k, _ in contexts]
    total = sum(need) + 5
    order = np.random.default_rng(seed).permutation(total)
    width = max(need) + 2
    table = np.full((len(contexts), width), -1, dtype=np.int32)
    pool = torch.full((entries, total, 2, kvh, page_size, hd), 37.0, dtype=dtype)   # rows that hold no key: finite, and loud if a mask lets one through
    at = 0
    for s, (k, v) in enumerate(contexts):
        for p in range(need[s]):
            page = int(order[at]); at += 1
            table[s, p] = page
            rows = slice(p * page_size, min((p + 1) * page_size, k.shape[0]))
            n = rows.stop - rows.start
            pool[entry, page, 0, :, :n] = k[rows].transpose(0, 1).to(dtype)
            pool[entry, page, 1, :, :n] = v[rows].transpose(0, 1).to(dtype)
    return KvLayerView(pool.to(DEV), entry, torch.from_numpy(table).to(DEV)), table


def _plant_window_edges(q, k, v, L, n, window, dtype, tile=128):
    """Make an off-by-one at a window's edge show. For the last query of the segment, and for the first and last query
    row of its last 128-row tile, at position p: the key at p - window (just outside) gets a direction aligned with that
    query and a loud value, so it must stay invisible; the key at p - window + 1 (the oldest visible one) gets the same
    direction and another loud value, so it must dominate that query's head 0. Letting the first in or dropping the
    second moves the output by several units."""
    used = set()
    rows = sorted({n - 1, (n - 1) // tile * tile, max(0, (n - 1) // tile * tile - 1)})
    for r in rows:
        p = L - n + r
        out_j, edge_j = p - window, p - window + 1
        if out_j < 0 or edge_j in used or out_j in used or edge_j >= p:
            continue
        u = q[r, 0] / q[r, 0].norm()
        k[out_j, 0] = (14.0 * u).to(dtype).float()
        v[out_j, 0] = -9.0
        k[edge_j, 0] = (12.0 * u).to(dtype).float()
        v[edge_j, 0] = 7.0
        used |= {out_j, edge_j}
    return len(used) // 2


def _attention_case(dtype, heads, kvh, hd, page_size, window, shapes, seed, needle=False):
    """shapes: (context length L, query tokens n) per segment; queries sit at the last n positions."""
    g = _g(seed)
    contexts, qs, refs, positions, seg_of = [], [], [], [], []
    for s, (L, n) in enumerate(shapes):
        k = torch.randn(L, kvh, hd, generator=g).to(dtype).float()
        v = torch.randn(L, kvh, hd, generator=g).to(dtype).float()
        q = torch.randn(n, heads, hd, generator=g).to(dtype).float()
        if needle and L > 40:   # one far key that must dominate head 0 of the last query
            k[3, 0] = 6.0 * q[-1, 0] / q[-1, 0].norm() * math.sqrt(hd) / math.sqrt(hd) * 1.0
            k[3, 0] = k[3, 0].to(dtype).float()
            v[3, 0] = 5.0
        if needle and window:
            _plant_window_edges(q, k, v, L, n, window, dtype)
        q_full = torch.zeros(L, heads, hd)
        q_full[L - n:] = q
        ref = P.attention_scores(q_full.double(), k.double(), v.double(), window)[L - n:]
        contexts.append((k, v)); qs.append(q.reshape(n, heads * hd)); refs.append(ref)
        positions += list(range(L - n, L)); seg_of += [s] * n
    view, _ = _paged(contexts, page_size, dtype, seed)
    return (torch.cat(qs).to(dtype).to(DEV), view, torch.tensor(positions, dtype=torch.int32, device=DEV),
            torch.tensor(seg_of, dtype=torch.int32, device=DEV), torch.cat(refs), shapes)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 10])
def test_attention_generic(status, dtype, window):
    from inference_bench_b200.kernels import ops
    heads, kvh, hd = 6, 3, 24
    q, view, pos, seg, ref, _ = _attention_case(dtype, heads, kvh, hd, 8, window, [(50, 50), (37, 1), (20, 3), (200, 2)], 11, needle=True)
    out = torch.empty_like(q)
    ops.attention_generic(q, view, pos, seg, window, 1 / math.sqrt(hd), out, heads, status)
    assert status.item() == 0
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    assert (out.cpu().double() - ref).abs().max() <= tol * ref.abs().max()


@pytest.mark.parametrize("hd,heads,kvh,page", [(128, 8, 2, 16), (64, 5, 1, 32), (128, 16, 1, 16), (64, 4, 4, 8), (128, 8, 2, 128), (64, 4, 2, 64), (128, 4, 1, 192)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("prefill", ["ws", "tcgen05"])
def test_attention_tensor_core_kernels(status, hd, heads, kvh, page, window, prefill):
    """Decode slices and prefill tiles (either prefill kernel) through the engine's dispatch, against the plain reference."""
    from inference_bench_b200.config.runtime_options import RuntimeOptions
    from inference_bench_b200.engine.context import Segment, build_context
    from inference_bench_b200.engine.runtime import Runtime
    from inference_bench_b200.kernels import attention
    shapes = [(300, 300), (500, 70), (1000, 1), (129, 1), (128, 1), (5, 2), (260, 1), (64, 64), (65, 65)]
    q, view, pos, seg, ref, _ = _attention_case(torch.bfloat16, heads, kvh, hd, page, window, shapes, 12, needle=True)
    rt = Runtime(DEV, options=RuntimeOptions(prefill_attention=prefill))
    segs = [Segment(i, i, L - n, [0] * n) for i, (L, n) in enumerate(shapes)]
    ctx = build_context(rt, segs)
    assert torch.equal(ctx.positions, pos) and torch.equal(ctx.seg_of_token, seg)
    assert attention.has_tensor_core_kernel(q.dtype, hd, heads, kvh)
    out = attention.paged_attention(ctx, q, view, heads, window, 1 / math.sqrt(hd))
    rt.check_status()
    err = (out.cpu().double() - ref).abs()
    assert err.max() <= 1.5e-2 * ref.abs().max(), f"row {int(err.max(dim=1).values.argmax())} is off by {err.max():.3e}"
    # the generic kernel gives the same up to rounding
    from inference_bench_b200.kernels import ops
    out2 = torch.empty_like(q)
    ops.attention_generic(q, view, pos, seg, window, 1 / math.sqrt(hd), out2, heads, status)
    assert (out2.float() - out.float()).abs().max() <= 2e-2 * ref.abs().max()


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_attention_random_shapes(status, seed):
    """Random mixes of prompt portions and decoded tokens through the dispatch that serving uses (head sizes, groups, page
    sizes, windows and lengths drawn at random, lengths around tile and page edges included), against the plain reference."""
    import random
    from inference_bench_b200.engine.context import Segment, build_context
    from inference_bench_b200.engine.runtime import Runtime
    from inference_bench_b200.kernels import attention
    rng = random.Random(seed)
    for case in range(8):
        hd = rng.choice([64, 128])
        kvh = rng.choice([1, 2, 4])
        heads = kvh * rng.choice([1, 2, 4, 7])
        page = rng.choice([8, 16, 32, 64, 128])
        window = rng.choice([None, None, rng.randint(3, 400)])
        shapes = []
        for _ in range(rng.randint(1, 5)):
            L = rng.choice([1, 2, 63, 64, 65, 127, 128, 129, 191, 192, 193, rng.randint(1, 1100), rng.randint(1500, 3000)])
            shapes.append((L, rng.choice([1, 1, L, rng.randint(1, L)])))
        q, view, pos, seg, ref, _ = _attention_case(torch.bfloat16, heads, kvh, hd, page, window, shapes, 1000 * seed + case, needle=True)
        rt = Runtime(DEV)
        ctx = build_context(rt, [Segment(i, i, L - n, [0] * n) for i, (L, n) in enumerate(shapes)])
        out = attention.paged_attention(ctx, q, view, heads, window, 1 / math.sqrt(hd))
        rt.check_status()
        err = (out.cpu().double() - ref).abs()
        assert err.max() <= 1.5e-2 * ref.abs().max(), f"case {case} (hd {hd}, heads {heads}/{kvh}, page {page}, window {window}, {shapes}): row {int(err.max(dim=1).values.argmax())} is off by {err.max():.3e}"


@pytest.mark.parametrize("tiles_per_slice", [1, 2, 8])
@pytest.mark.parametrize("kernel,page,hd", [("stream", 16, 128), ("stream", 64, 64), ("stream", 8, 128), ("stream", 128, 128), ("stream", 32, 64),
                                            ("auto", 24, 64), ("split", 16, 128), ("split", 64, 64), ("split", 8, 128), ("split", 24, 64), ("split", 128, 64)])
def test_attention_decode_slices_of_several_tiles(status, monkeypatch, tiles_per_slice, kernel, page, hd):
    """Both decode kernels (CTAs that stay and a ring filled by TMA; one CTA per slice, filled by cp.async)
    walking 1, 2 or 8 tiles per slice, windows starting inside a slice included. A page size of 24 can only
    be copied by cp.async, so "auto" takes the kernel with one CTA per slice there (and "stream" refuses it)."""
    from inference_bench_b200.config.runtime_options import RuntimeOptions
    from inference_bench_b200.engine.context import Segment, build_context
    from inference_bench_b200.engine.runtime import Runtime
    from inference_bench_b200.kernels import attention
    from inference_bench_b200.kernels import lib as L
    options = RuntimeOptions(decode_attention=kernel, stream_tiles_per_slice=tiles_per_slice, split_tiles_per_slice=tiles_per_slice)
    called = []
    real_call = L.call
    monkeypatch.setattr(L, "call", lambda name, *a: (called.append(name), real_call(name, *a))[1])
    heads, kvh = 8, 2
    shapes = [(1000, 1), (64, 1), (65, 1), (513, 1), (1, 1), (2047, 1), (128, 1), (192, 1), (193, 1)]
    for window in (None, 300):
        q, view, pos, seg, ref, _ = _attention_case(torch.bfloat16, heads, kvh, hd, page, window, shapes, 21, needle=True)
        assert (view.tma()[0] is not None) == (page != 24)
        rt = Runtime(DEV, options=options)
        ctx = build_context(rt, [Segment(i, i, L_ - n, [0] * n) for i, (L_, n) in enumerate(shapes)])
        out = attention.paged_attention(ctx, q, view, heads, window, 1 / math.sqrt(hd))
        rt.check_status()
        err = (out.cpu().double() - ref).abs()
        assert err.max() <= 1.5e-2 * ref.abs().max(), f"row {int(err.max(dim=1).values.argmax())} is off by {err.max():.3e}"
    assert called[-1] == ("ib_attention_decode_stream" if kernel == "stream" else "ib_attention_decode")
    if page == 24:
        with pytest.raises(L.KernelError, match="page size"):
            attention.paged_attention(build_context(Runtime(DEV, options=RuntimeOptions(decode_attention="stream")), [Segment(0, 0, 999, [0])]),
                                      q[:1], view, heads, None, 1 / math.sqrt(hd))


def test_attention_decode_stream_many_units_per_cta(status):
    """More units than CTAs that fit the device, with contexts of very different lengths: every CTA
    of the streaming kernel walks several units, and its ring runs across their ends."""
    from inference_bench_b200.config.runtime_options import RuntimeOptions
    from inference_bench_b200.engine.context import Segment, build_context
    from inference_bench_b200.engine.runtime import Runtime
    from inference_bench_b200.kernels import attention
    heads, kvh, hd, page = 8, 8, 128, 16
    shapes = [(L_, 1) for L_ in (1500, 3, 700, 64, 1100, 129, 1, 900, 1300, 450, 31, 640)]
    for fixed, window in ((1, None), (0, None), (0, 500), (0, 70)):   # slices of one tile at fixed places; each token's keys in equal parts
        rt = Runtime(DEV, options=RuntimeOptions(stream_tiles_per_slice=fixed))
        q, view, pos, seg, ref, _ = _attention_case(torch.bfloat16, heads, kvh, hd, page, window, shapes, 22, needle=True)
        ctx = build_context(rt, [Segment(i, i, L_ - n, [0] * n) for i, (L_, n) in enumerate(shapes)])
        out = attention.paged_attention(ctx, q, view, heads, window, 1 / math.sqrt(hd))
        rt.check_status()
        err = (out.cpu().double() - ref).abs()
        assert err.max() <= 1.5e-2 * ref.abs().max(), f"row {int(err.max(dim=1).values.argmax())} is off by {err.max():.3e}"


@pytest.mark.parametrize("n_dec,kv_heads,max_keys,want", [(8, 8, 4096, 4), (1, 8, 2048, 16), (64, 8, 4096, 4), (1, 8, 100, 1), (300, 1, 4096, 6), (37, 8, 65536, 1)])
def test_stream_slices(n_dec, kv_heads, max_keys, want):
    from inference_bench_b200.kernels import attention
    if torch.cuda.get_device_properties(DEV).multi_processor_count == 148:
        assert attention.stream_slices(n_dec, kv_heads, max_keys, 148) == want


@pytest.mark.parametrize("kernels", [("stream", "ws"), ("split", "tcgen05")])
@pytest.mark.parametrize("hd,page", [(128, 16), (64, 64)])
def test_window_edges_on_tile_slice_and_page_boundaries(status, kernels, hd, page):
    """Windows chosen so that the oldest visible key of the decoded token (and of a prompt portion's last row) is the
    first or the last key of a 64-key tile, of a slice and of a page, with the keys on both sides of the edge made loud
    (see _plant_window_edges): the plain float64 attention on one side, the tensor-core kernels on the other."""
    from inference_bench_b200.config.runtime_options import RuntimeOptions
    from inference_bench_b200.engine.context import Segment, build_context
    from inference_bench_b200.engine.runtime import Runtime
    from inference_bench_b200.kernels import attention
    decode, prefill = kernels
    heads, kvh = 8, 2
    L_ = 1000
    for edge in (64, 63, 128, 127, 512, 511, 16, 15, 1, 936):       # position of the oldest visible key of the last query
        window = L_ - edge
        for tps in (0, 1, 2):
            rt = Runtime(DEV, options=RuntimeOptions(decode_attention=decode, prefill_attention=prefill, stream_tiles_per_slice=tps,
                                                     split_tiles_per_slice=max(tps, 1)))
            shapes = [(L_, 1), (L_, 200), (L_, 129)]
            q, view, pos, seg, ref, _ = _attention_case(torch.bfloat16, heads, kvh, hd, page, window, shapes, 50 + edge, needle=True)
            ctx = build_context(rt, [Segment(i, i, L - n, [0] * n) for i, (L, n) in enumerate(shapes)])
            out = attention.paged_attention(ctx, q, view, heads, window, 1 / math.sqrt(hd))
            rt.check_status()
            err = (out.cpu().double() - ref).abs()
            assert ref.abs().max() > 5.0        # the planted edge key dominates somewhere
            assert err.max() <= 1.5e-2 * ref.abs().max(), f"edge {edge}, {tps} tiles a slice: row {int(err.max(dim=1).values.argmax())} is off by {err.max():.3e}"


@pytest.mark.parametrize("hd,page,window", [(128, 16, 300), (64, 64, 937), (128, 64, 64), (64, 8, 129)])
def test_attention_decode_fused_window_edges(status, hd, page, window):
    """The fused decode kernel (no norms, no rotation, so the queries are the projection's own values) with the keys on both
    sides of each token's window edge made loud, against the plain float64 attention."""
    from inference_bench_b200.config.runtime_options import RuntimeOptions
    from inference_bench_b200.engine.context import Segment, build_context
    from inference_bench_b200.engine.runtime import Runtime
    from inference_bench_b200.kernels import attention
    heads, kvh = 8, 2
    lengths = [1000, 513, 2047, 700, window + 1, window + 2]
    g = _g(61)
    contexts, qs, refs = [], [], []
    R = (heads + 2 * kvh) * hd
    qkv = torch.zeros(1, len(lengths), R)
    for s, L_ in enumerate(lengths):
        k = torch.randn(L_, kvh, hd, generator=g).to(torch.bfloat16).float()
        v = torch.randn(L_, kvh, hd, generator=g).to(torch.bfloat16).float()
        q = torch.randn(1, heads, hd, generator=g).to(torch.bfloat16).float()
        planted = _plant_window_edges(q, k, v, L_, 1, window, torch.bfloat16)
        assert planted == (1 if L_ - 1 - window >= 0 else 0)
        qkv[0, s] = torch.cat([q.reshape(-1), k[-1].reshape(-1), v[-1].reshape(-1)])      # the token's own key and value come from the projection
        q_full = torch.zeros(L_, heads, hd, dtype=torch.float64)
        q_full[-1] = q[0].double()
        refs.append(P.attention_scores(q_full, k.double(), v.double(), window)[-1])
        k2, v2 = k.clone(), v.clone()
        k2[-1], v2[-1] = 31.0, 31.0                                                        # what the cache holds there before the step: must be overwritten
        contexts.append((k2, v2))
    view, _ = _paged(contexts, page, torch.bfloat16, 62)
    rt = Runtime(DEV, options=RuntimeOptions(fuse_decode_max_pairs=1 << 30))
    ctx = build_context(rt, [Segment(i, i, L_ - 1, [0]) for i, L_ in enumerate(lengths)])
    out = attention.decode_fused(ctx, qkv.to(DEV), None, None, 1e-5, None, None, view, heads, window, 1 / math.sqrt(hd), True)
    rt.check_status()
    assert out is not None
    ref = torch.stack(refs)
    err = (out.cpu().double() - ref).abs()
    assert ref.abs().max() > 5.0
    assert err.max() <= 1.5e-2 * ref.abs().max(), f"row {int(err.max(dim=1).values.argmax())} is off by {err.max():.3e}"


@pytest.mark.parametrize("hd,page,heads,kvh,parts,norms,rope,window", [(128, 16, 8, 2, 3, True, True, None), (64, 64, 6, 2, 1, True, True, 300),
                                                                       (128, 64, 16, 1, 2, False, True, None), (64, 8, 4, 4, 2, True, False, 100)])
def test_attention_decode_fused_equals_the_two_steps(status, hd, page, heads, kvh, parts, norms, rope, window):
    """Decoded tokens through the fused kernel (norm, rotation, cache write and attention in one) against
    the q/k kernel followed by the decode kernel, and the cache rows both leave behind."""
    from inference_bench_b200.engine.context import Segment, build_context
    from inference_bench_b200.engine.runtime import Runtime
    from inference_bench_b200.kernels import attention, ops
    lengths = [1000, 64, 65, 513, 1, 2047, 128, 193, 700]           # context lengths with the new token
    shapes = [(L_, 1) for L_ in lengths]
    _, view, pos, seg, _, _ = _attention_case(torch.bfloat16, heads, kvh, hd, page, window, shapes, 31)
    T, R = len(lengths), (heads + 2 * kvh) * hd
    qkv = (torch.randn(parts, T, R, generator=_g(32)) * 0.7).to(DEV)
    qw = (1 + 0.1 * torch.randn(hd, generator=_g(33))).to(DEV) if norms else None
    kw = (1 + 0.1 * torch.randn(hd, generator=_g(34))).to(DEV) if norms else None
    from inference_bench_b200.config.runtime_options import RuntimeOptions
    rt = Runtime(DEV, options=RuntimeOptions(fuse_decode_max_pairs=1 << 30))
    ctx = build_context(rt, [Segment(i, i, L_ - 1, [0]) for i, L_ in enumerate(lengths)])
    cos = sin = None
    if rope:
        inv = (1.0 / torch.pow(torch.tensor(1e4, dtype=torch.float64), torch.arange(0, hd, 2, dtype=torch.float64) / hd)).float().to(DEV)
        cos, sin = torch.empty(T, hd // 2, device=DEV), torch.empty(T, hd // 2, device=DEV)
        ops.rope_table(ctx.positions, inv, cos, sin)
    scale = 1 / math.sqrt(hd)
    view2 = ops.KvLayerView(view.pool.clone(), view.entry, view.block_table)
    q = torch.empty(T, heads * hd, dtype=torch.bfloat16, device=DEV)
    ops.qk_norm_rope_kv(qkv, qw, kw, 1e-5, cos, sin, ctx.positions, ctx.seg_of_token, q, view, heads, rt.status)
    two = attention.paged_attention(ctx, q, view, heads, window, scale)
    ctx.memo = {}
    one = attention.decode_fused(ctx, qkv, qw, kw, 1e-5, cos, sin, view2, heads, window, scale, True)
    rt.check_status()
    assert one is not None
    assert (one.float() - two.float()).abs().max() <= 2.0 ** -7 * two.float().abs().max()
    a, b = view.pool.float(), view2.pool.float()
    assert (a - b).abs().max() <= 2.0 ** -7 * a.abs().max() and not torch.equal(view.pool, _attention_case(torch.bfloat16, heads, kvh, hd, page, window, shapes, 31)[1].pool)
    # a layer that reads another layer's cache must see that layer's key and value at its own position: not for the fused kernel
    assert attention.decode_fused(ctx, qkv, qw, kw, 1e-5, cos, sin, view2, heads, window, scale, False) is None
    # prompt portions in the step: the fused kernel declines
    ctx2 = build_context(rt, [Segment(0, 0, 5, [0, 0, 0])])
    assert attention.decode_fused(ctx2, qkv[:, :3].contiguous(), qw, kw, 1e-5, None if cos is None else cos[:3], None if sin is None else sin[:3], view, heads, window, scale, True) is None


def test_attention_reports_missing_page(status):
    from inference_bench_b200.kernels import ops
    q, view, pos, seg, ref, _ = _attention_case(torch.float32, 2, 1, 16, 8, None, [(30, 1)], 13)
    view.block_table[0, 1] = -1
    out = torch.empty_like(q)
    ops.attention_generic(q, view, pos, seg, None, 0.25, out, 2, status)
    assert status.item() == 1
    status.zero_()


@pytest.mark.parametrize("page", [16, 64])
def test_tensor_core_attention_reports_missing_pages(status, page):
    """A block table entry that is missing or out of range, under the TMA-fed kernels (decode, fused decode,
    prompt portions): the status word says so, nothing is read through the bad entry, and the run goes on."""
    from inference_bench_b200.engine.context import Segment, build_context
    from inference_bench_b200.engine.runtime import DeviceStatusError, Runtime
    from inference_bench_b200.kernels import attention, ops
    heads, kvh, hd = 8, 2, 128
    rt = Runtime(DEV, "bfloat16")
    for shapes, bad in (([(300, 1), (200, 1)], -1), ([(300, 1), (200, 1)], 10 ** 6), ([(300, 300)], -1)):
        q, view, pos, seg, ref, _ = _attention_case(torch.bfloat16, heads, kvh, hd, page, None, shapes, 41)
        view.block_table[0, 1] = bad
        ctx = build_context(rt, [Segment(i, i, L_ - n, [0] * n) for i, (L_, n) in enumerate(shapes)])
        out = attention.paged_attention(ctx, q, view, heads, None, 1 / math.sqrt(hd))
        with pytest.raises(DeviceStatusError, match="block table"):
            rt.check_status()
        assert torch.isfinite(out.float()).all()
        if shapes[0][1] == 1:   # the fused decode kernel, whose own position lies on the missing page for the second request
            view.block_table[1, (200 - 1) // page] = bad
            qkv = torch.randn(1, len(shapes), (heads + 2 * kvh) * hd, device=DEV)
            ctx.memo = {}
            out = attention.decode_fused(ctx, qkv, None, None, 1e-5, None, None, view, heads, None, 1 / math.sqrt(hd), True)
            assert out is not None
            with pytest.raises(DeviceStatusError, match="block table"):
                rt.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,rot,T", [(24, 24, 21), (64, 32, 21), (16, 0, 21), (64, 64, 21), (128, 128, 21), (128, 0, 21), (128, 128, 1031), (64, 64, 1100),
                                      (64, 0, 1025)])   # more than 8,192 (token, head) items: four per warp
def test_qk_norm_rope_kv(status, dtype, hd, rot, T):
    from inference_bench_b200.kernels import ops
    heads, kvh, page = 4, 2, 8
    R = (heads + 2 * kvh) * hd
    qkv = torch.randn(2, T, R, generator=_g(14))
    qw = 1 + 0.1 * torch.randn(hd, generator=_g(15))
    kw = 1 + 0.1 * torch.randn(hd, generator=_g(16))
    eps, theta, pos0 = 1e-5, 1e4, 13
    positions = torch.arange(pos0, pos0 + T, dtype=torch.int32)
    view, table = _paged([(torch.zeros(pos0 + T, kvh, hd), torch.zeros(pos0 + T, kvh, hd))], page, dtype, 17)
    cos = sin = None
    if rot:
        inv = (1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float().to(DEV)
        cos = torch.empty(T, rot // 2, device=DEV)
        sin = torch.empty(T, rot // 2, device=DEV)
        ops.rope_table(positions.to(DEV), inv, cos, sin)
    q_out = torch.empty(T, heads * hd, dtype=dtype, device=DEV)
    ops.qk_norm_rope_kv(qkv.to(DEV), qw.to(DEV), kw.to(DEV), eps, cos, sin, positions.to(DEV), torch.zeros(T, dtype=torch.int32, device=DEV), q_out,
                        view, heads, status)
    assert status.item() == 0
    s = qkv.double().sum(0)
    q = P.rmsnorm(s[:, :heads * hd].reshape(T, heads, hd), qw.double(), eps)
    k = P.rmsnorm(s[:, heads * hd:(heads + kvh) * hd].reshape(T, kvh, hd), kw.double(), eps)
    v = s[:, (heads + kvh) * hd:].reshape(T, kvh, hd)
    if rot and T < 100:
        q = torch.cat([P.rope_neox(q[..., :rot], positions, theta), q[..., rot:]], -1)
        k = torch.cat([P.rope_neox(k[..., :rot], positions, theta), k[..., rot:]], -1)
    elif rot:   # far positions: float32 angles (what the tables hold, by design) differ from float64 ones by more than this test's tolerance; turn by the tables
        c, sn = cos.cpu().double()[:, None, :], sin.cpu().double()[:, None, :]
        turn = lambda x: torch.cat([x[..., :rot // 2] * c - x[..., rot // 2:rot] * sn, x[..., rot // 2:rot] * c + x[..., :rot // 2] * sn, x[..., rot:]], -1)
        q, k = turn(q), turn(k)
    tol = 2e-5 if dtype == torch.float32 else 2.0 ** -7
    assert (q_out.cpu().double().reshape(T, heads, hd) - q).abs().max() <= tol * q.abs().max()
    pool = view.pool.cpu().double()
    for t in range(T):
        p = pos0 + t
        pg = table[0, p // page]
        assert (pool[1, pg, 0, :, p % page] - k[t]).abs().max() <= tol * k.abs().max()
        assert (pool[1, pg, 1, :, p % page] - v[t]).abs().max() <= tol * v.abs().max()
    assert (pool[0] == 37.0).all()   # the other layer's place in the pages is untouched


@pytest.mark.parametrize("T,heads,kvh,K,norms,rope,write_kv", [(300, 3, 1, 200, True, True, True), (130, 4, 2, 264, False, True, True),
                                                              (513, 2, 2, 1024, True, False, True), (257, 5, 1, 136, True, True, False)])
def test_gemm_qkv_epilogue_equals_the_two_steps(status, T, heads, kvh, K, norms, rope, write_kv):
    """The q/k/v projection with norm, rotation and cache write in its epilogue against the plain product followed by
    `qk_norm_rope_kv`, and against the float64 formulas: two requests at different positions, a number of heads that
    leaves the last tile half empty, a token count that is no multiple of the tile."""
    from inference_bench_b200.kernels import gemm_tcgen05 as G, ops
    hd, page, theta, eps = 128, 16, 1e4, 1e-5
    N = (heads + 2 * kvh) * hd
    x = (torch.randn(T, K, generator=_g(51)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=_g(52)) * 0.2).to(torch.bfloat16).to(DEV)
    qw = (1 + 0.1 * torch.randn(hd, generator=_g(53))).to(DEV) if norms else None
    kw = (1 + 0.1 * torch.randn(hd, generator=_g(54))).to(DEV) if norms else None
    n0 = T // 3
    lens = [(7 + n0, n0), (40 + T - n0, T - n0)]   # (context length after the step, tokens of the step)
    positions = torch.cat([torch.arange(L_ - n, L_, dtype=torch.int32) for L_, n in lens]).to(DEV)
    seg = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, (L_, n) in enumerate(lens)]).to(DEV)
    cos = sin = None
    if rope:
        inv = (1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), torch.arange(0, hd, 2, dtype=torch.float64) / hd)).float().to(DEV)
        cos, sin = torch.empty(T, hd // 2, device=DEV), torch.empty(T, hd // 2, device=DEV)
        ops.rope_table(positions, inv, cos, sin)
    outs = []
    for fused in (False, True):
        view, table = _paged([(torch.zeros(L_, kvh, hd), torch.zeros(L_, kvh, hd)) for L_, _ in lens], page, torch.bfloat16, 55)
        q = torch.full((T, heads * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        before = view.pool.float().cpu()
        if fused:
            G.gemm_qkv_pair(x, w, q, view, heads, qw, kw, eps, cos, sin, positions, seg, write_kv, status)
        else:
            qkv = torch.empty(1, T, N, device=DEV)
            G.gemm_pair(x, w, qkv[0], status)
            ops.qk_norm_rope_kv(qkv, qw, kw, eps, cos, sin, positions, seg, q, view, heads, status, write_kv=write_kv)
        assert status.item() == 0
        outs.append((q.float().cpu(), view.pool.float().cpu(), table))
    (q_a, pool_a, table), (q_b, pool_b, _) = outs
    # the two ways differ by the order of a float32 sum at most: a bfloat16 value may round the other way
    assert (q_a - q_b).abs().max() <= 2.0 ** -7 * q_a.abs().max()
    assert (pool_a - pool_b).abs().max() <= 2.0 ** -7 * max(pool_a[1].abs().max(), 1.0)
    assert (pool_b[0] == 37.0).all()
    if not write_kv:
        assert torch.equal(pool_a, before) and torch.equal(pool_b, before)
    # and against the formulas in float64
    s_ = x.cpu().double() @ w.cpu().double().T
    qr = s_[:, :heads * hd].reshape(T, heads, hd)
    kr = s_[:, heads * hd:(heads + kvh) * hd].reshape(T, kvh, hd)
    vr = s_[:, (heads + kvh) * hd:].reshape(T, kvh, hd)
    if norms:
        qr, kr = P.rmsnorm(qr, qw.cpu().double(), eps), P.rmsnorm(kr, kw.cpu().double(), eps)
    if rope:
        c, sn = cos.cpu().double()[:, None, :], sin.cpu().double()[:, None, :]
        turn = lambda z: torch.cat([z[..., :hd // 2] * c - z[..., hd // 2:] * sn, z[..., hd // 2:] * c + z[..., :hd // 2] * sn], -1)
        qr, kr = turn(qr), turn(kr)
    assert (q_b.double().reshape(T, heads, hd) - qr).abs().max() <= 2.0 ** -7 * qr.abs().max()
    if write_kv:
        pos = positions.cpu().tolist()
        sg = seg.cpu().tolist()
        for t in range(0, T, 7):
            pg = table[sg[t], pos[t] // page]
            assert (pool_b[1, pg, 0, :, pos[t] % page].double() - kr[t]).abs().max() <= 2.0 ** -7 * kr.abs().max()
            assert (pool_b[1, pg, 1, :, pos[t] % page].double() - vr[t]).abs().max() <= 2.0 ** -7 * vr.abs().max()


# ------------------------------------------------------------------------------------------ sampling
def test_sample_rows_matches_plain():
    from inference_bench_b200.kernels import ops
    from inference_bench_b200.sampling.params import SamplingParams
    V = 1003
    logits = torch.randn(8, V, generator=_g(18)) * 3
    logits[0, 17] = logits[0, 900] = logits[0].max() + 1     # a tie: the lowest index wins
    params = [SamplingParams(), SamplingParams(temperature=0.7, seed=1), SamplingParams(temperature=1.5, seed=2, top_k=5),
              SamplingParams(temperature=1.0, seed=3, top_p=0.6), SamplingParams(temperature=1.0, seed=4, min_p=0.1),
              SamplingParams(temperature=2.0, seed=5, top_k=50, top_p=0.9, min_p=0.01), SamplingParams(temperature=0.3, seed=2**31 + 5),
              SamplingParams(temperature=1.0, seed=7, top_k=1)]
    steps = [0, 3, 1, 9, 2, 100, 5, 0]
    rows = torch.tensor([p.row(s) for p, s in zip(params, steps)], dtype=torch.int32, device=DEV)
    toks = torch.empty(8, dtype=torch.int32, device=DEV)
    ops.sample_rows(logits.to(DEV), rows, toks)
    want = [P.sample_token(logits[i], p.temperature, p.seed, steps[i], p.top_k, p.top_p, p.min_p) for i, p in enumerate(params)]
    assert toks.cpu().tolist() == want
    assert want[0] == 17 and want[7] == int(logits[7].argmax())
