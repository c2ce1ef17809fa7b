"""Each CUDA kernel alone against a plain float32/float64 computation of the same op, at sizes other
than the engine tests use (widths and vocabularies that are no power of two, every head size in
steps of 16, odd head groups, page sizes 1..64)."""
import math

import numpy as np
import pytest
import torch

from plain import qwen3_plain as P
from plain import sampling_plain as S

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    from imp_b200.ops import kernels, library
    library.require_device()
    return kernels


def decode_reference(qkv, kc0, vc0, bt, lengths, Hq, Hkv, Dh, page, window, qw, kw, theta=1e4, eps=1e-6):
    """One decode step in double precision from the raw q | k | v rows and the cache before the step: per-head
    norm and rotation of q and of the new key, the new key and value appended, one query over its sequence."""
    B, G = len(lengths), Hq // Hkv
    out = torch.zeros(B, Hq, Dh, dtype=torch.float64)
    rows = qkv.double().cpu()
    for s, n in enumerate(lengths):
        q = rows[s, :Hq * Dh].view(1, Hq, Dh)
        k = rows[s, Hq * Dh:(Hq + Hkv) * Dh].view(1, Hkv, Dh)
        v = rows[s, (Hq + Hkv) * Dh:].view(Hkv, Dh)
        if qw is not None:
            q, k = P.rmsnorm(q, qw.double().cpu(), eps), P.rmsnorm(k, kw.double().cpu(), eps)
        q, k = P.rope(q, [n - 1], theta)[0], P.rope(k, [n - 1], theta)[0]
        keys = torch.stack([kc0[int(bt[s, p // page]), :, p % page].double() for p in range(n - 1)] + [k]) if n > 1 else k[None]
        vals = torch.stack([vc0[int(bt[s, p // page]), :, p % page].double() for p in range(n - 1)] + [v]) if n > 1 else v[None]
        lo = max(0, n - window) if window else 0
        for h in range(Hq):
            sc = (keys[lo:, h // G] @ q[h]) / math.sqrt(Dh)
            out[s, h] = torch.softmax(sc, 0) @ vals[lo:, h // G]
    return out


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(got, want, dtype, scale=None):
    got, want = got.float().cpu(), want.float().cpu()
    scale = float(want.abs().max()) if scale is None else scale
    if dtype == torch.float32:
        atol, rtol = 1e-5 * max(scale, 1.0), 1e-5
    else:
        atol, rtol = 0.01 * max(scale, 1e-3), 0.01      # bfloat16 storage: 8 bits of mantissa
    err = (got - want).abs()
    assert (err <= atol + rtol * want.abs()).all(), f"max error {err.max().item():.3g} (scale {scale:.3g})"


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_embedding(K, wdtype):
    V, d = 1003, 200
    table = rnd(V, d, dtype=wdtype).to(DEV)
    ids = torch.tensor([0, 1002, 17, 17, 500], dtype=torch.int32, device=DEV)
    out = torch.empty(5, d, dtype=torch.float32, device=DEV)
    status = K.new_status(DEV)
    K.embedding(out, table, ids, 1.0, status)
    assert torch.equal(out.cpu(), table.float().cpu()[ids.cpu().long()])
    K.embedding(out, table, ids, 2.5, status)
    assert torch.allclose(out.cpu(), table.float().cpu()[ids.cpu().long()] * 2.5)
    K.check_status(status)
    bad = torch.tensor([3, V, 1, 2, 3], dtype=torch.int32, device=DEV)
    K.embedding(out, table, bad, 1.0, status)
    with pytest.raises(Exception, match="token id"):
        K.check_status(status)
    assert (out[1] == 0).all()


# ----------------------------------------------------------------------- norms
@pytest.mark.parametrize("adtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [64, 200, 4096 + 24])
def test_add_rmsnorm(K, adtype, wdtype, d):
    T = 7
    h = rnd(T, d, seed=1, scale=3.0)
    br = rnd(T, d, dtype=adtype, seed=2)
    w = (1 + 0.1 * rnd(d, seed=3)).to(wdtype)
    hd, out = h.clone().to(DEV), torch.empty(T, d, dtype=adtype, device=DEV)
    K.add_rmsnorm(hd, br.to(DEV), w.to(DEV), out, 1e-5)
    hs = h + br.float()
    assert torch.equal(hd.cpu(), hs)                      # the residual sum itself is exact float32
    close(out, P.rmsnorm(hs.double(), w.double(), 1e-5), adtype)
    # no branch; weight offset; eps matters
    K.add_rmsnorm(hd, None, w.to(DEV), out, 0.5, weight_offset=1.0)
    assert torch.equal(hd.cpu(), hs)
    close(out, P.rmsnorm(hs.double(), w.double() + 1.0, 0.5), adtype)
    # gather mode: chosen rows, h untouched, branch still added
    rows = torch.tensor([6, 0, 6, 3], dtype=torch.int32, device=DEV)
    h2 = h.clone().to(DEV)
    out2 = torch.empty(4, d, dtype=adtype, device=DEV)
    K.add_rmsnorm(h2, br.to(DEV), w.to(DEV), out2, 1e-5, rows=rows)
    assert torch.equal(h2.cpu(), h)
    close(out2, P.rmsnorm(hs.double(), w.double(), 1e-5)[rows.cpu().long()], adtype)


@pytest.mark.parametrize("adtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_rows_strided(K, adtype):
    x = rnd(9, 5 * 48, dtype=adtype, seed=4).to(DEV)
    w = (1 + 0.1 * rnd(48, seed=5)).to(DEV)
    view = x.view(9, 5, 48)[:, 2, :]                      # rows 480 apart
    out = torch.empty(9, 48, dtype=adtype, device=DEV)
    K.rmsnorm_rows(view, w, out, 1e-6)
    close(out, P.rmsnorm(view.double().cpu(), w.double().cpu(), 1e-6), adtype)


# ---------------------------------------------------------------------- swiglu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_and_cast(K, dtype):
    T, F = 5, 333
    gu = rnd(T, 2 * F, dtype=dtype, seed=6, scale=3.0).to(DEV)
    out = torch.empty(T, F, dtype=dtype, device=DEV)
    K.swiglu(out, gu)
    g, u = gu.double().cpu()[:, :F], gu.double().cpu()[:, F:]
    close(out, g / (1 + torch.exp(-g)) * u, dtype)
    # interleaved layout: runs of 8 gate columns and 8 up columns alternate
    F8 = 336
    gu8 = rnd(T, 2 * F8, dtype=dtype, seed=8, scale=3.0)
    g8 = gu8.view(T, F8 // 8, 2, 8)[:, :, 0, :].reshape(T, F8).double()
    u8 = gu8.view(T, F8 // 8, 2, 8)[:, :, 1, :].reshape(T, F8).double()
    out8 = K.swiglu(torch.empty(T, F8, dtype=dtype, device=DEV), gu8.to(DEV), 8)
    close(out8, g8 / (1 + torch.exp(-g8)) * u8, dtype)
    src = rnd(1001, seed=7).to(DEV)
    b = K.cast(torch.empty(1001, dtype=torch.bfloat16, device=DEV), src)
    assert torch.equal(b.cpu(), src.cpu().to(torch.bfloat16))
    f = K.cast(torch.empty(1001, dtype=torch.float32, device=DEV), b)
    assert torch.equal(f.cpu(), b.cpu().float())


# ---------------------------------------------------------------------- matmul
@pytest.mark.parametrize("M,N,K_", [(1, 7, 5), (3, 130, 70), (65, 64, 16), (130, 257, 129), (2, 1000, 4100)])
def test_gemm_f32(K, M, N, K_):
    a, w = rnd(M, K_, seed=8).to(DEV), rnd(N, K_, seed=9).to(DEV)
    out = K.gemm_f32(torch.empty(M, N, device=DEV), a, w)
    want = a.double().cpu() @ w.double().cpu().T
    close(out, want, torch.float32)
    # every output is the same bits whatever other rows are in the product
    one = K.gemm_f32(torch.empty(1, N, device=DEV), a[M - 1:M], w)
    assert torch.equal(one[0], out[M - 1])
    # strided operands (a view of a wider buffer)
    wide = torch.zeros(M, K_ + 9, device=DEV)
    wide[:, 3:3 + K_] = a
    out2 = K.gemm_f32(torch.empty(M, N, device=DEV), wide[:, 3:3 + K_], w)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("M", [1, 2, 3, 4, 7, 8, 9, 16])
@pytest.mark.parametrize("N,K_", [(10, 64), (257, 200), (96, 4104), (50, 100)])
@pytest.mark.parametrize("odtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16_small_m(K, M, N, K_, odtype):
    a, w = rnd(M, K_, dtype=torch.bfloat16, seed=10).to(DEV), rnd(N, K_, dtype=torch.bfloat16, seed=11).to(DEV)
    out = K.gemm_bf16_small_m(torch.empty(M, N, dtype=odtype, device=DEV), a, w)
    want = a.double().cpu() @ w.double().cpu().T
    if odtype == torch.float32:
        close(out, want, torch.float32, scale=float(want.abs().max()) * 4)   # float32 sums of bf16 products
    else:
        close(out, want, torch.bfloat16)
    one = K.gemm_bf16_small_m(torch.empty(1, N, dtype=odtype, device=DEV), a[M - 1:M], w)
    assert torch.equal(one[0], out[M - 1])                # the same bits for a row, alone or in a batch


@pytest.mark.parametrize("M", [1, 2, 5, 8, 9, 13, 16])
@pytest.mark.parametrize("N,K_", [(16, 64), (10, 64), (257, 200), (96, 4104), (50, 104), (4096, 1024)])
@pytest.mark.parametrize("odtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16_stream(K, M, N, K_, odtype):
    a, w = rnd(M, K_, dtype=torch.bfloat16, seed=10).to(DEV), rnd(N, K_, dtype=torch.bfloat16, seed=11).to(DEV)
    out = K.gemm_bf16_stream(torch.full((M, N), float("nan"), dtype=odtype, device=DEV), a, w)
    want = a.double().cpu() @ w.double().cpu().T
    if odtype == torch.float32:
        close(out, want, torch.float32, scale=float(want.abs().max()) * 4)
    else:
        close(out, want, torch.bfloat16)
    one = K.gemm_bf16_stream(torch.empty(1, N, dtype=odtype, device=DEV), a[M - 1:M], w)
    assert torch.equal(one[0], out[M - 1])                # the same bits for a row, alone or in a batch
    # operands inside wider buffers (row strides that still allow 16-byte loads)
    wide_w = torch.zeros(N, K_ + 16, dtype=torch.bfloat16, device=DEV)
    wide_w[:, 8:8 + K_] = w
    out2 = K.gemm_bf16_stream(torch.empty(M, N, dtype=odtype, device=DEV), a, wide_w[:, 8:8 + K_])
    assert torch.equal(out2, out)


@pytest.mark.parametrize("M", [1, 3, 8, 11, 16, 40])
@pytest.mark.parametrize("F,K_", [(8, 64), (200, 96), (3072, 1024), (24, 100)])
def test_linear_swiglu_fused(K, M, F, K_):
    x = rnd(M, K_, dtype=torch.bfloat16, seed=30).to(DEV)
    wg = rnd(F, K_, dtype=torch.bfloat16, seed=31, scale=0.3).to(DEV)
    wu = rnd(F, K_, dtype=torch.bfloat16, seed=32, scale=0.3).to(DEV)
    w = K.interleave_gate_up(wg, wu)
    assert torch.equal(w[:8], wg[:8]) and torch.equal(w[8:16], wu[:8])
    out = K.linear_swiglu(torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV), x, w)
    g = x.double().cpu() @ wg.double().cpu().T
    u = x.double().cpu() @ wu.double().cpu().T
    close(out, g / (1 + torch.exp(-g)) * u, torch.bfloat16)


@pytest.mark.parametrize("M,N,K_", [(128, 256, 64), (1, 8, 8), (130, 264, 72), (300, 520, 200), (257, 1000, 4104),
                                    (2048, 512, 1024)])
@pytest.mark.parametrize("odtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16_tcgen05(K, M, N, K_, odtype):
    """TMA-fed tcgen05 product: tiles cut by the matrix edges in every dimension, both output types."""
    a, w = rnd(M, K_, dtype=torch.bfloat16, seed=40).to(DEV), rnd(N, K_, dtype=torch.bfloat16, seed=41).to(DEV)
    status = K.new_status(DEV)
    out = torch.full((M, N), float("nan"), dtype=odtype, device=DEV)
    assert K.gemm_bf16_tc(out, a, w, None, status)
    K.check_status(status)
    want = a.double().cpu() @ w.double().cpu().T
    if odtype == torch.float32:
        close(out, want, torch.float32, scale=float(want.abs().max()) * 8)   # float32 sums of bf16 products
    else:
        close(out, want, torch.bfloat16)
    # operands inside wider buffers, output into a wider buffer
    wide_a = torch.zeros(M, K_ + 24, dtype=torch.bfloat16, device=DEV)
    wide_a[:, 8:8 + K_] = a
    wide_o = torch.full((M, N + 16), 7.0, dtype=odtype, device=DEV)
    assert K.gemm_bf16_tc(wide_o[:, 8:8 + N], wide_a[:, 8:8 + K_], w, None, status)
    K.check_status(status)
    assert torch.equal(wide_o[:, 8:8 + N], out) and (wide_o[:, :8] == 7).all() and (wide_o[:, 8 + N:] == 7).all()
    # a row stride that does not allow 16-byte tensor copies is declined, not mangled
    odd = torch.zeros(M, K_ + 3, dtype=torch.bfloat16, device=DEV)
    assert not K.gemm_bf16_tc(out, odd[:, :K_], w, None, status)


@pytest.mark.parametrize("M", [1, 8, 17, 32, 33, 64, 65, 100, 128])
@pytest.mark.parametrize("N,K_", [(128, 64), (130, 72), (1000, 4104), (4096, 1024), (200, 12288), (260, 2560)])
@pytest.mark.parametrize("odtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16_tcgen05_few_rows(K, M, N, K_, odtype):
    """Weights on the M side of the MMA, K split over CTAs: every edge case of rows, columns and K."""
    a, w = rnd(M, K_, dtype=torch.bfloat16, seed=50).to(DEV), rnd(N, K_, dtype=torch.bfloat16, seed=51).to(DEV)
    status = K.new_status(DEV)
    out = torch.full((M, N), float("nan"), dtype=odtype, device=DEV)
    assert K.gemm_bf16_tc_swap(out, a, w, None, status)
    K.check_status(status)
    want = a.double().cpu() @ w.double().cpu().T
    if odtype == torch.float32:
        close(out, want, torch.float32, scale=float(want.abs().max()) * 8)
    else:
        close(out, want, torch.bfloat16)
    again = torch.empty_like(out)
    assert K.gemm_bf16_tc_swap(again, a, w, None, status) and torch.equal(again, out)   # split sums have a fixed order


@pytest.mark.parametrize("M,F,K_", [(20, 136, 96), (64, 3072, 1024), (128, 8, 64)])
def test_gemm_bf16_tcgen05_few_rows_fused_swiglu(K, M, F, K_):
    x = rnd(M, K_, dtype=torch.bfloat16, seed=52).to(DEV)
    wg = rnd(F, K_, dtype=torch.bfloat16, seed=53, scale=0.3).to(DEV)
    wu = rnd(F, K_, dtype=torch.bfloat16, seed=54, scale=0.3).to(DEV)
    status = K.new_status(DEV)
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert K.gemm_bf16_tc_swap(out, x, K.interleave_gate_up(wg, wu), K.TC_OUT_SWIGLU, status)
    K.check_status(status)
    g = x.double().cpu() @ wg.double().cpu().T
    u = x.double().cpu() @ wu.double().cpu().T
    close(out, g / (1 + torch.exp(-g)) * u, torch.bfloat16)


@pytest.mark.parametrize("M,F,K_", [(200, 136, 96), (2048, 3072, 1024), (33, 8, 64)])
def test_gemm_bf16_tcgen05_fused_swiglu(K, M, F, K_):
    x = rnd(M, K_, dtype=torch.bfloat16, seed=42).to(DEV)
    wg = rnd(F, K_, dtype=torch.bfloat16, seed=43, scale=0.3).to(DEV)
    wu = rnd(F, K_, dtype=torch.bfloat16, seed=44, scale=0.3).to(DEV)
    status = K.new_status(DEV)
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert K.gemm_bf16_tc(out, x, K.interleave_gate_up(wg, wu), K.TC_OUT_SWIGLU, status)
    K.check_status(status)
    g = x.double().cpu() @ wg.double().cpu().T
    u = x.double().cpu() @ wu.double().cpu().T
    close(out, g / (1 + torch.exp(-g)) * u, torch.bfloat16)


@pytest.mark.parametrize("M,N,K_", [(512, 4096, 12288), (300, 1024, 6144), (256, 520, 9224), (1000, 2048, 6208), (160, 2048, 6208)])
@pytest.mark.parametrize("odtype", [torch.bfloat16, torch.float32])
def test_linear_with_the_k_range_in_parts(K, M, N, K_, odtype):
    """A portion of a prompt times a weight with few rows and a long K: fewer 256 x 256 tiles than half the CTA pairs,
    so the library cuts K into parts that are units of work of their own and adds the partial products in order.  The
    ragged cases: rows and columns that do not fill tiles, a K that the parts do not divide."""
    from imp_b200.ops import library as L
    assert L.load().imp_gemm_bf16_tc_splits(M, N, K_) >= 2
    a, w = rnd(M, K_, dtype=torch.bfloat16, seed=60).to(DEV), (rnd(N, K_, dtype=torch.bfloat16, seed=61) * 0.05).to(DEV)
    out = K.linear(torch.full((M, N), float("nan"), dtype=odtype, device=DEV), a, w)
    want = a.double().cpu() @ w.double().cpu().T
    if odtype == torch.float32:
        close(out, want, torch.float32, scale=float(want.abs().max()) * 8)
    else:
        close(out, want, torch.bfloat16)
    before = K.fallback_calls()
    K.linear(out, a, w)
    assert K.fallback_calls() == before
    # the same product the same way twice: the same bits (the parts are added in a fixed order)
    again = K.linear(torch.empty_like(out), a, w)
    assert torch.equal(out, again)


def test_linear_dispatch(K):
    x = rnd(40, 96, dtype=torch.bfloat16, seed=12).to(DEV)
    w = rnd(50, 96, dtype=torch.bfloat16, seed=13).to(DEV)
    want = x.double().cpu() @ w.double().cpu().T
    close(K.linear(torch.empty(40, 50, dtype=torch.bfloat16, device=DEV), x, w), want, torch.bfloat16)
    close(K.linear(torch.empty(40, 50, dtype=torch.float32, device=DEV), x, w), want, torch.float32, scale=40.0)
    close(K.linear(torch.empty(3, 50, dtype=torch.float32, device=DEV), x[:3], w), want[:3], torch.float32, scale=40.0)
    # a weight the checkpoint stores in 32 bits stays so: the product runs in float32
    w32 = rnd(50, 96, seed=14).to(DEV)
    want32 = x.double().cpu() @ w32.double().cpu().T
    close(K.linear(torch.empty(40, 50, dtype=torch.float32, device=DEV), x, w32), want32, torch.float32)
    close(K.linear(torch.empty(40, 50, dtype=torch.bfloat16, device=DEV), x, w32), want32, torch.bfloat16)


# ---------------------------------------------------- q/k norm + rotary + cache write
def paged_layout(lengths, page_size, n_extra_pages=3, seed=0):
    """A shuffled assignment of pages to sequences: (block table [B, max_pages] with -1 padding, num_pages)."""
    rng = np.random.default_rng(seed)
    need = [(n + page_size - 1) // page_size for n in lengths]
    num_pages = sum(need) + n_extra_pages
    perm = rng.permutation(num_pages)
    bt = -np.ones((len(lengths), max(need) + 2), dtype=np.int32)
    k = 0
    for s, n in enumerate(need):
        bt[s, :n] = perm[k:k + n]
        k += n
    return torch.from_numpy(bt), num_pages


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,Dh,rot,page", [(4, 2, 16, 16, 4), (6, 3, 32, 32, 16), (5, 5, 48, 24, 3), (8, 1, 128, 128, 16),
                                                (2, 1, 256, 256, 16), (3, 1, 80, 40, 5), (2, 2, 16, 6, 4)])
def test_qk_norm_rope_kv_write(K, dtype, Hq, Hkv, Dh, rot, page):
    lengths = [11, 1, 30]
    starts = [4, 0, 17]                                    # tokens of this step continue sequences at these positions
    bt, num_pages = paged_layout(lengths, page)
    toks = [(s, p) for s, (st, n) in enumerate(zip(starts, lengths)) for p in range(st, n)]
    T = len(toks)
    seq = torch.tensor([s for s, _ in toks], dtype=torch.int32)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32)
    width = (Hq + 2 * Hkv) * Dh
    qkv = rnd(T, width, dtype=dtype, seed=15)
    qw, kw = (1 + 0.2 * rnd(Dh, seed=16)), (1 + 0.2 * rnd(Dh, seed=17))
    max_pos = 64
    i = torch.arange(rot // 2, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (1e4 ** (-2.0 * i / rot))[None, :]
    cos, sin = ang.cos().float(), ang.sin().float()
    kc = torch.zeros(num_pages, Hkv, page, Dh, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    status = K.new_status(DEV)
    qd = qkv.clone().to(DEV)
    K.qk_norm_rope_kv_write(qd, Hq, Hkv, Dh, qw.to(DEV), kw.to(DEV), 1e-6, cos.to(DEV), sin.to(DEV), rot,
                            pos.to(DEV), seq.to(DEV), bt.to(DEV), kc, vc, status)
    K.check_status(status)
    x = qkv.double()
    q = P.rmsnorm(x[:, :Hq * Dh].view(T, Hq, Dh), qw.double(), 1e-6)
    k = P.rmsnorm(x[:, Hq * Dh:(Hq + Hkv) * Dh].view(T, Hkv, Dh), kw.double(), 1e-6)
    v = x[:, (Hq + Hkv) * Dh:].view(T, Hkv, Dh)

    def rot_part(z):
        return torch.cat([P.rope(z[..., :rot].contiguous(), pos.tolist(), 1e4), z[..., rot:]], dim=-1)
    q, k = rot_part(q), rot_part(k)
    close(qd[:, :Hq * Dh].view(T, Hq, Dh), q, dtype)
    assert torch.equal(qd[:, (Hq + Hkv) * Dh:].cpu(), qkv[:, (Hq + Hkv) * Dh:])     # v is left in place
    kc_c, vc_c = kc.cpu(), vc.cpu()
    touched = torch.zeros(num_pages, page, dtype=torch.bool)
    for n, (s, p) in enumerate(toks):
        pg, sl = int(bt[s, p // page]), p % page
        close(kc_c[pg, :, sl, :], k[n], dtype)
        assert torch.equal(vc_c[pg, :, sl, :].double(), v[n])
        touched[pg, sl] = True
    assert (kc_c[~touched.unsqueeze(1).expand(-1, Hkv, -1)] == 0).all()             # nothing else was written
    # without norm weights and without a table: plain copy of k and v into the pages
    kc.zero_(); vc.zero_()
    qd = qkv.clone().to(DEV)
    K.qk_norm_rope_kv_write(qd, Hq, Hkv, Dh, None, None, 1e-6, None, None, 0, pos.to(DEV), seq.to(DEV), bt.to(DEV),
                            kc, vc, status)
    n, (s, p) = T - 1, toks[-1]
    assert torch.equal(kc.cpu()[int(bt[s, p // page]), :, p % page, :].reshape(-1), qkv[n, Hq * Dh:(Hq + Hkv) * Dh])
    assert torch.equal(qd.cpu()[:, :Hq * Dh], qkv[:, :Hq * Dh])
    # a position outside the table and a page outside the pool are reported, not written
    badpos = pos.clone(); badpos[0] = max_pos
    K.qk_norm_rope_kv_write(qd, Hq, Hkv, Dh, qw.to(DEV), kw.to(DEV), 1e-6, cos.to(DEV), sin.to(DEV), rot,
                            badpos.to(DEV), seq.to(DEV), bt.to(DEV), kc, vc, status)
    with pytest.raises(Exception, match="position"):
        K.check_status(status)
    badbt = bt.clone(); badbt[0, starts[0] // page] = num_pages
    K.qk_norm_rope_kv_write(qd, Hq, Hkv, Dh, None, None, 1e-6, None, None, 0, pos.to(DEV), seq.to(DEV),
                            badbt.to(DEV), kc, vc, status)
    with pytest.raises(Exception, match="page"):
        K.check_status(status)


# ------------------------------------------------------------------- attention
def attention_case(lengths, q_counts, Hq, Hkv, Dh, page, dtype, seed=0, spike=None):
    """Dense K/V per sequence scattered into shuffled pages; queries are the last q_counts[s] tokens."""
    bt, num_pages = paged_layout(lengths, page, seed=seed)
    kc = torch.zeros(num_pages, Hkv, page, Dh, dtype=dtype)
    vc = torch.zeros_like(kc)
    dense, toks, qs = [], [], []
    for s, n in enumerate(lengths):
        k = rnd(n, Hkv, Dh, dtype=dtype, seed=seed * 100 + 3 * s)
        v = rnd(n, Hkv, Dh, dtype=dtype, seed=seed * 100 + 3 * s + 1)
        q = rnd(n, Hq, Dh, dtype=dtype, seed=seed * 100 + 3 * s + 2)
        if spike is not None:
            # one far key that the last query must find: its score stands out by a wide margin
            j = spike(n)
            k[j] = (q[n - 1].view(Hkv, Hq // Hkv, Dh)[:, 0, :] * 4.0).to(dtype)
            v[j] = 5.0
        for p in range(n):
            kc[int(bt[s, p // page]), :, p % page, :] = k[p]
            vc[int(bt[s, p // page]), :, p % page, :] = v[p]
        dense.append((q, k, v))
        for p in range(n - q_counts[s], n):
            toks.append((s, p))
            qs.append(q[p])
    return bt, num_pages, kc, vc, dense, toks, torch.stack(qs)


def attention_reference(dense, toks, window):
    out = []
    cache = {}
    for s, p in toks:
        if s not in cache:
            q, k, v = dense[s]
            cache[s] = P.attention(q.double(), k.double(), v.double(), window)
        out.append(cache[s][p])
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,Dh,page,window", [(4, 2, 16, 4, 0), (6, 3, 32, 16, 24), (3, 1, 80, 5, 0), (8, 8, 64, 1, 7),
                                                   (2, 1, 256, 64, 0)])
def test_attention_generic(K, dtype, Hq, Hkv, Dh, page, window):
    lengths, q_counts = [37, 1, 150, 64], [37, 1, 9, 1]
    bt, num_pages, kc, vc, dense, toks, q = attention_case(lengths, q_counts, Hq, Hkv, Dh, page, dtype)
    T = len(toks)
    seq = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    out = torch.empty(T, Hq * Dh, dtype=dtype, device=DEV)
    status = K.new_status(DEV)
    K.paged_attention_generic(out, q.reshape(T, Hq * Dh).to(DEV), Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), bt.to(DEV),
                              seq, pos, 1 / math.sqrt(Dh), window, status)
    K.check_status(status)
    close(out.view(T, Hq, Dh), attention_reference(dense, toks, window), dtype)


ALL_HEAD_DIMS = list(range(16, 257, 16))


@pytest.mark.parametrize("Dh", ALL_HEAD_DIMS)
def test_attention_mma_every_head_size(K, Dh):
    """Decode and prefill tensor-core kernels at every head size the configuration allows."""
    from imp_b200.ops import attention as A
    Hq, Hkv, page = 6, 2, 16
    lengths = [70, 33, 1, 129]
    status = K.new_status(DEV)
    # decode: one query per sequence, with and without key splits
    bt, num_pages, kc, vc, dense, toks, q = attention_case(lengths, [1, 1, 1, 1], Hq, Hkv, Dh, page, torch.bfloat16, seed=Dh)
    T = len(toks)
    seq = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    want = attention_reference(dense, toks, 0)
    for splits in (1, 3, None):
        out = torch.full((T, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
        A.decode_attention(out, q.reshape(T, Hq * Dh).to(DEV), Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), bt.to(DEV), seq, pos,
                           1 / math.sqrt(Dh), 0, status, n_splits=splits)
        K.check_status(status)
        close(out.view(T, Hq, Dh), want, torch.bfloat16)
    # prefill: portions of 20, 33, 1 and 40 tokens at the ends of the sequences
    counts = [20, 33, 1, 40]
    bt, num_pages, kc, vc, dense, toks, q = attention_case(lengths, counts, Hq, Hkv, Dh, page, torch.bfloat16, seed=Dh + 1)
    T = len(toks)
    seq = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    tiles0, tilesn, t = [], [], 0
    for n in counts:
        for a in range(0, n, 32):
            tiles0.append(t + a); tilesn.append(min(32, n - a))
        t += n
    out = torch.full((T, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
    A.prefill_attention(out, q.reshape(T, Hq * Dh).to(DEV), Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), bt.to(DEV), seq, pos,
                        torch.tensor(tiles0, dtype=torch.int32, device=DEV),
                        torch.tensor(tilesn, dtype=torch.int32, device=DEV), 1 / math.sqrt(Dh), 0, status)
    K.check_status(status)
    close(out.view(T, Hq, Dh), attention_reference(dense, toks, 0), torch.bfloat16)


@pytest.mark.parametrize("Hq,Hkv,page,window", [(4, 4, 16, 0), (5, 1, 4, 0), (12, 3, 1, 0), (40, 2, 16, 0), (8, 2, 8, 19),
                                                (3, 3, 64, 100), (4, 1, 3, 16), (4, 2, 32, 0), (6, 2, 32, 45), (4, 1, 48, 0),
                                                (8, 2, 128, 70), (2, 2, 64, 0), (4, 4, 96, 33)])
def test_attention_mma_groups_pages_windows(K, Hq, Hkv, page, window):
    from imp_b200.ops import attention as A
    Dh = 64
    lengths = [300, 17, 64, 100]
    status = K.new_status(DEV)
    for counts in ([1, 1, 1, 1], [50, 17, 2, 33]):
        bt, num_pages, kc, vc, dense, toks, q = attention_case(lengths, counts, Hq, Hkv, Dh, page, torch.bfloat16, seed=7)
        T = len(toks)
        seq = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
        pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
        want = attention_reference(dense, toks, window)
        btd = bt.clone()
        if window:
            # pages wholly behind every query's window are gone, as the cache manager leaves them
            for s, n in enumerate(lengths):
                first = max(0, (n - counts[s]) - window + 1)
                btd[s, :first // page] = -1
        out = torch.full((T, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
        qd = q.reshape(T, Hq * Dh).to(DEV)
        if counts == [1, 1, 1, 1]:
            for splits in (1, 4, None):
                A.decode_attention(out, qd, Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), btd.to(DEV), seq, pos,
                                   1 / math.sqrt(Dh), window, status, n_splits=splits)
                K.check_status(status)
                close(out.view(T, Hq, Dh), want, torch.bfloat16)
        tiles0, tilesn, t = [], [], 0
        for n in counts:
            for a in range(0, n, 16):
                tiles0.append(t + a); tilesn.append(min(16, n - a))
            t += n
        out.fill_(float("nan"))
        A.prefill_attention(out, qd, Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), btd.to(DEV), seq, pos,
                            torch.tensor(tiles0, dtype=torch.int32, device=DEV),
                            torch.tensor(tilesn, dtype=torch.int32, device=DEV), 1 / math.sqrt(Dh), window, status)
        K.check_status(status)
        close(out.view(T, Hq, Dh), want, torch.bfloat16)
        # the plain kernel agrees on the same pages
        out.fill_(float("nan"))
        K.paged_attention_generic(out, qd, Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), btd.to(DEV), seq, pos,
                                  1 / math.sqrt(Dh), window, status)
        K.check_status(status)
        close(out.view(T, Hq, Dh), want, torch.bfloat16)


@pytest.mark.parametrize("where", ["first", "page_edge", "far"])
def test_attention_finds_one_far_key_among_hundreds(K, where):
    """Random keys would hide a wrong page or a dropped key; here one key's score stands out, and its
    value (5.0 everywhere) must dominate the output."""
    from imp_b200.ops import attention as A
    Hq, Hkv, Dh, page = 4, 2, 64, 16
    spike = {"first": lambda n: 0, "page_edge": lambda n: 16 * (n // 32) - 1, "far": lambda n: n // 7}[where]
    lengths = [700, 333]
    bt, num_pages, kc, vc, dense, toks, q = attention_case(lengths, [1, 1], Hq, Hkv, Dh, page, torch.bfloat16, seed=3,
                                                           spike=spike)
    T = len(toks)
    seq = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    want = attention_reference(dense, toks, 0)
    assert (want.view(T, Hkv, Hq // Hkv, Dh)[:, :, 0, :] > 4.5).all()        # the spike dominates head 0 of each group
    status = K.new_status(DEV)
    qd = q.reshape(T, Hq * Dh).to(DEV)
    for splits in (1, 7, None):
        out = torch.full((T, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
        A.decode_attention(out, qd, Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), bt.to(DEV), seq, pos, 1 / math.sqrt(Dh), 0,
                           status, n_splits=splits)
        K.check_status(status)
        close(out.view(T, Hq, Dh), want, torch.bfloat16)
    for dtype in (torch.bfloat16, torch.float32):
        out = torch.full((T, Hq * Dh), float("nan"), dtype=dtype, device=DEV)
        K.paged_attention_generic(out, qd.to(dtype), Hq, Hkv, Dh, kc.to(DEV).to(dtype), vc.to(DEV).to(dtype),
                                  bt.to(DEV), seq, pos, 1 / math.sqrt(Dh), 0, status)
        K.check_status(status)
        close(out.view(T, Hq, Dh), want, dtype)


def run_prefill_tc(K, lengths, counts, Hq, Hkv, Dh, page, window, seed=11, spike=None, holes=True):
    """The tensor-memory prefill kernel on the last `counts` tokens of each sequence, in tiles of 128."""
    from imp_b200.ops import attention as A
    status = K.new_status(DEV)
    bt, num_pages, kc, vc, dense, toks, q = attention_case(lengths, counts, Hq, Hkv, Dh, page, torch.bfloat16, seed=seed,
                                                           spike=spike)
    T = len(toks)
    seq = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    btd = bt.clone()
    if window and holes:
        for s, n in enumerate(lengths):
            first = max(0, (n - counts[s]) - window + 1)
            btd[s, :first // page] = -1
    tiles0, tilesn, t = [], [], 0
    for n in counts:
        for a in range(0, n, 128):
            tiles0.append(t + a); tilesn.append(min(128, n - a))
        t += n
    qd = q.reshape(T, Hq * Dh).to(DEV)
    assert A.prefill_tc_supported(Dh, qd, qd, kc.to(DEV))
    out = torch.full((T, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
    A.prefill_attention_tc(out, qd, Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), btd.to(DEV), seq, pos,
                           torch.tensor(tiles0, dtype=torch.int32, device=DEV),
                           torch.tensor(tilesn, dtype=torch.int32, device=DEV), 1 / math.sqrt(Dh), window, status)
    K.check_status(status)
    want = attention_reference(dense, toks, window)
    close(out.view(T, Hq, Dh), want, torch.bfloat16)
    return out, want


@pytest.mark.parametrize("Dh,Hq,Hkv,page,window", [
    (128, 8, 2, 16, 0),      # the common shape: groups of 4, two heads per CTA
    (128, 3, 3, 16, 0),      # no grouping: one head per CTA
    (128, 6, 2, 8, 0),       # odd group: one head per CTA
    (64, 4, 1, 32, 0), (64, 2, 2, 128, 0), (64, 4, 2, 64, 0),
    (128, 4, 2, 16, 100), (64, 4, 4, 8, 300), (128, 2, 1, 32, 128), (64, 6, 3, 16, 37),
])
def test_attention_tc_prefill_shapes_pages_windows(K, Dh, Hq, Hkv, page, window):
    # whole prompts, portions that start inside a page and a tile, single rows, a ragged last tile
    run_prefill_tc(K, [300, 517, 129, 700], [300, 200, 1, 131], Hq, Hkv, Dh, page, window)
    run_prefill_tc(K, [1000], [128], Hq, Hkv, Dh, page, window, seed=12)
    run_prefill_tc(K, [257, 64], [257, 64], Hq, Hkv, Dh, page, window, seed=13)


@pytest.mark.parametrize("Dh,Hq,Hkv,window", [(64, 8, 8, 0), (128, 16, 4, 0), (64, 16, 8, 200)])
def test_attention_tc_prefill_more_items_than_sms(K, Dh, Hq, Hkv, window):
    """22 query tiles x 8 (tile, head group) units = 176 work items: more than the device has SMs, so CTAs of the
    persistent kernel work through two items each (heavy first, forth and back), with barrier phases, ring slots and
    tensor memory carried from one item to the next."""
    from imp_b200.ops import library as L
    units = Hkv * max(1, (Hq // Hkv) // 2) if (Hq // Hkv) % 2 == 0 else Hq
    assert 22 * units > L.load().imp_device_sm_count()
    run_prefill_tc(K, [1500, 1200], [1500, 1200], Hq, Hkv, Dh, 16, window, seed=21)
    # the same with a far key that the last query of each sequence must find among a thousand
    out, want = run_prefill_tc(K, [1500, 1200], [1500, 1200], Hq, Hkv, Dh, 16, 0, seed=22, spike=lambda n: n // 9)
    G = Hq // Hkv
    for last in (1499, 2699):
        assert (want.view(-1, Hkv, G, Dh)[last, :, 0, :] > 4.5).all() and (out.view(-1, Hkv, G, Dh)[last, :, 0, :].float() > 4.5).all()


@pytest.mark.parametrize("where", ["first", "page_edge", "tile_edge", "far"])
def test_attention_tc_prefill_finds_one_far_key(K, where):
    """One key's score stands out in every sequence; its value (5.0 everywhere) must dominate head 0 of each group."""
    spike = {"first": lambda n: 0, "page_edge": lambda n: 16 * (n // 32) - 1, "tile_edge": lambda n: 128 * (n // 256),
             "far": lambda n: n // 7}[where]
    out, want = run_prefill_tc(K, [900, 400], [1, 130], 4, 2, 128, 16, 0, seed=3, spike=spike)
    assert (want[0].view(2, 2, 128)[:, 0, :] > 4.5).all()


def test_attention_tc_prefill_rescales_when_the_maximum_grows(K):
    """Scores that grow along the keys force the accumulator in tensor memory through its rescale path; scores
    that fall never rescale after the first tile.  Both must agree with the plain reference."""
    from imp_b200.ops import attention as A
    Hq, Hkv, Dh, page, n = 2, 1, 128, 16, 640
    for direction in (1.0, -1.0):
        status = K.new_status(DEV)
        bt, num_pages, kc, vc, dense, toks, q = attention_case([n], [n], Hq, Hkv, Dh, page, torch.bfloat16, seed=5)
        # key j gets a component along dimension 0 that grows (or falls) with j; queries look along dimension 0
        ramp = (direction * torch.arange(n, dtype=torch.float32) * 0.25).to(torch.bfloat16)
        qd_, kd_, vd_ = dense[0]
        kd_[:, :, 0] = ramp[:, None]
        qd_[:, :, 0] = 8.0
        q[:, :, 0] = 8.0
        for j in range(n):
            kc[int(bt[0, j // page]), :, j % page, 0] = ramp[j]
        T = n
        seq = torch.zeros(T, dtype=torch.int32, device=DEV)
        pos = torch.arange(T, dtype=torch.int32, device=DEV)
        tiles0 = list(range(0, n, 128))
        out = torch.full((T, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
        A.prefill_attention_tc(out, q.reshape(T, Hq * Dh).to(DEV), Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), bt.to(DEV), seq, pos,
                               torch.tensor(tiles0, dtype=torch.int32, device=DEV),
                               torch.full((len(tiles0),), 128, dtype=torch.int32, device=DEV), 1 / math.sqrt(Dh), 0, status)
        K.check_status(status)
        close(out.view(T, Hq, Dh), attention_reference(dense, toks, 0), torch.bfloat16)


def test_attention_tc_prefill_reports_a_bad_page(K):
    from imp_b200.ops import attention as A
    Hq, Hkv, Dh, page = 2, 1, 64, 16
    bt, num_pages, kc, vc, dense, toks, q = attention_case([200], [200], Hq, Hkv, Dh, page, torch.bfloat16)
    bt[0, 3] = num_pages + 5
    seq = torch.zeros(200, dtype=torch.int32, device=DEV)
    pos = torch.arange(200, dtype=torch.int32, device=DEV)
    status = K.new_status(DEV)
    out = torch.empty(200, Hq * Dh, dtype=torch.bfloat16, device=DEV)
    A.prefill_attention_tc(out, q.reshape(200, -1).to(DEV), Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), bt.to(DEV), seq, pos,
                           torch.tensor([0, 128], dtype=torch.int32, device=DEV),
                           torch.tensor([128, 72], dtype=torch.int32, device=DEV), 0.1, 0, status)
    with pytest.raises(Exception, match="page"):
        K.check_status(status)


def test_attention_reports_a_bad_page(K):
    from imp_b200.ops import attention as A
    Hq, Hkv, Dh, page = 2, 1, 32, 16
    bt, num_pages, kc, vc, dense, toks, q = attention_case([40], [1], Hq, Hkv, Dh, page, torch.bfloat16)
    bt[0, 1] = num_pages + 5
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    pos = torch.tensor([39], dtype=torch.int32, device=DEV)
    status = K.new_status(DEV)
    out = torch.empty(1, Hq * Dh, dtype=torch.bfloat16, device=DEV)
    A.decode_attention(out, q.reshape(1, -1).to(DEV), Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), bt.to(DEV), seq, pos, 0.1, 0,
                       status, n_splits=1)
    with pytest.raises(Exception, match="page"):
        K.check_status(status)
    K.paged_attention_generic(out, q.reshape(1, -1).to(DEV), Hq, Hkv, Dh, kc.to(DEV), vc.to(DEV), bt.to(DEV), seq, pos,
                              0.1, 0, status)
    with pytest.raises(Exception, match="page"):
        K.check_status(status)


# -------------------------------------------------------------------- sampling
def test_argmax_ties_and_large_vocab(K):
    V = 151936 + 7
    x = rnd(3, V, seed=20).to(DEV)
    x[0, 100] = x[0, 90000] = 50.0                        # tie: the lowest index wins
    x[1, V - 1] = 60.0
    x[2] = -1e30
    x[2, 12345] = -5.0
    assert K.argmax(x).tolist() == [100, V - 1, 12345]
    wide = torch.zeros(2, 300, device=DEV)                # rows of a wider buffer
    wide[0, 7] = 1.0
    wide[1, 250] = 1.0
    assert K.argmax(wide[:, :200]).tolist() == [7, 0]


def run_sample(K, logits, temperature, u, top_k=0, top_p=1.0, min_p=0.0):
    R = logits.shape[0]
    f = lambda v: torch.full((R,), float(v), dtype=torch.float32, device=DEV)  # noqa: E731
    return K.sample(logits.to(DEV), f(temperature), torch.full((R,), int(top_k), dtype=torch.int32, device=DEV),
                    f(top_p), f(min_p), torch.as_tensor(u, dtype=torch.float32, device=DEV)).tolist()


@pytest.mark.parametrize("filters", [{}, {"top_k": 5}, {"top_p": 0.7}, {"min_p": 0.1}, {"top_k": 40, "top_p": 0.9},
                                     {"top_k": 7, "top_p": 0.5, "min_p": 0.02}])
def test_sample_matches_the_plain_twin(K, filters):
    V, R = 1003, 64
    logits = rnd(1, V, seed=21, scale=2.0).repeat(R, 1)
    us = np.random.default_rng(1).random(R).astype(np.float32)
    got = run_sample(K, logits, 0.8, us, **filters)
    x = logits[0].numpy()
    keep, _ = S.kept_set(x, 0.8, **filters)
    for tok, u in zip(got, us):
        assert keep[tok], f"token {tok} is outside the kept set of {filters}"
        lo, hi, _ = S.draw_interval(x, 0.8, tok, **filters)
        assert lo - 1e-5 <= u <= hi + 1e-5, f"u={u} does not select token {tok} (interval [{lo}, {hi}))"
    if filters.get("top_k"):
        assert len(set(got)) <= filters["top_k"]


def test_sample_greedy_paths_and_distribution(K):
    V = 200
    logits = rnd(1, V, seed=22, scale=1.5)
    am = int(logits[0].argmax())
    assert run_sample(K, logits, 0.0, [0.7]) == [am]
    assert run_sample(K, logits, 1.0, [0.7], top_k=1) == [am]
    R = 20000
    us = np.random.default_rng(2).random(R).astype(np.float32)
    got = np.array(run_sample(K, logits.repeat(R, 1), 1.0, us))
    freq = np.bincount(got, minlength=V) / R
    p = torch.softmax(logits[0].double(), 0).numpy()
    assert np.abs(freq - p).max() < 0.012
    # rows are independent of one another: a row alone gives what it gives in a batch
    assert run_sample(K, logits, 1.0, [us[17]]) == [got[17]]


def test_penalties(K):
    V = 300
    logits = rnd(3, V, seed=23, scale=2.0)
    hist = [[5, 5, 7, 299], [], [1, 2, 3, 1, 1]]
    flat = torch.tensor([t for h in hist for t in h], dtype=torch.int32, device=DEV)
    start = torch.tensor([0, 4, 4, 9], dtype=torch.int32, device=DEV)
    rep = torch.tensor([1.3, 1.0, 1.0], device=DEV)
    freq = torch.tensor([0.2, 0.0, 0.5], device=DEV)
    pres = torch.tensor([0.1, 0.0, 0.0], device=DEV)
    x = logits.clone().to(DEV)
    K.apply_penalties(x, flat, start, 5, rep, freq, pres, torch.empty(3 * V, dtype=torch.int32, device=DEV))
    for r in range(3):
        want = S.penalize(logits[r].numpy(), hist[r], float(rep[r]), float(freq[r]), float(pres[r]))
        assert np.allclose(x[r].cpu().numpy(), want, atol=1e-5)


def test_dry_penalty_matches_the_plain_scan(K):
    from imp_b200.sampling.sampler import dry_penalties
    rng = np.random.default_rng(5)
    for trial in range(20):
        n = int(rng.integers(2, 80))
        toks = rng.integers(0, 4, n).tolist()            # tiny alphabet: long repeats are common
        last_n = int(rng.choice([0, 5, 17]))
        allowed = int(rng.integers(0, 4))
        want = S.dry(toks, 0.8, 1.75, allowed, last_n)
        got = dry_penalties(toks, 0.8, 1.75, allowed, last_n)
        assert got.keys() == want.keys() and all(abs(got[t] - want[t]) <= 1e-6 * want[t] for t in want), (toks, last_n, allowed)
    # "a b c d a b c" -> after c came d: a 3-token repeat would become 4 long
    assert S.dry([1, 2, 3, 4, 1, 2, 3], 1.0, 2.0, 2) == {4: 2.0}
    V = 50
    logits = rnd(3, V, seed=31)
    x = logits.clone().to(DEV)
    rows = torch.tensor([0, 2, 2], dtype=torch.int32, device=DEV)
    toks = torch.tensor([4, 49, 0], dtype=torch.int32, device=DEV)
    vals = torch.tensor([2.0, 0.5, 1.25], dtype=torch.float32, device=DEV)
    K.sparse_subtract(x, rows, toks, vals)
    want = logits.clone()
    want[0, 4] -= 2.0
    want[2, 49] -= 0.5
    want[2, 0] -= 1.25
    assert torch.equal(x.cpu(), want)


@pytest.mark.parametrize("typical_p,min_p", [(0.2, 0.0), (0.5, 0.0), (0.9, 0.0), (0.6, 0.05)])
def test_typical_filter_matches_the_plain_twin(K, typical_p, min_p):
    V = 1003
    logits = rnd(3, V, seed=33, scale=2.5)
    logits[2, ::7] = -float("inf")                       # tokens an earlier mask removed
    x = logits.clone().to(DEV)
    tp = torch.tensor([typical_p, 1.0, typical_p], dtype=torch.float32, device=DEV)
    mp = torch.full((3,), min_p, dtype=torch.float32, device=DEV)
    K.typical_filter(x, tp, mp)
    got = x.cpu()
    assert torch.equal(got[1], logits[1]), "a row with typical_p = 1 is left alone"
    for r in (0, 2):
        keep, dev, cut = S.typical_keep(logits[r].numpy(), typical_p, min_p)
        kept = torch.isfinite(got[r]).numpy()
        edge = np.abs(dev - cut) < 1e-3                  # float32 vs float64 at the cut
        assert ((kept == keep) | edge).all(), f"row {r}: kept set differs away from the cut"
        assert torch.equal(got[r][torch.from_numpy(kept)], logits[r][torch.from_numpy(kept)])
        assert 0 < kept.sum() < np.isfinite(logits[r].numpy()).sum()
    # the most probable token can be atypical: a peaked head over a flat tail
    peaked = torch.zeros(1, 400)
    peaked[0, 0] = 4.0
    y = peaked.clone().to(DEV)
    K.typical_filter(y, torch.tensor([0.3], device=DEV), torch.zeros(1, device=DEV))
    keep, _, _ = S.typical_keep(peaked[0].numpy(), 0.3)
    assert (torch.isfinite(y[0]).cpu().numpy() == keep).all()


def test_mirostat_draw_and_surprise(K):
    V, R = 777, 48
    logits = rnd(1, V, seed=34, scale=2.0).repeat(R, 1)
    rng = np.random.default_rng(6)
    us = rng.random(R).astype(np.float32)
    mus = rng.uniform(1.0, 12.0, R).astype(np.float32)
    mus[0] = -5.0                                        # nothing passes: falls back to every token
    active = torch.ones(R, dtype=torch.int32, device=DEV)
    active[5] = 0
    out = torch.full((R,), -7, dtype=torch.int32, device=DEV)
    sur = torch.full((R,), -1.0, dtype=torch.float32, device=DEV)
    K.sample_mirostat(logits.to(DEV), active, torch.full((R,), 0.9, device=DEV), torch.from_numpy(mus).to(DEV),
                      torch.from_numpy(us).to(DEV), out, sur)
    out, sur = out.tolist(), sur.tolist()
    assert out[5] == -7 and sur[5] == -1.0, "inactive rows are not written"
    x = logits[0].numpy()
    for r in range(R):
        if r == 5:
            continue
        tok, s, keep = S.mirostat_v2(x, 0.9, float(mus[r]), float(us[r]))
        assert keep[out[r]], f"row {r}: token {out[r]} has surprise above mu={mus[r]}"
        mass = np.where(keep, np.exp((x - x.max()) / 0.9), 0.0)
        cum = np.cumsum(mass) / mass.sum()
        lo, hi = cum[out[r]] - mass[out[r]] / mass.sum(), cum[out[r]]
        assert lo - 1e-5 <= us[r] <= hi + 1e-5
        e = np.exp((x - x.max()) / 0.9)
        s_want = -math.log2(e[out[r]] / e.sum())         # surprise under the unfiltered distribution
        assert abs(sur[r] - s_want) < 1e-3


def test_sampler_mirostat_state_typical_and_dry_through_the_class(K):
    from imp_b200.sampling.sampler import Sampler, SamplerState, SamplingParams, uniform_for
    V = 300
    sampler = Sampler(V, 4, DEV)
    base = rnd(1, V, seed=35, scale=2.0)
    # Mirostat: mu starts at 2 * tau and moves by -eta * (surprise - tau) after every draw
    p = SamplingParams(temperature=1.0, mirostat=2, mirostat_tau=3.0, mirostat_eta=0.2, seed=11)
    st = SamplerState()
    mu = 6.0
    for step in range(5):
        tok = sampler.sample(base.clone().to(DEV), [p], [11], [step], None, [st])[0]
        want_tok, s, _ = S.mirostat_v2(base[0].numpy(), 1.0, mu, uniform_for(11, step))
        assert tok == want_tok
        mu -= 0.2 * (s - 3.0)
        assert abs(st.mirostat_mu - mu) < 1e-3
    # typical-p before greedy: the argmax is taken among the typical tokens
    peaked = torch.zeros(1, V)
    peaked[0, 0] = 4.0
    peaked[0, 17] = 0.01
    g = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, typical_p=0.3)
    keep, _, _ = S.typical_keep(peaked[0].numpy(), 0.3)
    assert not keep[0]
    assert sampler.sample(peaked.clone().to(DEV), [g], [1], [0])[0] == 17
    # DRY: the token that would extend a repeat loses multiplier * base ** (match - allowed)
    hist = [9, 8, 7, 6, 9, 8, 7]
    d = SamplingParams(temperature=0.0, dry_multiplier=50.0, dry_base=1.75, dry_allowed_length=2)
    x = torch.zeros(1, V)
    x[0, 6] = 5.0
    x[0, 3] = 1.0
    assert sampler.sample(x.clone().to(DEV), [SamplingParams.greedy()], [1], [0], [hist])[0] == 6
    assert sampler.sample(x.clone().to(DEV), [d], [1], [0], [hist])[0] == 3
    # a mixed batch: each row as it would be alone
    rows = [p, g, d, SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=4)]
    logits = torch.cat([base, peaked, x, base]).to(DEV)
    st2 = [SamplerState() for _ in rows]
    got = sampler.sample(logits.clone(), rows, [11, 1, 1, 4], [0, 0, 0, 3], [[], [], hist, []], st2)
    alone = [sampler.sample(logits[i:i + 1].clone(), [rows[i]], [[11, 1, 1, 4][i]], [[0, 0, 0, 3][i]],
                            [[[], [], hist, []][i]], [SamplerState()])[0] for i in range(4)]
    assert got == alone


@pytest.mark.parametrize("Hq,Hkv,Dh,page,with_norm", [(32, 8, 128, 16, True), (3, 1, 64, 8, True), (5, 2, 128, 32, False),
                                                      (8, 4, 64, 16, True)])
def test_fused_qkv_projection_matches_projection_then_rotary_kernel(K, Hq, Hkv, Dh, page, with_norm):
    """The q,k,v product with norm, rotation and cache write in its epilogue against the plain computation
    (and, loosely, against the two-kernel path): q buffer, K pages and V pages; rows in two sequences that
    start inside pages; a width that leaves the last 256-column tile of the product partly empty."""
    T, Kd = 300, 192
    lengths, starts = [210, 177], [40, 47]                 # 170 + 130 new tokens
    bt, num_pages = paged_layout(lengths, page, seed=4)
    toks = [(s, p) for s, (st, n) in enumerate(zip(starts, lengths)) for p in range(st, n)]
    assert len(toks) == T
    seq = torch.tensor([s for s, _ in toks], dtype=torch.int32)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32)
    N = (Hq + 2 * Hkv) * Dh
    x = rnd(T, Kd, dtype=torch.bfloat16, seed=41)
    w = rnd(N, Kd, dtype=torch.bfloat16, seed=42, scale=0.1)
    qw = (1 + 0.2 * rnd(Dh, seed=43)) if with_norm else None
    kw = (1 + 0.2 * rnd(Dh, seed=44)) if with_norm else None
    max_pos = 256
    i = torch.arange(Dh // 2, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (1e4 ** (-2.0 * i / Dh))[None, :]
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    kc = torch.zeros(num_pages, Hkv, page, Dh, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.full((T, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = K.new_status(DEV)
    ran = K.linear_qkv_rope(q_out, x.to(DEV), w.to(DEV), Hq, Hkv, Dh, None if qw is None else qw.to(DEV),
                            None if kw is None else kw.to(DEV), 1e-6, cos, sin, pos.to(DEV), seq.to(DEV), bt.to(DEV), kc, vc,
                            status)
    assert ran, "the fused kernel should take this shape"
    K.check_status(status)
    # plain computation in double precision
    y = x.double() @ w.double().T
    q = y[:, :Hq * Dh].view(T, Hq, Dh)
    k = y[:, Hq * Dh:(Hq + Hkv) * Dh].view(T, Hkv, Dh)
    v = y[:, (Hq + Hkv) * Dh:].view(T, Hkv, Dh)
    if with_norm:
        q, k = P.rmsnorm(q, qw.double(), 1e-6), P.rmsnorm(k, kw.double(), 1e-6)
    q, k = P.rope(q, pos.tolist(), 1e4), P.rope(k, pos.tolist(), 1e4)
    close(q_out.view(T, Hq, Dh), q, torch.bfloat16)
    kc_c, vc_c = kc.cpu(), vc.cpu()
    touched = torch.zeros(num_pages, page, dtype=torch.bool)
    for n, (s, p) in enumerate(toks):
        pg, sl = int(bt[s, p // page]), p % page
        close(kc_c[pg, :, sl, :], k[n], torch.bfloat16)
        close(vc_c[pg, :, sl, :], v[n], torch.bfloat16)
        touched[pg, sl] = True
    assert (kc_c[~touched.unsqueeze(1).expand(-1, Hkv, -1)] == 0).all() and (vc_c[~touched.unsqueeze(1).expand(-1, Hkv, -1)] == 0).all()
    # fewer than 256 rows, or another head size: declined, nothing written
    q2 = torch.full((100, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert not K.linear_qkv_rope(q2, x[:100].to(DEV), w.to(DEV), Hq, Hkv, Dh, None, None, 1e-6, cos, sin, pos[:100].to(DEV),
                                 seq[:100].to(DEV), bt.to(DEV), kc, vc, status)
    assert torch.isnan(q2.float()).all()
    # a page outside the pool is reported, its rows are not written
    badbt = bt.clone()
    badbt[1, starts[1] // page] = num_pages + 3
    K.linear_qkv_rope(q_out, x.to(DEV), w.to(DEV), Hq, Hkv, Dh, None, None, 1e-6, cos, sin, pos.to(DEV), seq.to(DEV),
                      badbt.to(DEV), kc, vc, status)
    with pytest.raises(Exception, match="page"):
        K.check_status(status)


@pytest.mark.parametrize("scale,filters", [(4.0, {"top_k": 40, "top_p": 0.9}), (4.0, {"top_p": 0.95}), (0.3, {"top_p": 0.9}),
                                           (2.0, {"top_k": 2000}), (2.0, {"top_k": 1000, "min_p": 0.001}),
                                           (3.0, {"top_k": 5, "top_p": 0.3})])
def test_sample_large_vocabulary_short_list_and_general_passes(K, scale, filters):
    """At a real vocabulary the sampler finds the kept tokens by a radix selection into a short list of at
    most 1024 candidates; a nucleus or a top-k wider than that takes the general passes.  Both must pick
    what the plain twin picks."""
    V, R = 50021, 24
    logits = rnd(1, V, seed=51, scale=scale).repeat(R, 1)
    logits[:, 123] = logits[:, 77]                       # a tie inside the distribution
    us = np.random.default_rng(3).random(R).astype(np.float32)
    got = run_sample(K, logits, 0.8, us, **filters)
    x = logits[0].numpy()
    keep, _ = S.kept_set(x, 0.8, **filters)
    for tok, u in zip(got, us):
        assert keep[tok], f"token {tok} is outside the kept set of {filters}"
        lo, hi, _ = S.draw_interval(x, 0.8, tok, **filters)
        assert lo - 2e-5 <= u <= hi + 2e-5, f"u={u} does not select token {tok} (interval [{lo}, {hi}))"


# ------------------------------------------------------------------ products left unsummed
@pytest.mark.parametrize("M,N,K_", [(8, 4096, 4096), (1, 1024, 3072), (20, 200, 12288), (64, 1000, 4104)])
def test_split_sum_summed_equals_the_plain_product(K, M, N, K_):
    a, w = rnd(M, K_, dtype=torch.bfloat16, seed=60).to(DEV), rnd(N, K_, dtype=torch.bfloat16, seed=61).to(DEV)
    want = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    assert K.gemm_bf16_tc_swap(want, a, w)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    sp = K.gemm_bf16_tc_swap_partials(out, a, w)
    assert sp is not None and sp.n_splits >= 2 and sp.parts.shape == (sp.n_splits, M, N)
    assert torch.isnan(out.float()).all()                      # nothing summed yet
    assert K.summed(sp) is out and torch.equal(out, want)
    assert K.summed(out) is out


@pytest.mark.parametrize("adtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [9, 40])
@pytest.mark.parametrize("d,splits,use_rows", [(4096, 8, False), (200, 3, False), (1032, 2, True), (8200, 2, False),
                                               (5120, 7, False), (8192, 4, True)])
def test_add_rmsnorm_of_an_unsummed_branch(K, adtype, wdtype, d, splits, use_rows, T):
    """h += round(sum of parts); out = rmsnorm(h): the stream gets the same bits as by summing first, the output
    the same up to the order in which the squares are added (few rows: a row is shared by a cluster of CTAs).
    d = 8200 is wider than the register-resident kernels take, so the wrapper sums first by itself."""
    h0 = rnd(T, d, seed=62).to(DEV)
    parts = rnd(splits, T, d, seed=63).to(DEV)
    w = (1 + 0.1 * rnd(d, seed=64)).to(wdtype).to(DEV)
    acc = torch.zeros(T, d, device=DEV)
    for s in range(splits):
        acc += parts[s]
    branch = acc.to(adtype)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV) if use_rows else None
    n_out = 3 if use_rows else T
    h_a, h_b = h0.clone(), h0.clone()
    out_a = torch.empty(n_out, d, dtype=adtype, device=DEV)
    out_b = torch.empty_like(out_a)
    K.add_rmsnorm(h_a, branch, w, out_a, 1e-5, 0.0, rows=rows)
    sp = K.SplitSum(torch.full((T, d), float("nan"), dtype=adtype, device=DEV), parts, splits)
    K.add_rmsnorm(h_b, sp, w, out_b, 1e-5, 0.0, rows=rows)
    assert torch.equal(h_a, h_b)
    close(out_b, out_a.double().cpu(), adtype)
    if use_rows:
        assert torch.equal(h_b, h0)


def test_linear_defers_only_when_asked_and_only_split_products(K):
    a, w = rnd(8, 4096, dtype=torch.bfloat16, seed=68).to(DEV), rnd(4096, 4096, dtype=torch.bfloat16, seed=69).to(DEV)
    out = torch.empty(8, 4096, dtype=torch.bfloat16, device=DEV)
    before = K.fallback_calls()
    assert K.linear(out, a, w) is out
    assert K.fallback_calls() == before
    got = K.linear(torch.empty_like(out), a, w, may_defer=True)
    assert isinstance(got, K.SplitSum) and torch.equal(got.summed(), out)
    big = rnd(32000, 4096, dtype=torch.bfloat16, seed=70).to(DEV)       # enough weight-row tiles: no split, a tensor
    assert isinstance(K.linear(torch.empty(8, 32000, dtype=torch.bfloat16, device=DEV), a, big, may_defer=True), torch.Tensor)
    a1 = a[:1]                                                          # one row: the weight-streaming kernel
    assert isinstance(K.linear(torch.empty(1, 4096, dtype=torch.bfloat16, device=DEV), a1, w, may_defer=True), torch.Tensor)


# ------------------------------------------------------------------ decode attention from the raw q,k,v rows
@pytest.mark.parametrize("Hq,Hkv,Dh,page,window,with_norm", [(8, 2, 128, 16, 0, True), (4, 4, 64, 16, 0, True),
                                                             (12, 1, 64, 32, 0, False), (2, 1, 256, 16, 0, True),
                                                             (6, 3, 128, 64, 40, True), (3, 1, 192, 48, 0, True)])
def test_decode_attention_from_raw_qkv_equals_rotary_kernel_then_attention(K, Hq, Hkv, Dh, page, window, with_norm):
    """One kernel does what two do: q and the new key are normalised and rotated inside the decode attention, the
    new key and value land in their pages (the same bits as the rotary kernel writes; lengths put the new key at a
    page's first row, its last row, inside a 16-key step, and at position 0), outputs agree to bfloat16 rounding."""
    from imp_b200.ops import attention as A
    lengths = [page * 3 + 1, page * 2, 70, 1, 300]
    B = len(lengths)
    bt, num_pages = paged_layout(lengths, page, seed=9)
    N = (Hq + 2 * Hkv) * Dh
    kc0 = 0.5 * rnd(num_pages, Hkv, page, Dh, dtype=torch.bfloat16, seed=90)     # history (and stale rows) everywhere
    vc0 = 0.5 * rnd(num_pages, Hkv, page, Dh, dtype=torch.bfloat16, seed=91)
    qkv = rnd(B, N, dtype=torch.bfloat16, seed=92).to(DEV)
    qw = (1 + 0.2 * rnd(Dh, seed=93)).to(DEV) if with_norm else None
    kw = (1 + 0.2 * rnd(Dh, seed=94)).to(DEV) if with_norm else None
    max_pos = 512
    i = torch.arange(Dh // 2, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (1e4 ** (-2.0 * i / Dh))[None, :]
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    btd = bt.to(DEV)
    status = K.new_status(DEV)
    for splits in (1, 3, None):
        # two kernels
        kc_a, vc_a, qkv_a = kc0.to(DEV).clone(), vc0.to(DEV).clone(), qkv.clone()
        K.qk_norm_rope_kv_write(qkv_a, Hq, Hkv, Dh, qw, kw, 1e-6, cos, sin, Dh, pos, seq, btd, kc_a, vc_a, status)
        out_a = torch.full((B, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
        A.decode_attention(out_a, qkv_a[:, :Hq * Dh], Hq, Hkv, Dh, kc_a, vc_a, btd, seq, pos, 1 / math.sqrt(Dh), window, status,
                           n_splits=splits)
        # one kernel
        kc_b, vc_b = kc0.to(DEV).clone(), vc0.to(DEV).clone()
        out_b = torch.full((B, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert A.decode_attention_fused(out_b, qkv, Hq, Hkv, Dh, kc_b, vc_b, btd, seq, pos, 1 / math.sqrt(Dh), window,
                                        qw, kw, 1e-6, cos, sin, status, n_splits=splits)
        K.check_status(status)
        assert torch.equal(vc_a, vc_b)
        assert (kc_a != kc_b).float().mean() < 1e-3                    # the sum of squares adds in another order
        close(kc_b, kc_a.double().cpu(), torch.bfloat16)
        close(out_b, out_a.double().cpu(), torch.bfloat16)
        # and both against the computation in double precision (keys enter it as the bfloat16 values of the cache)
        want = decode_reference(qkv, kc0, vc0, bt, lengths, Hq, Hkv, Dh, page, window, qw, kw)
        close(out_b.view(B, Hq, Dh), want, torch.bfloat16)
        close(out_a.view(B, Hq, Dh), want, torch.bfloat16)
    # head sizes and page sizes the one-kernel path does not take are declined, nothing written
    kc_c = torch.zeros(4, 1, 8, 64, dtype=torch.bfloat16, device=DEV)
    assert not A.decode_attention_fused(torch.empty(1, 64, dtype=torch.bfloat16, device=DEV),
                                        torch.zeros(1, 192, dtype=torch.bfloat16, device=DEV), 1, 1, 64, kc_c, kc_c.clone(),
                                        torch.zeros(1, 4, dtype=torch.int32, device=DEV), seq[:1], pos[:1], 0.125, 0, None, None,
                                        1e-6, cos[:, :32].contiguous(), sin[:, :32].contiguous(), status)
