"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some callers cannot call cudaMalloc (a serving thread that must not touch the allocator after
start-up, a plug-in inside a process that owns all device memory).  For them the library exports
`imp_attn_decode_noalloc`, whose scratch for the split-key partial results is a fixed 4 MiB buffer
inside the library image.  This test calls it twice in a row on different inputs, both times with
more key splits than a thread-block cluster merges on chip, so that both calls go through the
built-in buffer and the second finds the first call's leftovers in it.  Each result is compared
with the regular entry point given freshly allocated scratch and with the same attention computed
in double precision; the driver's count of free device memory must not move across the call (a
cudaMalloc inside it would show there, whoever's allocator it went through); and a request beyond
the buffer is refused.  It is collected last so that a run that stops at the first failure has run
everything else.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
SCRATCH_FLOATS = 1 << 20


def _case(seed, lengths, Hq, Hkv, Dh, page):
    g = torch.Generator().manual_seed(seed)
    need = [(n + page - 1) // page for n in lengths]
    num_pages = sum(need) + 2
    perm = torch.randperm(num_pages, generator=g)
    bt = -torch.ones(len(lengths), max(need) + 1, dtype=torch.int32)
    k = 0
    for s, n in enumerate(need):
        bt[s, :n] = perm[k:k + n].to(torch.int32)
        k += n
    kc = torch.randn(num_pages, Hkv, page, Dh, generator=g).to(torch.bfloat16)
    vc = torch.randn(num_pages, Hkv, page, Dh, generator=g).to(torch.bfloat16)
    q = torch.randn(len(lengths), Hq * Dh, generator=g).to(torch.bfloat16)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32)
    seq = torch.arange(len(lengths), dtype=torch.int32)
    return [t.to(DEV) for t in (q, kc, vc, bt, seq, pos)], num_pages


def _reference(q, kc, vc, bt, lengths, Hq, Hkv, Dh, page):
    """softmax(q K^T / sqrt(Dh)) V per sequence and head, in double precision, keys through the block table."""
    q, kc, vc, bt = q.double().cpu().view(len(lengths), Hq, Dh), kc.double().cpu(), vc.double().cpu(), bt.cpu()
    out = torch.zeros(len(lengths), Hq, Dh, dtype=torch.float64)
    for s, n in enumerate(lengths):
        keys = torch.stack([kc[int(bt[s, p // page]), :, p % page] for p in range(n)])   # [n, Hkv, Dh]
        vals = torch.stack([vc[int(bt[s, p // page]), :, p % page] for p in range(n)])
        for h in range(Hq):
            g = h // (Hq // Hkv)
            out[s, h] = torch.softmax(keys[:, g] @ q[s, h] / math.sqrt(Dh), 0) @ vals[:, g]
    return out.view(len(lengths), Hq * Dh)


def test_decode_attention_without_allocation_matches_the_regular_entry_point():
    from imp_b200.ops import attention as A
    from imp_b200.ops import kernels as K
    from imp_b200.ops import library

    library.require_device()
    Hq, Hkv, Dh, page = 8, 2, 64, 16
    lib = A.variant(Dh)
    fn = lib.imp_attn_decode_noalloc          # the exported C symbol itself
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    status = K.new_status(DEV)
    scale = 1 / math.sqrt(Dh)
    stream = torch.cuda.current_stream().cuda_stream
    # 5 and 7 key splits: above the four a cluster merges in shared memory, so both calls use the buffer
    for call, (seed, lengths, splits) in enumerate([(1, [300, 41, 129], 5), (2, [77, 512, 16, 200], 7)]):
        (q, kc, vc, bt, seq, pos), num_pages = _case(seed, lengths, Hq, Hkv, Dh, page)
        T = len(lengths)
        want = torch.full((T, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
        A.decode_attention(want, q, Hq, Hkv, Dh, kc, vc, bt, seq, pos, scale, 0, status, n_splits=splits)
        got = torch.full((T, Hq * Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert lib.imp_attn_decode_scratch_floats(T, Hq, splits) > 0, "this split count must need scratch"
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()
        rc = fn(got.data_ptr(), got.stride(0), q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(),
                bt.stride(0), seq.data_ptr(), pos.data_ptr(), T, T, Hq, Hkv, page, num_pages, scale, 0, splits,
                status.data_ptr(), stream)
        assert rc == 0, lib.imp_last_error().decode()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert torch.cuda.memory_allocated() == before
        assert free_after == free_before, "the driver's free memory moved: something inside the call allocated"
        K.check_status(status)
        # same kernels, same split of the keys, same order of additions: the results are the same bits,
        # which is well within the tolerance the other attention tests use (1% of the scale)
        assert not torch.isnan(got.float()).any()
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 0.01 * want.float().abs().max().item(), f"call {call}: max error {err}"
        assert torch.equal(got, want), f"call {call}: differs from the regular entry point"
        ref = _reference(q, kc, vc, bt, lengths, Hq, Hkv, Dh, page)
        err = (got.double().cpu() - ref).abs().max().item()
        assert err <= 0.01 * ref.abs().max().item(), f"call {call}: differs from the plain attention by {err}"
    # a request beyond the built-in buffer is refused before anything runs
    T_big = SCRATCH_FLOATS // (Hq * 4 * (Dh + 2)) + 1
    rc = fn(None, 0, None, 0, None, None, None, 0, None, None, T_big, T_big, Hq, Hkv, page, 4, scale, 0, 4, None, stream)
    assert rc != 0
    msg = lib.imp_last_error().decode()
    assert "scratch" in msg and str(SCRATCH_FLOATS) in msg
