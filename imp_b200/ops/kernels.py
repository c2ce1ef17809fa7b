"""Raw kernel launchers on torch tensors, for kernel tests, tools and measurement.

Each function checks shapes and dtypes, then launches on torch's current
stream.  Nothing here computes with torch: tensors are only memory.  The
engine itself does not come here: its host is C++ (csrc/host).  `linear`,
`linear_swiglu` and `add_rmsnorm` call the library's own choice of kernel
(csrc/host/linear.cpp), so that what a test or a measurement sees is what the
engine runs.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import library as L

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

SMALL_M_MAX = 16        # most rows the weight-streaming kernel takes


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise L.KernelError(f"unsupported element type {t.dtype} (bfloat16 or float32)") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise L.KernelError("kernel arguments must be CUDA tensors (no CPU path exists)")


def new_status(device) -> torch.Tensor:
    """The device status word kernels report bad indices to (0 = ok)."""
    return torch.zeros(1, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor, what: str = "step") -> None:
    """Read the status word (synchronises) and raise if a kernel reported a bad index."""
    code = int(status.item())
    if code != 0:
        status.zero_()
        raise L.KernelError(f"{what}: device reported '{L.load().imp_status_string(code).decode()}' (code {code})")


def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0,
              status: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(out, table, ids)
    T, d = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous()
    assert table.dim() == 2 and table.shape[1] == d and table.is_contiguous()
    assert ids.dtype == torch.int32 and ids.numel() == T and ids.is_contiguous()
    lib = L.load()
    L.check(lib.imp_embedding(out.data_ptr(), table.data_ptr(), ids.data_ptr(), T, d, table.shape[0], _dt(table),
                              float(scale), _ptr(status), _stream()), "embedding")
    return out


def swiglu(out: torch.Tensor, gate_up: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """out[t, f] = silu(gate) * up.  interleave == 0: gate_up holds gate columns then up columns;
    interleave == b: runs of b gate columns and b up columns alternate."""
    _need_cuda(out, gate_up)
    T, F = out.shape
    assert gate_up.shape == (T, 2 * F) and gate_up.dtype == out.dtype
    assert out.is_contiguous() and gate_up.is_contiguous()
    L.check(L.load().imp_swiglu(out.data_ptr(), gate_up.data_ptr(), T, F, int(interleave), _dt(out), _stream()),
            "swiglu")
    return out


SWIGLU_INTERLEAVE = 8   # rows of gate, then rows of up, alternating, for the fused matrix product


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stack gate[F, d] and up[F, d] as runs of 8 gate rows and their 8 up rows (F a multiple of 8)."""
    F, d = gate.shape
    b = SWIGLU_INTERLEAVE
    assert up.shape == gate.shape and F % b == 0
    return torch.stack([gate.view(F // b, b, d), up.view(F // b, b, d)], dim=1).reshape(2 * F, d).contiguous()


def _view(t: Optional[torch.Tensor]):
    from ..parts.base import to_imp
    return to_imp(t)


def _op_check(rc: int, what: str) -> None:
    L.launch_calls += 1
    if rc != 0:
        raise L.KernelError(f"{what} failed ({rc}): {L.load().imp_op_error_message().decode(errors='replace')}")


def linear_swiglu(out: torch.Tensor, x: torch.Tensor, w_interleaved: torch.Tensor) -> torch.Tensor:
    """out[M, F] = silu(x Wg^T) * (x Wu^T) with Wg and Wu interleaved by `interleave_gate_up`: the library's
    choice of kernel (csrc/host/linear.cpp `linear_swiglu`)."""
    _need_cuda(out, x, w_interleaved)
    if x.shape[0] == 0:
        return out
    o, a, w = _view(out), _view(x), _view(w_interleaved)
    _op_check(L.load().imp_op_linear_swiglu(ctypes.byref(o), ctypes.byref(a), ctypes.byref(w), _stream(), None), "linear_swiglu")
    return out


def cast(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    _need_cuda(dst, src)
    assert dst.numel() == src.numel() and dst.is_contiguous() and src.is_contiguous()
    L.check(L.load().imp_cast(dst.data_ptr(), _dt(dst), src.data_ptr(), _dt(src), src.numel(), _stream()), "cast")
    return dst


class SplitSum:
    """A matrix product whose contraction was cut over CTAs and whose parts have not been added yet.

    `parts` [n_splits, M, N] float32 (in the library's scratch: valid until the call after next) holds what
    each split contributes; the value is their sum in split order, rounded to `out`'s type, and `out` [M, N]
    is where it belongs.  `linear(..., may_defer=True)` returns one instead of a tensor when that saves the
    summing kernel; `add_rmsnorm` takes one and adds the parts while it reads them.  Anyone else calls
    `summed()` first."""

    __slots__ = ("out", "parts_ptr", "n_splits", "parts")

    def __init__(self, out: torch.Tensor, parts, n_splits: int):
        # parts: an address in the library's scratch, or a tensor [n_splits, M, N] float32 of the caller's
        self.parts = parts if hasattr(parts, "data_ptr") else None
        self.out, self.n_splits = out, n_splits
        self.parts_ptr = parts.data_ptr() if hasattr(parts, "data_ptr") else int(parts)

    @property
    def shape(self):
        return self.out.shape

    def summed(self) -> torch.Tensor:
        """Add the parts into `out` (the separate summing kernel) and return it."""
        M, N = self.out.shape
        epi = TC_OUT_F32 if self.out.dtype == torch.float32 else TC_OUT_BF16
        L.check(L.load().imp_gemm_bf16_tc_swap_sum(self.out.data_ptr(), self.out.stride(0), epi, self.parts_ptr,
                                                   M, N, self.n_splits, _stream()), "gemm_bf16_tc_swap_sum")
        return self.out


def summed(x):
    """x itself, or the tensor a SplitSum stands for."""
    return x.summed() if isinstance(x, SplitSum) else x


def add_rmsnorm(h: torch.Tensor, branch, weight: torch.Tensor, out: torch.Tensor,
                eps: float, weight_offset: float = 0.0, rows: Optional[torch.Tensor] = None,
                write_h: bool = True) -> torch.Tensor:
    """h (+= branch); out = rmsnorm(h) * (weight + offset).  With `rows`, output row r reads stream row rows[r]
    and h is left untouched.  `branch` may be a SplitSum: its parts are added on the way.  The library's own
    choice of kernel (csrc/host/linear.cpp `add_rmsnorm`)."""
    sp = branch if isinstance(branch, SplitSum) else None
    bt = sp.out if sp is not None else branch
    _need_cuda(h, bt, weight, out, rows)
    hv, bv, wv, ov = _view(h), _view(bt), _view(weight), _view(out)
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    _op_check(L.load().imp_op_add_rmsnorm(ctypes.byref(hv), ctypes.byref(bv) if bt is not None else None,
                                          sp.parts_ptr if sp is not None else None, sp.n_splits if sp is not None else 0,
                                          ctypes.byref(wv), ctypes.byref(ov), float(eps), float(weight_offset),
                                          _ptr(rows), rows.numel() if rows is not None else 0, _stream()), "add_rmsnorm")
    return out


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
                 weight_offset: float = 0.0) -> torch.Tensor:
    """Row-wise RMSNorm of a 2-D tensor whose rows may be strided."""
    _need_cuda(x, weight, out)
    n, d = x.shape
    assert out.shape == x.shape and out.dtype == x.dtype and x.stride(1) == 1 and out.stride(1) == 1
    assert weight.numel() == d and weight.is_contiguous()
    L.check(L.load().imp_rmsnorm_rows(x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0),
                                      n, d, float(eps), float(weight_offset), _dt(x), _dt(weight), _stream()),
            "rmsnorm_rows")
    return out


def qk_norm_rope_kv_write(qkv: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int,
                          q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                          cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot_dim: int,
                          positions: torch.Tensor, seq_of_token: Optional[torch.Tensor],
                          block_table: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], status: Optional[torch.Tensor] = None,
                          weight_offset: float = 0.0) -> None:
    _need_cuda(qkv, q_norm_w, k_norm_w, cos, sin, positions, seq_of_token, block_table, k_cache, v_cache)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.shape[1] >= (n_q_heads + 2 * n_kv_heads) * head_dim
    assert positions.dtype == torch.int32 and positions.numel() == T
    w_dtype = _dt(q_norm_w) if q_norm_w is not None else F32
    if q_norm_w is not None:
        assert q_norm_w.numel() == head_dim and k_norm_w.numel() == head_dim and k_norm_w.dtype == q_norm_w.dtype
    max_pos = 0
    if cos is not None:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape == sin.shape
        assert cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] * 2 == rot_dim
        max_pos = cos.shape[0]
    bt_stride = n_seqs = page_size = num_pages = 0
    if k_cache is not None:
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
        num_pages, hk, page_size, dh = k_cache.shape
        assert hk == n_kv_heads and dh == head_dim
        assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1
        assert seq_of_token.dtype == torch.int32 and seq_of_token.numel() == T
        n_seqs, bt_stride = block_table.shape[0], block_table.stride(0)
    L.check(L.load().imp_qk_norm_rope_kv_write(
        qkv.data_ptr(), qkv.stride(0), T, n_q_heads, n_kv_heads, head_dim,
        _ptr(q_norm_w), _ptr(k_norm_w), float(eps), float(weight_offset), w_dtype,
        _ptr(cos), _ptr(sin), int(rot_dim), max_pos,
        positions.data_ptr(), _ptr(seq_of_token), _ptr(block_table), bt_stride, n_seqs,
        _ptr(k_cache), _ptr(v_cache), page_size, num_pages, _dt(qkv), _ptr(status), _stream()),
        "qk_norm_rope_kv_write")


def linear_qkv_rope(q_out: torch.Tensor, x: torch.Tensor, w_qkv: torch.Tensor, n_q_heads: int, n_kv_heads: int,
                    head_dim: int, q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                    cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                    block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    status: Optional[torch.Tensor] = None) -> bool:
    """q, k, v = x w_qkv^T with the per-head norm, the rotation over the whole head and the cache write in
    the product's epilogue: q goes to q_out [T, Hq*Dh], k and v to the pages.  Norm weights in float32.
    Returns False, having done nothing, when the shape or the backend rules the fused kernel out
    (fewer than 256 rows, a head size other than 64 / 128, alignment, IMP_B200_GEMM=cublas): the caller
    then uses `linear` and `qk_norm_rope_kv_write`."""
    if x.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16:
        return False
    T, Kd = x.shape
    if T < 256 or head_dim not in (64, 128) or cos.shape[1] * 2 != head_dim:
        return False
    _need_cuda(q_out, x, w_qkv, q_norm_w, k_norm_w, cos, sin, positions, seq_of_token, block_table, k_cache, v_cache)
    assert w_qkv.shape == ((n_q_heads + 2 * n_kv_heads) * head_dim, Kd) and x.stride(1) == 1 and w_qkv.stride(1) == 1
    assert q_out.dtype == torch.bfloat16 and q_out.shape == (T, n_q_heads * head_dim) and q_out.stride(1) == 1
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    if q_norm_w is not None:
        assert q_norm_w.dtype == torch.float32 and k_norm_w.dtype == torch.float32
        assert q_norm_w.numel() == head_dim and k_norm_w.numel() == head_dim
    assert k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()
    num_pages, hk, page_size, dh = k_cache.shape
    assert hk == n_kv_heads and dh == head_dim and k_cache.shape == v_cache.shape
    assert positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32 and block_table.dtype == torch.int32
    rc = L.load().imp_gemm_bf16_tc_qkv_rope(
        x.data_ptr(), x.stride(0), w_qkv.data_ptr(), w_qkv.stride(0), T, Kd, n_q_heads, n_kv_heads, head_dim,
        _ptr(q_norm_w), _ptr(k_norm_w), float(eps), cos.data_ptr(), sin.data_ptr(), cos.shape[0],
        positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0),
        block_table.shape[0], q_out.data_ptr(), q_out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), page_size,
        num_pages, _ptr(status), _stream())
    if rc == -2:
        return False
    L.check(rc, "gemm_bf16_tc_qkv_rope")
    return True


def paged_attention_generic(out: torch.Tensor, q: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int,
                            k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                            seq_of_token: torch.Tensor, positions: torch.Tensor, scale: float, window: int = 0,
                            status: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(out, q, k_cache, v_cache, block_table, seq_of_token, positions)
    T = q.shape[0]
    assert out.shape[0] == T and out.stride(1) == 1 and q.stride(1) == 1 and out.dtype == q.dtype
    assert k_cache.dtype == q.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    num_pages, hk, page_size, dh = k_cache.shape
    assert hk == n_kv_heads and dh == head_dim and v_cache.shape == k_cache.shape
    assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
    assert seq_of_token.dtype == torch.int32 and positions.dtype == torch.int32
    L.check(L.load().imp_paged_attention_generic(
        out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), seq_of_token.data_ptr(), positions.data_ptr(), T,
        block_table.shape[0], n_q_heads, n_kv_heads, head_dim, page_size, num_pages, float(scale), int(window),
        _dt(q), _ptr(status), _stream()), "paged_attention_generic")
    return out


def gemm_f32(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[M,N] = a[M,K] @ w[N,K]^T, true 32-bit."""
    _need_cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.dtype == w.dtype == out.dtype == torch.float32
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    L.check(L.load().imp_gemm_f32(out.data_ptr(), out.stride(0), a.data_ptr(), a.stride(0), w.data_ptr(),
                                  w.stride(0), M, N, K, _stream()), "gemm_f32")
    return out


def gemm_bf16_small_m(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    _need_cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.dtype == w.dtype == torch.bfloat16
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    L.check(L.load().imp_gemm_bf16_small_m(out.data_ptr(), out.stride(0), _dt(out), a.data_ptr(), a.stride(0),
                                           w.data_ptr(), w.stride(0), M, N, K, _stream()), "gemm_bf16_small_m")
    return out


def gemm_bf16_stream(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[M,N] = a[M,K] @ w[N,K]^T for M <= 16 on the tensor cores, streaming w once.  Falls back to
    the scalar-load kernel when K or the row strides do not allow 16-byte loads."""
    _need_cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and M <= SMALL_M_MAX
    assert a.dtype == w.dtype == torch.bfloat16
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    rc = L.load().imp_gemm_bf16_stream(out.data_ptr(), out.stride(0), _dt(out), a.data_ptr(), a.stride(0),
                                       w.data_ptr(), w.stride(0), M, N, K, _stream())
    if rc == -2:
        return gemm_bf16_small_m(out, a, w)
    L.check(rc, "gemm_bf16_stream")
    return out


TC_OUT_BF16, TC_OUT_F32, TC_OUT_SWIGLU = 0, 1, 2


def gemm_bf16_tc(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int = None,
                 status: Optional[torch.Tensor] = None) -> bool:
    """out = a[M,K] @ w[N,K]^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory).
    epilogue: TC_OUT_BF16 / TC_OUT_F32 write [M,N]; TC_OUT_SWIGLU writes silu(gate)*up [M,N/2] for
    interleaved gate/up rows.  Returns False when the operands' alignment rules it out."""
    _need_cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    if epilogue is None:
        epilogue = TC_OUT_F32 if out.dtype == torch.float32 else TC_OUT_BF16
    assert w.shape[1] == K and a.dtype == w.dtype == torch.bfloat16
    assert out.shape == (M, N // 2 if epilogue == TC_OUT_SWIGLU else N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    rc = L.load().imp_gemm_bf16_tc(out.data_ptr(), out.stride(0), epilogue, a.data_ptr(), a.stride(0), w.data_ptr(),
                                   w.stride(0), M, N, K, _ptr(status), _stream())
    if rc == -2:
        return False
    L.check(rc, "gemm_bf16_tc")
    return True


TC_SWAP_MAX_M = 128   # rows up to which the weights take the M side of the tcgen05 product


def gemm_bf16_tc_swap(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int = None,
                      status: Optional[torch.Tensor] = None) -> bool:
    """out = a[M,K] @ w[N,K]^T for M <= 128 with the weight rows on the M side of the tcgen05 MMA and the
    K range split over CTAs when there are few weight-row tiles.  Returns False if alignment rules it out."""
    _need_cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    if epilogue is None:
        epilogue = TC_OUT_F32 if out.dtype == torch.float32 else TC_OUT_BF16
    assert w.shape[1] == K and a.dtype == w.dtype == torch.bfloat16 and M <= TC_SWAP_MAX_M
    assert out.shape == (M, N // 2 if epilogue == TC_OUT_SWIGLU else N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    lib = L.load()
    n_scratch = lib.imp_gemm_bf16_tc_swap_scratch_floats(M, N, K, epilogue)
    scratch = torch.empty(n_scratch, dtype=torch.float32, device=a.device) if n_scratch else None
    rc = lib.imp_gemm_bf16_tc_swap(out.data_ptr(), out.stride(0), epilogue, a.data_ptr(), a.stride(0), w.data_ptr(),
                                   w.stride(0), M, N, K, _ptr(scratch), _ptr(status), _stream())
    if rc == -2:
        return False
    L.check(rc, "gemm_bf16_tc_swap")
    return True


def gemm_bf16_tc_swap_partials(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor,
                               status: Optional[torch.Tensor] = None) -> Optional[SplitSum]:
    """a[M,K] @ w[N,K]^T left as the partial results of the K splits of the swap-AB tcgen05 kernel; None where
    that kernel would not split this shape (or cannot take it)."""
    _need_cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and a.dtype == w.dtype == torch.bfloat16 and M <= TC_SWAP_MAX_M and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1
    lib = L.load()
    n_splits = lib.imp_gemm_bf16_tc_swap_splits(M, N, K)
    if n_splits < 2:
        return None
    parts = torch.empty((n_splits, M, N), dtype=torch.float32, device=a.device)
    rc = lib.imp_gemm_bf16_tc_swap_partials(parts.data_ptr(), a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0),
                                            M, N, K, _ptr(status), _stream())
    if rc == -2:
        return None
    L.check(rc, "gemm_bf16_tc_swap_partials")
    return SplitSum(out, parts, n_splits)


def linear(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, may_defer: bool = False):
    """out[M,N] = x[M,K] @ w[N,K]^T with 32-bit accumulation: the library's choice of kernel
    (csrc/host/linear.cpp `linear`).

    may_defer: the caller hands the result to add_rmsnorm (or calls summed() on it), so a product the tcgen05
    kernel splits over K may come back as a SplitSum, its summing kernel saved.
    """
    _need_cuda(out, x, w)
    if x.shape[0] == 0:
        return out
    o, a, wv = _view(out), _view(x), _view(w)
    parts, n_splits = ctypes.c_void_p(), ctypes.c_int(0)
    _op_check(L.load().imp_op_linear(ctypes.byref(o), ctypes.byref(a), ctypes.byref(wv), 1 if may_defer else 0,
                                     ctypes.byref(parts), ctypes.byref(n_splits), _stream(), None), "linear")
    if n_splits.value > 0:
        return SplitSum(out, parts.value, n_splits.value)
    return out


def fallback_calls() -> int:
    """Matrix products (on this thread) that no fast kernel took and the plain kernel ran."""
    return int(L.load().imp_op_fallback_calls())


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(logits, out)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    if out is None:
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
    lib = L.load()
    scratch = torch.empty(lib.imp_argmax_scratch_words(R), dtype=torch.int32, device=logits.device) if V >= 8192 else None
    L.check(lib.imp_argmax(logits.data_ptr(), logits.stride(0), R, V, out.data_ptr(), _ptr(scratch), _stream()),
            "argmax")
    return out


def apply_penalties(logits: torch.Tensor, history: torch.Tensor, hist_start: torch.Tensor, max_hist: int,
                    rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor, counts: torch.Tensor) -> None:
    _need_cuda(logits, history, hist_start, rep, freq, pres, counts)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert history.dtype == torch.int32 and hist_start.dtype == torch.int32 and hist_start.numel() == R + 1
    assert counts.dtype == torch.int32 and counts.numel() >= R * V and counts.is_contiguous()
    for t in (rep, freq, pres):
        assert t.dtype == torch.float32 and t.numel() == R
    L.check(L.load().imp_apply_penalties(logits.data_ptr(), logits.stride(0), R, V, history.data_ptr(),
                                         hist_start.data_ptr(), int(max_hist), rep.data_ptr(), freq.data_ptr(),
                                         pres.data_ptr(), counts.data_ptr(), _stream()), "apply_penalties")


def sparse_subtract(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor, values: torch.Tensor) -> None:
    """logits[rows[i], tokens[i]] -= values[i]; every (row, token) pair listed once."""
    _need_cuda(logits, rows, tokens, values)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert rows.dtype == torch.int32 and tokens.dtype == torch.int32 and values.dtype == torch.float32
    n = rows.numel()
    assert tokens.numel() == n and values.numel() == n
    L.check(L.load().imp_sparse_subtract(logits.data_ptr(), logits.stride(0), R, V, rows.data_ptr(),
                                         tokens.data_ptr(), values.data_ptr(), n, _stream()), "sparse_subtract")


def typical_filter(logits: torch.Tensor, typical_p: torch.Tensor, min_p: torch.Tensor) -> None:
    """Locally typical filtering in place; rows whose typical_p is outside (0, 1) stay as they are."""
    _need_cuda(logits, typical_p, min_p)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    for t in (typical_p, min_p):
        assert t.dtype == torch.float32 and t.numel() == R
    L.check(L.load().imp_typical_filter(logits.data_ptr(), logits.stride(0), R, V, typical_p.data_ptr(),
                                        min_p.data_ptr(), _stream()), "typical_filter")


def sample_mirostat(logits: torch.Tensor, active: torch.Tensor, temperature: torch.Tensor, mu: torch.Tensor,
                    uniform: torch.Tensor, out: torch.Tensor, surprise: torch.Tensor) -> None:
    """Mirostat v2 draw for the rows with active != 0: token into `out`, its surprise (bits) into `surprise`."""
    _need_cuda(logits, active, temperature, mu, uniform, out, surprise)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert active.dtype == torch.int32 and out.dtype == torch.int32
    for t in (temperature, mu, uniform, surprise):
        assert t.dtype == torch.float32 and t.numel() == R
    assert active.numel() == R and out.numel() == R
    L.check(L.load().imp_sample_mirostat(logits.data_ptr(), logits.stride(0), R, V, active.data_ptr(),
                                         temperature.data_ptr(), mu.data_ptr(), uniform.data_ptr(), out.data_ptr(),
                                         surprise.data_ptr(), _stream()), "sample_mirostat")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(logits, temperature, top_k, top_p, min_p, uniform, out)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert top_k.dtype == torch.int32
    for t in (temperature, top_p, min_p, uniform):
        assert t.dtype == torch.float32 and t.numel() == R
    if out is None:
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
    L.check(L.load().imp_sample(logits.data_ptr(), logits.stride(0), R, V, temperature.data_ptr(), top_k.data_ptr(),
                                top_p.data_ptr(), min_p.data_ptr(), uniform.data_ptr(), out.data_ptr(), _stream()),
            "sample")
    return out
