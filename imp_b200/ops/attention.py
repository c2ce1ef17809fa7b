"""Raw launchers of the per-head-size attention kernels on torch tensors, for kernel tests and tools.

The libraries of csrc/variants/attention_mma.cu (split-key decode kernel, 32-token prefill kernel)
and csrc/variants/attention_tc.cu (tensor-memory prefill kernel, head sizes 64 and 128) are built
on first use for a head size.  Which of them a step of the engine runs is decided in
csrc/host/attention.cpp; `decode_splits` here asks the library for its choice of key splits.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p
import os
from typing import Dict, Optional

import torch

from . import kernels as K
from . import library as L

_variants: Dict[int, ctypes.CDLL] = {}

DECODE_MAX_SPLITS = 32


def variant(head_dim: int) -> ctypes.CDLL:
    lib = _variants.get(head_dim)
    if lib is None:
        from ..csrc.build import ATTENTION_HEAD_DIMS, build_variant
        if head_dim not in ATTENTION_HEAD_DIMS:
            raise L.KernelError(f"attention kernels exist for head sizes {ATTENTION_HEAD_DIMS[0]}..."
                                f"{ATTENTION_HEAD_DIMS[-1]} in steps of 16, not {head_dim}")
        path = build_variant("attention_mma.cu", {"IMP_ATTN_DH": head_dim})
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise L.KernelError(f"cannot load {path}: {e}") from None
        lib.imp_last_error.restype = ctypes.c_char_p
        lib.imp_attn_head_dim.restype = c_int
        assert lib.imp_attn_head_dim() == head_dim
        lib.imp_attn_decode_scratch_floats.restype = c_int64
        lib.imp_attn_decode_scratch_floats.argtypes = [c_int, c_int, c_int]
        lib.imp_attn_decode.restype = c_int
        lib.imp_attn_decode.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                        c_int, c_void_p, c_void_p, c_void_p]
        lib.imp_attn_decode_fused.restype = c_int
        lib.imp_attn_decode_fused.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                              c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
                                              c_void_p, c_void_p]
        lib.imp_attn_prefill.restype = c_int
        lib.imp_attn_prefill.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                         c_int, c_float, c_int, c_void_p, c_void_p]
        _variants[head_dim] = lib
    return lib


TC_HEAD_DIMS = (64, 128)
PREFILL_BACKEND = os.environ.get("IMP_B200_ATTN_PREFILL", "tcgen05")   # "tcgen05" | "mma"
_tc_variants: Dict[int, ctypes.CDLL] = {}


def tc_variant(head_dim: int) -> ctypes.CDLL:
    """The tensor-memory prefill kernel for this head size (64 or 128), built on first use."""
    lib = _tc_variants.get(head_dim)
    if lib is None:
        from ..csrc.build import build_variant
        if head_dim not in TC_HEAD_DIMS:
            raise L.KernelError(f"the tensor-memory prefill kernel exists for head sizes {TC_HEAD_DIMS}, not {head_dim}")
        path = build_variant("attention_tc.cu", {"IMP_ATTN_DH": head_dim})
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise L.KernelError(f"cannot load {path}: {e}") from None
        lib.imp_last_error.restype = ctypes.c_char_p
        lib.imp_attn_tc_head_dim.restype = c_int
        assert lib.imp_attn_tc_head_dim() == head_dim
        lib.imp_attn_prefill_tc_supported.restype = c_int
        lib.imp_attn_prefill_tc_supported.argtypes = [c_int64, c_int64, c_int]
        lib.imp_attn_prefill_tc.restype = c_int
        lib.imp_attn_prefill_tc.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                            c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                            c_int, c_int, c_float, c_int, c_void_p, c_void_p]
        _tc_variants[head_dim] = lib
    return lib


def prefill_tc_supported(head_dim: int, q, out, k_cache) -> bool:
    """Whether the tensor-memory prefill kernel takes this geometry (else the 32-token kernel runs)."""
    if PREFILL_BACKEND != "tcgen05" or head_dim not in TC_HEAD_DIMS or q.dtype != torch.bfloat16:
        return False
    if q.data_ptr() % 16 or out.data_ptr() % 16 or k_cache.data_ptr() % 16:
        return False
    return bool(tc_variant(head_dim).imp_attn_prefill_tc_supported(q.stride(0), out.stride(0), k_cache.shape[2]))


def prefill_attention_tc(out, q, n_q_heads, n_kv_heads, head_dim, k_cache, v_cache, block_table, seq_of_token,
                         positions, tile_tok0, tile_rows, scale, window, status):
    """Tiles of up to 128 consecutive query tokens of one sequence over the cached keys, on tcgen05 (bfloat16)."""
    lib = tc_variant(head_dim)
    num_pages, hk, page_size, dh = k_cache.shape
    assert hk == n_kv_heads and dh == head_dim and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert tile_tok0.dtype == torch.int32 and tile_rows.dtype == torch.int32 and tile_tok0.numel() == tile_rows.numel()
    _check(lib, lib.imp_attn_prefill_tc(
        out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), q.shape[0], k_cache.data_ptr(), v_cache.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), seq_of_token.data_ptr(), positions.data_ptr(),
        tile_tok0.data_ptr(), tile_rows.data_ptr(), tile_tok0.numel(), block_table.shape[0], n_q_heads, n_kv_heads,
        page_size, num_pages, float(scale), int(window), None if status is None else status.data_ptr(),
        torch.cuda.current_stream().cuda_stream), "attention prefill (tcgen05)")
    return out


def _check(lib, rc: int, what: str) -> None:
    L.launch_calls += 1
    if rc != 0:
        raise L.KernelError(f"{what} failed ({rc}): {lib.imp_last_error().decode(errors='replace')}")


def decode_splits(n_tokens: int, n_kv_heads: int, group: int, page_size: int = 16, sm_count: int = 0, context: int = 0) -> int:
    """Key splits of the decode kernel as the library chooses them (csrc/host/attention.cpp `decode_splits`): a function
    of the batch size and of the sequences' typical length (`context`, 0: 4,096; the engine keeps one captured graph
    per batch size and context class).  `sm_count` 0 asks the device."""
    return int(L.load().imp_op_decode_splits(n_tokens, n_kv_heads, group, page_size, sm_count, context))


def decode_attention(out, q, n_q_heads, n_kv_heads, head_dim, k_cache, v_cache, block_table, seq_of_token, positions,
                     scale, window, status, n_splits=None):
    """One query token per sequence over its cached keys (bfloat16)."""
    lib = variant(head_dim)
    T = q.shape[0]
    num_pages, hk, page_size, dh = k_cache.shape
    assert hk == n_kv_heads and dh == head_dim and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    if n_splits is None:
        n_splits = decode_splits(T, n_kv_heads, n_q_heads // n_kv_heads, page_size)
    scratch = None
    n_floats = lib.imp_attn_decode_scratch_floats(T, n_q_heads, n_splits)
    if n_floats:
        scratch = torch.empty(n_floats, dtype=torch.float32, device=q.device)
    _check(lib, lib.imp_attn_decode(
        out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), seq_of_token.data_ptr(), positions.data_ptr(), T,
        block_table.shape[0], n_q_heads, n_kv_heads, page_size, num_pages, float(scale), int(window), n_splits,
        None if scratch is None else scratch.data_ptr(), None if status is None else status.data_ptr(),
        torch.cuda.current_stream().cuda_stream), "attention decode")
    return out


DECODE_FUSED = os.environ.get("IMP_B200_ATTN_FUSED", "1") != "0"   # 0: the rotary kernel runs before every decode attention


def decode_attention_fused(out, qkv, n_q_heads, n_kv_heads, head_dim, k_cache, v_cache, block_table, seq_of_token,
                           positions, scale, window, q_norm_w, k_norm_w, eps, cos, sin, status, n_splits=None) -> bool:
    """The decode step from the raw rows of the q,k,v product (bfloat16, q heads | k heads | v heads): per-head norm
    (32-bit weights or None) and rotation of q and of the new key happen inside the attention kernel, which writes
    the new key and value into their pages.  Returns False, with nothing done, where that kernel does not apply
    (head sizes that are no multiple of 64, page sizes that are no multiple of 16, IMP_B200_ATTN_FUSED=0)."""
    if not DECODE_FUSED or head_dim % 64 or k_cache.shape[2] % 16:
        return False
    lib = variant(head_dim)
    T = qkv.shape[0]
    num_pages, hk, page_size, dh = k_cache.shape
    assert hk == n_kv_heads and dh == head_dim and qkv.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert qkv.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert qkv.shape[1] >= (n_q_heads + 2 * n_kv_heads) * head_dim
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape == sin.shape
    assert cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] * 2 == head_dim
    if q_norm_w is not None:
        assert q_norm_w.dtype == torch.float32 and k_norm_w.dtype == torch.float32
        assert q_norm_w.numel() == head_dim and k_norm_w.numel() == head_dim
    if n_splits is None:
        n_splits = decode_splits(T, n_kv_heads, n_q_heads // n_kv_heads, page_size)
    scratch = None
    n_floats = lib.imp_attn_decode_scratch_floats(T, n_q_heads, n_splits)
    if n_floats:
        scratch = torch.empty(n_floats, dtype=torch.float32, device=qkv.device)
    rc = lib.imp_attn_decode_fused(
        out.data_ptr(), out.stride(0), qkv.data_ptr(), qkv.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), seq_of_token.data_ptr(), positions.data_ptr(), T,
        block_table.shape[0], n_q_heads, n_kv_heads, page_size, num_pages, float(scale), int(window), n_splits,
        None if scratch is None else scratch.data_ptr(), None if q_norm_w is None else q_norm_w.data_ptr(),
        None if k_norm_w is None else k_norm_w.data_ptr(), float(eps), cos.data_ptr(), sin.data_ptr(), cos.shape[0],
        None if status is None else status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    if rc == -2:
        return False
    _check(lib, rc, "attention decode (fused)")
    return True


def prefill_attention(out, q, n_q_heads, n_kv_heads, head_dim, k_cache, v_cache, block_table, seq_of_token, positions,
                      tile_tok0, tile_rows, scale, window, status):
    """Tiles of up to 32 consecutive query tokens of one sequence over the cached keys (bfloat16)."""
    lib = variant(head_dim)
    num_pages, hk, page_size, dh = k_cache.shape
    assert hk == n_kv_heads and dh == head_dim and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert tile_tok0.dtype == torch.int32 and tile_rows.dtype == torch.int32 and tile_tok0.numel() == tile_rows.numel()
    _check(lib, lib.imp_attn_prefill(
        out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), seq_of_token.data_ptr(), positions.data_ptr(),
        tile_tok0.data_ptr(), tile_rows.data_ptr(), tile_tok0.numel(), block_table.shape[0], n_q_heads, n_kv_heads,
        page_size, num_pages, float(scale), int(window), None if status is None else status.data_ptr(),
        torch.cuda.current_stream().cuda_stream), "attention prefill")
    return out
