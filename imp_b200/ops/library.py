"""Loads the compiled CUDA library and declares its C entry points.

There is no fallback: if the library cannot be built or loaded, or the device
is not a Blackwell data-centre GPU (compute capability 10.x), the first use of
any op raises.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

_lib = None
_lock = threading.Lock()


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error."""


_SIGNATURES = {
    "imp_last_error": (c_char_p, []),
    "imp_status_string": (c_char_p, [c_int]),
    "imp_abi_version": (c_int, []),
    "imp_device_arch": (c_int, []),
    "imp_device_sm_count": (c_int, []),
    "imp_embedding": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    "imp_swiglu": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "imp_cast": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_void_p]),
    "imp_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float,
                                c_int, c_int, c_int, c_void_p]),
    "imp_rmsnorm_rows": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_float,
                                 c_int, c_int, c_void_p]),
    "imp_qk_norm_rope_kv_write": (c_int, [
        c_void_p, c_int64, c_int, c_int, c_int, c_int,          # qkv, row_stride, n_tokens, Hq, Hkv, Dh
        c_void_p, c_void_p, c_float, c_float, c_int,            # q_norm_w, k_norm_w, eps, weight_offset, w_dtype
        c_void_p, c_void_p, c_int, c_int,                       # cos, sin, rot_dim, max_pos
        c_void_p, c_void_p, c_void_p, c_int, c_int,             # positions, seq_of_token, block_table, bt_stride, n_seqs
        c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),  # k_cache, v_cache, P, pages, dtype, status, stream
    "imp_paged_attention_generic": (c_int, [
        c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,   # out, out_stride, q, q_stride, k_cache, v_cache
        c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,          # block_table, bt_stride, seq_of_token, positions, T, B
        c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,   # Hq, Hkv, Dh, P, pages, scale, window, dtype
        c_void_p, c_void_p]),                                       # status, stream
    "imp_gemm_f32": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "imp_gemm_bf16_small_m": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int,
                                      c_int, c_void_p]),
    "imp_gemm_bf16_stream": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int,
                                     c_int, c_void_p]),
    "imp_gemm_bf16_stream_swiglu": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int,
                                            c_int, c_void_p]),
    "imp_gemm_bf16_tc": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int,
                                 c_void_p, c_void_p]),
    "imp_gemm_bf16_tc_qkv_rope": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                          c_void_p, c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
                                          c_void_p, c_void_p]),
    "imp_gemm_bf16_tc_swap": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int,
                                      c_void_p, c_void_p, c_void_p]),
    "imp_gemm_bf16_tc_swap_scratch_floats": (c_int64, [c_int, c_int, c_int, c_int]),
    "imp_gemm_bf16_tc_swap_splits": (c_int, [c_int, c_int, c_int]),
    "imp_gemm_bf16_tc_splits": (c_int, [c_int, c_int, c_int]),
    "imp_gemm_tc_test_hooks": (c_int, [ctypes.c_uint, c_int]),
    "imp_gemm_bf16_tc_swap_partials": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int,
                                               c_void_p, c_void_p]),
    "imp_gemm_bf16_tc_swap_sum": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int, c_int, c_int, c_void_p]),
    "imp_add_rmsnorm_split": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                      c_float, c_float, c_int, c_int, c_int, c_void_p]),
    "imp_argmax": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "imp_argmax_scratch_words": (c_int, [c_int]),
    "imp_apply_penalties": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_void_p]),
    "imp_sample": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_void_p, c_void_p]),
    "imp_sparse_subtract": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "imp_typical_filter": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "imp_sample_mirostat": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_void_p]),
}

_SIGNATURES.update({
    "imp_op_error_message": (c_char_p, []),
    "imp_op_fallback_calls": (c_int64, []),
    "imp_op_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "imp_op_linear_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "imp_op_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p,
                                   c_int, c_void_p]),
    "imp_op_decode_splits": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int]),
})

# Entry points that newer sources add; declared when present so an older build still loads in tools
# that only list symbols.  Every name in _SIGNATURES is required.
_OPTIONAL_SIGNATURES = {}


def declare(name: str, restype, argtypes, optional: bool = False) -> None:
    """Declare one more entry point (used by op modules that own their kernels' signatures)."""
    (_OPTIONAL_SIGNATURES if optional else _SIGNATURES)[name] = (restype, argtypes)
    if _lib is not None:
        _bind(_lib, name, restype, argtypes, optional)


def _bind(lib, name, restype, argtypes, optional):
    try:
        fn = getattr(lib, name)
    except AttributeError:
        if optional:
            return
        raise KernelError(f"the compiled library lacks the entry point {name}; rebuild it "
                          "(python -m imp_b200.csrc.build --force)") from None
    fn.restype = restype
    fn.argtypes = argtypes


def load():
    """The ctypes handle of the library, built on first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from ..csrc.build import build
        path = build()
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the CUDA library {path}: {e}") from None
        for name, (restype, argtypes) in _SIGNATURES.items():
            _bind(lib, name, restype, argtypes, False)
        for name, (restype, argtypes) in _OPTIONAL_SIGNATURES.items():
            _bind(lib, name, restype, argtypes, True)
        _lib = lib
        return lib


_arch_checked = False


def require_device() -> None:
    """Raise unless a CUDA device of compute capability 10.x is current."""
    global _arch_checked
    if _arch_checked:
        return
    import torch
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this engine runs only on a B200-class GPU (no CPU path exists)")
    lib = load()
    arch = lib.imp_device_arch()
    if arch < 0:
        raise KernelError(f"cannot query the device: {lib.imp_last_error().decode()}")
    if arch // 10 != 10:
        raise KernelError(f"the kernels are built for sm_100a only; this device is sm_{arch}")
    _arch_checked = True


launch_calls = 0   # launcher calls made through `check` (each enqueues at least one kernel of this library)


def check(rc: int, what: str) -> None:
    global launch_calls
    launch_calls += 1
    if rc != 0:
        msg = load().imp_last_error().decode(errors="replace")
        raise KernelError(f"{what} failed ({rc}): {msg}")


def loaded_library_path():
    return getattr(_lib, "_name", None)
