"""ctypes bindings of the C API (include/imp_b200/imp.h, imp_parts.h).

Everything the Python package does goes through these entry points; the host
of the engine (configuration, loader, cache manager, scheduler, step function,
sampler glue) is C++ inside the shared library that `csrc/build.py` makes.
Nothing here needs torch.
"""
from __future__ import annotations

import ctypes
import json
import threading
from ctypes import (CFUNCTYPE, POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint8,
                    c_void_p)

# ---------------------------------------------------------------------------------- errors
IMP_SUCCESS = 0
IMP_ERROR_INVALID_ARG = -1
IMP_ERROR_OUT_OF_MEMORY = -2
IMP_ERROR_CUDA = -3
IMP_ERROR_FILE_NOT_FOUND = -4
IMP_ERROR_INVALID_MODEL = -5
IMP_ERROR_UNSUPPORTED = -6
IMP_ERROR_INTERNAL = -7
IMP_ERROR_CANCELLED = -8


class ImpError(RuntimeError):
    """A call of the C API failed; `.code` is its ImpError."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


class KernelError(ImpError):
    """A launcher refused its arguments or CUDA reported an error."""


class ConfigError(ImpError, ValueError):
    """A config.json that is missing a key, or holds a value the engine cannot run."""


class WeightError(ImpError, ValueError):
    """A checkpoint does not match the plan.  `.missing`, `.unexpected`, `.wrong_shape`, `.wrong_type`."""

    def __init__(self, code: int, message: str):
        super().__init__(code, message)
        self.missing, self.unexpected, self.wrong_shape, self.wrong_type = [], [], [], []
        for line in message.splitlines():
            line = line.strip()
            for key, attr, sep in (("missing tensors", "missing", ", "), ("unexpected tensors", "unexpected", ", "),
                                   ("wrong shapes", "wrong_shape", "; "), ("wrong element types", "wrong_type", "; ")):
                if line.startswith(key):
                    setattr(self, attr, line.split(": ", 1)[1].split(sep))


class SafetensorsError(ImpError, ValueError):
    """A safetensors file that cannot be read."""


class OutOfPages(ImpError):
    """Not enough free pages (or state slots) for what was asked."""


class CacheError(ImpError):
    """Misuse of the cache manager (unknown request, double free, ...)."""


# --------------------------------------------------------------------------------- structs
class ImpConfig(Structure):
    _fields_ = [("device_id", c_int), ("kv_cache_max_blocks", c_size_t), ("kv_cache_tokens", c_size_t),
                ("kv_block_size", c_int), ("max_batch_size", c_int), ("max_seq_len", c_int), ("max_batch_tokens", c_int),
                ("prefill_chunk_size", c_int), ("compute_dtype", c_int), ("enable_cuda_graphs", c_int),
                ("gpu_memory_fraction", c_float), ("state_slots", c_int), ("lookahead", c_int)]


class ImpGenerateParams(Structure):
    _fields_ = [("temperature", c_float), ("top_p", c_float), ("top_k", c_int), ("max_tokens", c_int), ("seed", c_int64),
                ("min_p", c_float), ("typical_p", c_float), ("repetition_penalty", c_float), ("frequency_penalty", c_float),
                ("presence_penalty", c_float), ("repeat_last_n", c_int), ("dry_multiplier", c_float), ("dry_base", c_float),
                ("dry_allowed_length", c_int), ("dry_penalty_last_n", c_int), ("mirostat", c_int), ("mirostat_tau", c_float),
                ("mirostat_eta", c_float), ("ignore_eos", c_int)]


class ImpStepOutput(Structure):
    _fields_ = [("id", c_int64), ("token", c_int32), ("finished", c_int32), ("status", c_int32), ("finish_reason", c_int32)]


class ImpRequestInfo(Structure):
    _fields_ = [("status", c_int32), ("finish_reason", c_int32), ("n_prompt", c_int32), ("n_output", c_int32),
                ("n_computed", c_int32), ("n_preempted", c_int32)]


class ImpStepEntry(Structure):
    _fields_ = [("id", c_int64), ("tokens", POINTER(c_int32)), ("n_tokens", c_int), ("want", POINTER(c_int32)),
                ("n_want", c_int)]


class ImpTensor(Structure):
    _fields_ = [("data", c_void_p), ("dtype", c_int32), ("ndim", c_int32), ("shape", c_int64 * 4), ("stride0", c_int64)]


class ImpBatchView(Structure):
    _fields_ = [("n_tokens", c_int32), ("n_seqs", c_int32), ("n_rows", c_int32), ("decode_only", c_int32),
                ("max_q_len", c_int32), ("max_kv_len", c_int32),
                ("token_ids", c_void_p), ("positions", c_void_p), ("seq_of_token", c_void_p), ("logit_rows", c_void_p),
                ("q_start", c_void_p), ("kv_len", c_void_p), ("state_slots", c_void_p),
                ("host_q_lens", POINTER(c_int32)), ("host_starts", POINTER(c_int32)), ("host_slots", POINTER(c_int32)),
                ("stream", c_void_p), ("status", c_void_p), ("compute_dtype", c_int32), ("step", c_void_p)]


class ImpCacheView(Structure):
    _fields_ = [("kind", c_int32), ("writes", c_int32), ("k_pages", c_void_p), ("v_pages", c_void_p),
                ("num_pages", c_int32), ("kv_heads", c_int32), ("page_size", c_int32), ("head_dim", c_int32),
                ("window", c_int32), ("block_table", c_void_p), ("bt_stride", c_int32), ("n_states", c_int32),
                ("states", ImpTensor * 4)]


class ImpCall(Structure):
    _fields_ = [("batch", POINTER(ImpBatchView)), ("cache", POINTER(ImpCacheView)), ("h", ImpTensor), ("branch", ImpTensor),
                ("x", ImpTensor), ("q", ImpTensor), ("k", ImpTensor), ("out", ImpTensor), ("rows", c_void_p),
                ("n_rows", c_int32), ("has_out", c_int32)]


STRING_FN = CFUNCTYPE(c_void_p, c_void_p, c_char_p)
CREATE_FN = CFUNCTYPE(c_void_p, c_void_p, c_char_p, c_int, POINTER(c_char_p), POINTER(ImpTensor), c_int, POINTER(c_char_p),
                      POINTER(c_void_p), c_int, c_int)
FORWARD_FN = CFUNCTYPE(c_int, c_void_p, POINTER(ImpCall))
DESTROY_FN = CFUNCTYPE(None, c_void_p)
PLAN_FN = CFUNCTYPE(c_void_p, c_void_p, c_char_p)
RESOLVER_FN = CFUNCTYPE(c_void_p, c_char_p, c_int)


class ImpPartVTable(Structure):
    _fields_ = [("user", c_void_p), ("tensor_specs", STRING_FN), ("cache_spec", STRING_FN), ("part_slots", STRING_FN),
                ("create", CREATE_FN), ("forward", FORWARD_FN), ("destroy", DESTROY_FN)]


ELEM_F32, ELEM_BF16, ELEM_I32 = 0, 1, 2
COMPUTE_FP32, COMPUTE_BF16 = 0, 1

_E = c_int    # ImpError
_H = c_void_p  # opaque handles

_SIGNATURES = {
    "imp_error_string": (c_char_p, [c_int]),
    "imp_error_message": (c_char_p, []),
    "imp_version": (c_char_p, []),
    "imp_config_default": (ImpConfig, []),
    "imp_generate_params_default": (ImpGenerateParams, []),
    "imp_model_load": (_E, [c_char_p, POINTER(_H)]),
    "imp_model_random": (_E, [c_char_p, c_int64, c_float, c_float, POINTER(_H)]),
    "imp_model_write_random": (_E, [c_char_p, c_char_p, c_int64, c_float, c_float, c_char_p]),
    "imp_model_free": (None, [_H]),
    "imp_model_arch": (c_char_p, [_H]),
    "imp_model_n_layers": (c_int, [_H]),
    "imp_model_d_model": (c_int, [_H]),
    "imp_model_vocab_size": (c_int, [_H]),
    "imp_model_max_seq_len": (c_int, [_H]),
    "imp_model_config_json": (c_char_p, [_H]),
    "imp_model_plan_json": (c_char_p, [_H]),
    "imp_model_tensor_info_json": (c_char_p, [_H, c_int]),
    "imp_context_create": (_E, [_H, POINTER(ImpConfig), POINTER(_H)]),
    "imp_context_free": (None, [_H]),
    "imp_context_reset": (_E, [_H]),
    "imp_context_info_json": (c_char_p, [_H]),
    "imp_context_timer_start": (_E, [_H]),
    "imp_context_timer_stop": (_E, [_H, POINTER(c_float)]),
    "imp_context_set_eos": (_E, [_H, POINTER(c_int32), c_int]),
    "imp_context_check": (_E, [_H]),
    "imp_submit": (_E, [_H, POINTER(c_int32), c_int, POINTER(ImpGenerateParams), POINTER(c_int64)]),
    "imp_cancel": (_E, [_H, c_int64]),
    "imp_step": (_E, [_H, POINTER(ImpStepOutput), c_int, POINTER(c_int)]),
    "imp_drain": (_E, [_H, POINTER(ImpStepOutput), c_int, POINTER(c_int)]),
    "imp_has_work": (c_int, [_H]),
    "imp_request_info": (_E, [_H, c_int64, POINTER(ImpRequestInfo)]),
    "imp_request_output": (_E, [_H, c_int64, POINTER(c_int32), c_int, POINTER(c_int)]),
    "imp_request_release": (_E, [_H, c_int64]),
    "imp_generate": (_E, [_H, POINTER(c_int32), c_int, POINTER(ImpGenerateParams), POINTER(c_int32), c_int, POINTER(c_int)]),
    "imp_prefill": (_E, [_H, POINTER(c_int32), c_int, POINTER(ImpGenerateParams)]),
    "imp_decode_step": (_E, [_H, POINTER(c_int32)]),
    "imp_step_tokens": (_E, [_H, POINTER(ImpStepEntry), c_int, c_void_p, c_size_t]),
    "imp_end": (_E, [_H, c_int64]),
    # parts and architectures
    "imp_register_part": (_E, [c_char_p, c_char_p, POINTER(ImpPartVTable)]),
    "imp_unregister_part": (_E, [c_char_p, c_char_p]),
    "imp_known_parts": (c_char_p, [c_char_p]),
    "imp_part_set_error": (None, [c_char_p]),
    "imp_part_forward": (_E, [c_void_p, POINTER(ImpCall)]),
    "imp_step_alloc": (c_void_p, [c_void_p, c_size_t]),
    "imp_register_architecture": (_E, [c_char_p, PLAN_FN, c_void_p]),
    "imp_unregister_architecture": (_E, [c_char_p]),
    "imp_known_architectures": (c_char_p, []),
    "imp_config_parse": (_E, [c_char_p, c_char_p, POINTER(c_char_p)]),
    "imp_plan_for_config": (_E, [c_char_p, POINTER(c_char_p)]),
    "imp_plan_expected_tensors": (_E, [c_char_p, POINTER(c_char_p)]),
    "imp_set_variant_resolver": (None, [RESOLVER_FN]),
    # single parts
    "imp_bench_create": (_E, [c_int, c_int, c_char_p, c_int, c_int, c_int, c_int, c_int, POINTER(_H)]),
    "imp_bench_free": (None, [_H]),
    "imp_bench_build_part": (_E, [_H, c_char_p, c_char_p, c_int, POINTER(c_char_p), POINTER(ImpTensor), POINTER(c_void_p)]),
    "imp_bench_build_block": (_E, [_H, c_char_p, c_char_p, c_int, POINTER(c_char_p), POINTER(c_void_p), POINTER(c_void_p)]),
    "imp_bench_prepare": (_E, [_H, POINTER(ImpStepEntry), c_int, POINTER(POINTER(ImpBatchView))]),
    "imp_bench_cache_view": (_E, [_H, c_int, c_int, POINTER(POINTER(ImpCacheView))]),
    "imp_bench_commit": (_E, [_H]),
    "imp_bench_end": (_E, [_H, c_int64]),
    "imp_bench_sync": (_E, [_H]),
    "imp_bench_stream": (c_void_p, [_H]),
    "imp_bench_cache_info_json": (c_char_p, [_H]),
    # host components
    "imp_cache_create": (_E, [c_char_p, c_int, c_int, c_int, c_int, POINTER(_H)]),
    "imp_cache_free": (None, [_H]),
    "imp_cache_add_request": (_E, [_H, c_int64, POINTER(c_int)]),
    "imp_cache_reserve": (_E, [_H, c_int64, c_int]),
    "imp_cache_commit": (_E, [_H, c_int64, c_int, POINTER(c_int)]),
    "imp_cache_release": (_E, [_H, c_int64]),
    "imp_cache_check": (_E, [_H]),
    "imp_cache_info_json": (c_char_p, [_H]),
    "imp_scheduler_create": (_E, [_H, c_int, c_int, c_int, c_int, POINTER(_H)]),
    "imp_scheduler_free": (None, [_H]),
    "imp_scheduler_add": (_E, [_H, c_int64, POINTER(c_int32), c_int, POINTER(ImpGenerateParams), POINTER(c_int32), c_int,
                               POINTER(c_int)]),
    "imp_scheduler_cancel": (_E, [_H, c_int64]),
    "imp_scheduler_schedule": (_E, [_H, POINTER(c_char_p)]),
    "imp_scheduler_complete": (_E, [_H, POINTER(c_int32), c_int, POINTER(c_char_p)]),
    "imp_scheduler_info_json": (c_char_p, [_H]),
}

_lib = None
_lock = threading.Lock()
_keep = []   # callbacks handed to the library must outlive it


def _resolve_variant(source: bytes, head_dim: int):
    """Build (on first use) and name the attention library of a head size for the C++ host."""
    from .csrc.build import build_variant
    try:
        path = build_variant(source.decode(), {"IMP_ATTN_DH": int(head_dim)})
    except Exception as e:  # reported by the host as "not built"
        import sys
        print(f"[imp_b200] cannot build {source.decode()} for head size {head_dim}: {e}", file=sys.stderr)
        return None
    buf = ctypes.create_string_buffer(path.encode())
    _keep.append(buf)
    return ctypes.addressof(buf)


def load():
    """The ctypes handle of the library, built on first use.  Raises if it cannot be built or loaded:
    there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from .csrc.build import build
        path = build()
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(IMP_ERROR_INTERNAL, f"cannot load the library {path}: {e}") from None
        for name, (restype, argtypes) in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                raise KernelError(IMP_ERROR_INTERNAL, f"the compiled library lacks the entry point {name}; rebuild it "
                                  "(python -m imp_b200.csrc.build --force)") from None
            fn.restype = restype
            fn.argtypes = argtypes
        resolver = RESOLVER_FN(_resolve_variant)
        _keep.append(resolver)
        lib.imp_set_variant_resolver(resolver)
        _lib = lib
        return lib


def loaded_library_path():
    return getattr(_lib, "_name", None)


_BY_CODE = {IMP_ERROR_CUDA: KernelError, IMP_ERROR_OUT_OF_MEMORY: OutOfPages}


def check(rc: int, kind=None) -> None:
    """Raise the exception that fits a failed call: `kind` for model errors, else by the error code."""
    if rc == IMP_SUCCESS:
        return
    msg = load().imp_error_message().decode(errors="replace")
    if rc == IMP_ERROR_INVALID_MODEL and kind is not None:
        raise kind(rc, msg)
    if rc == IMP_ERROR_FILE_NOT_FOUND and kind is not None:
        raise kind(rc, msg)
    if rc == IMP_ERROR_INVALID_ARG:
        raise _InvalidArg(rc, msg)
    raise _BY_CODE.get(rc, ImpError)(rc, msg)


class _InvalidArg(ImpError, ValueError):
    pass


InvalidArgument = _InvalidArg


def model_error(rc: int) -> None:
    """Errors of model loading: configuration, container and binding errors by their messages."""
    if rc == IMP_SUCCESS:
        return
    msg = load().imp_error_message().decode(errors="replace")
    if "does not match the model" in msg:
        raise WeightError(rc, msg)
    if ".safetensors" in msg and rc in (IMP_ERROR_INVALID_MODEL, IMP_ERROR_FILE_NOT_FOUND):
        raise SafetensorsError(rc, msg)
    if rc in (IMP_ERROR_INVALID_MODEL, IMP_ERROR_FILE_NOT_FOUND):
        raise ConfigError(rc, msg)
    check(rc)


def text(p) -> str:
    return p.decode() if p else ""


def call_json(fn, *args, kind=ConfigError):
    """Call an entry point whose last argument receives a JSON string; returns the parsed value."""
    out = c_char_p()
    rc = fn(*args, ctypes.byref(out))
    if rc != IMP_SUCCESS:
        if kind is ConfigError:
            model_error(rc)
        check(rc, kind)
    return json.loads(out.value.decode())


def int32_array(values):
    n = len(values)
    arr = (c_int32 * n)(*values) if n else (c_int32 * 1)()
    return arr, n
