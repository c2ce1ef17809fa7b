"""Part kinds written in Python: base classes, and the glue that registers them with the library.

The library builds a model from parts by kind (include/imp_b200/imp_parts.h).  A
kind can be implemented outside the library as a table of C functions; this
module makes such a table from a Python class, so that a new mixer,
feed-forward, norm, position encoding, block, embedding or head can be
defined in a test or a user's module and used by any plan without touching the
library.  Device memory reaches the class as torch tensors that alias the
library's buffers, and its work runs on the library's stream.

Categories and what each class provides (all also `tensor_specs(params)`):

  norm          add_norm(h, branch, rows=None) -> normalised activations; h is the 32-bit
                residual stream, `branch` (or None) is added into it first; with `rows` only
                those rows are produced and h is left as it is.
  position      apply(q, k, ctx): rewrite q [T, Hq, Dh] and k [T, Hkv, Dh] in place.
  mixer         cache_spec(params) (classmethod) -> PagedKVSpec | StateSpec | None;
                forward(x, ctx, cache) -> [T, hidden] branch output.
  feed_forward  forward(x, ctx) -> [T, hidden] branch output.
  block         part_slots(params) (classmethod) -> [(slot name, category), ...] (at most one
                mixer); built with its parts by slot name (handles with the methods above);
                forward(h, pending, ctx, cache) -> the branch it leaves pending, or None.
  embedding     forward(token_ids, ctx) -> [T, hidden] float32 stream.
  head          forward(x_rows) -> [R, vocab] float32 logits.

A part written in Python never meets an unsummed branch (the library adds the
parts first), and a model that holds one does not capture CUDA graphs.
"""
from __future__ import annotations

import ctypes
import json
import threading
import traceback
from typing import Any, Dict, List, Optional

from .. import capi
from .plan import TensorSpec

_local = threading.local()   # the batch of the part call that is under way (for handles called from a block)


# ----------------------------------------------------------------------------- tensor views
class _Alias:
    def __init__(self, t: "capi.ImpTensor"):
        shape = tuple(int(t.shape[i]) for i in range(t.ndim))
        item = 2 if t.dtype == capi.ELEM_BF16 else 4
        inner = 1
        for s in shape[1:]:
            inner *= s
        strides, acc = [], item
        for s in reversed(shape[1:]):
            strides.append(acc)
            acc *= s
        strides = tuple([int(t.stride0) * item] + list(reversed(strides))) if shape else ()
        self.__cuda_array_interface__ = {
            "shape": shape, "typestr": {capi.ELEM_F32: "<f4", capi.ELEM_BF16: "<i2", capi.ELEM_I32: "<i4"}[t.dtype],
            "data": (int(t.data), False), "version": 2, "strides": strides if shape and int(t.stride0) != inner else None}


def as_torch(t: "capi.ImpTensor", device: int = 0):
    """A torch tensor over the memory an ImpTensor names (None for an empty view)."""
    import torch
    if not t.data:
        return None
    n = 1
    for i in range(t.ndim):
        n *= int(t.shape[i])
    if n == 0:
        dt = {capi.ELEM_F32: torch.float32, capi.ELEM_BF16: torch.bfloat16, capi.ELEM_I32: torch.int32}[t.dtype]
        return torch.empty(tuple(int(t.shape[i]) for i in range(t.ndim)), dtype=dt, device=f"cuda:{device}")
    x = torch.as_tensor(_Alias(t), device=f"cuda:{device}")
    return x.view(torch.bfloat16) if t.dtype == capi.ELEM_BF16 else x


def int_view(ptr, n: int, device: int = 0):
    import torch
    if not ptr or n <= 0:
        return torch.empty(0, dtype=torch.int32, device=f"cuda:{device}")
    t = capi.ImpTensor()
    t.data, t.dtype, t.ndim, t.stride0 = ptr, capi.ELEM_I32, 1, 1
    t.shape[0] = n
    return as_torch(t, device)


def to_imp(x) -> "capi.ImpTensor":
    """The ImpTensor that names a torch tensor's memory (rows may be strided, the rest dense)."""
    import torch
    t = capi.ImpTensor()
    if x is None:
        return t
    code = {torch.float32: capi.ELEM_F32, torch.bfloat16: capi.ELEM_BF16, torch.int32: capi.ELEM_I32}.get(x.dtype)
    if code is None:
        raise TypeError(f"element type {x.dtype} cannot cross into the library (float32, bfloat16, int32)")
    if not x.is_cuda or x.dim() > 4 or x.dim() == 0:
        raise TypeError("the library takes CUDA tensors of one to four dimensions")
    if x.dim() > 1 and not x[0].is_contiguous():
        x = x.contiguous()
    t.data, t.dtype, t.ndim = x.data_ptr(), code, x.dim()
    for i, s in enumerate(x.shape):
        t.shape[i] = s
    t.stride0 = x.stride(0) if x.shape[0] > 1 or x.dim() == 1 else max(1, x[0].numel() if x.dim() > 1 else 1)
    t._keep = x
    return t


# ------------------------------------------------------------------------------ what parts see
class Runtime:
    """What every part is built with: the precision and the device."""

    def __init__(self, compute_dtype: int, device_id: int):
        import torch
        self.dtype = torch.float32 if compute_dtype == capi.ELEM_F32 else torch.bfloat16
        self.device = torch.device(f"cuda:{device_id}")
        self.device_id = device_id

    @property
    def is_float32(self) -> bool:
        import torch
        return self.dtype == torch.float32

    def empty(self, shape, dtype=None):
        import torch
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


class StepContext:
    """The batch of one step as a part sees it: device arrays (int32) and their host-side sizes."""

    def __init__(self, view: "capi.ImpBatchView", view_ptr, device: int):
        self._view, self._ptr = view, view_ptr
        self.n_tokens, self.n_seqs, self.n_rows = view.n_tokens, view.n_seqs, view.n_rows
        T, B = view.n_tokens, view.n_seqs
        self.decode_only = bool(view.decode_only)
        self.max_q_len, self.max_kv_len = view.max_q_len, view.max_kv_len
        self.token_ids = int_view(view.token_ids, T, device)
        self.positions = int_view(view.positions, T, device)
        self.seq_of_token = int_view(view.seq_of_token, T, device)
        self.logit_rows = int_view(view.logit_rows, view.n_rows, device)
        self.q_start = int_view(view.q_start, B + 1, device)
        self.kv_len = int_view(view.kv_len, B, device)
        self.state_slots = int_view(view.state_slots, B, device)
        self.q_lens = [int(view.host_q_lens[i]) for i in range(B)]
        self.starts = [int(view.host_starts[i]) for i in range(B)]
        self.slots = [int(view.host_slots[i]) for i in range(B)]
        self.fresh = [s == 0 for s in self.starts]
        self.stream = view.stream


class LayerCache:
    """What a mixer gets of the cache for one step.

    kind "paged": `kv` is [2, pages, kv_heads, page_size, head_dim] (0 = keys, 1 = values),
    `block_table` [B, max_pages] int32 rows in batch order, `writes` tells whether this layer owns the
    cache (False when it reads another layer's).  kind "state": `states` are the tensors [slots, ...]
    of the cache spec, in its order (`state` is the first); the request's slot ids are ctx.state_slots
    (ctx.slots on the host), and ctx.fresh marks requests whose state starts at zero in this step."""

    def __init__(self, view: "capi.ImpCacheView", view_ptr, n_seqs: int, device: int):
        self._view, self._ptr = view, view_ptr
        self.kind = {0: None, 1: "paged", 2: "state"}[view.kind]
        self.writes = bool(view.writes)
        self.page_size, self.window = view.page_size, view.window
        self.kv = self.block_table = self.state = None
        self.states: List[Any] = []
        if view.kind == 1:
            t = capi.ImpTensor()
            dt = None
            # keys and values of a layer lie one behind the other
            t.data, t.ndim = view.k_pages, 4
            elem = (view.v_pages - view.k_pages) // max(1, view.num_pages * view.kv_heads * view.page_size * view.head_dim)
            t.dtype = capi.ELEM_F32 if elem == 4 else capi.ELEM_BF16
            t.shape[0], t.shape[1], t.shape[2], t.shape[3] = 2 * view.num_pages, view.kv_heads, view.page_size, view.head_dim
            t.stride0 = view.kv_heads * view.page_size * view.head_dim
            self.kv = as_torch(t, device).view(2, view.num_pages, view.kv_heads, view.page_size, view.head_dim)
            bt = capi.ImpTensor()
            bt.data, bt.dtype, bt.ndim, bt.stride0 = view.block_table, capi.ELEM_I32, 2, view.bt_stride
            bt.shape[0], bt.shape[1] = n_seqs, view.bt_stride
            self.block_table = as_torch(bt, device)
        elif view.kind == 2:
            self.states = [as_torch(view.states[i], device) for i in range(view.n_states)]
            self.state = self.states[0] if self.states else None


# ----------------------------------------------------------------------------------- parts
class Part:
    category = "part"

    def __init__(self, params: Dict[str, Any], tensors: Dict[str, Any], rt: Runtime):
        self.params = params
        self.tensors = tensors
        self.rt = rt

    @classmethod
    def tensor_specs(cls, params: Dict[str, Any]) -> Dict[str, TensorSpec]:
        return {}


class Norm(Part):
    category = "norm"

    def add_norm(self, h, branch, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    category = "position"

    def apply(self, q, k, ctx) -> None:
        """Encode positions into q [T, Hq, Dh] and k [T, Hkv, Dh] in place."""
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"

    @classmethod
    def cache_spec(cls, params: Dict[str, Any]):
        return None

    def forward(self, x, ctx, cache):
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, x, ctx):
        raise NotImplementedError


class Embedding(Part):
    category = "embedding"

    def forward(self, token_ids, ctx):
        raise NotImplementedError


class Head(Part):
    category = "head"

    def forward(self, x):
        raise NotImplementedError


class Block:
    """Arrangement of one layer.  Built from the layer's already built parts, by slot name."""

    category = "block"

    def __init__(self, params: Dict[str, Any], parts: Dict[str, "PartHandle"], rt: Runtime):
        self.params, self.parts, self.rt = params, parts, rt

    @classmethod
    def part_slots(cls, params: Dict[str, Any]):
        return [("mixer_norm", "norm"), ("mixer", "mixer"), ("ffn_norm", "norm"), ("feed_forward", "feed_forward")]

    @classmethod
    def tensor_specs(cls, params):
        return {}

    def forward(self, h, pending, ctx, cache):
        raise NotImplementedError


# ------------------------------------------------------------------- parts of the library, called
class PartHandle:
    """A built part (the library's own or a registered one) that Python code can run: what a block
    written in Python does with its parts.  Outputs alias the library's workspace and live until
    the end of the layer."""

    def __init__(self, ptr, device: int = 0):
        self.ptr, self.device = ptr, device

    def _call(self, call: "capi.ImpCall", ctx: Optional[StepContext]):
        ctx = ctx or getattr(_local, "ctx", None)
        if ctx is None:
            raise RuntimeError("a part can only run inside a step (no batch is under way)")
        call.batch = ctypes.cast(ctx._ptr, ctypes.POINTER(capi.ImpBatchView))
        capi.check(capi.load().imp_part_forward(self.ptr, ctypes.byref(call)))
        return call

    def add_norm(self, h, branch=None, rows=None, ctx: Optional[StepContext] = None):
        c = capi.ImpCall()
        c.h, c.branch = to_imp(h), to_imp(branch)
        if rows is not None:
            c.rows, c.n_rows = rows.data_ptr(), rows.numel()
        return as_torch(self._call(c, ctx).out, self.device)

    def forward(self, x, ctx: Optional[StepContext] = None, cache: Optional[LayerCache] = None):
        """mixer: forward(x, ctx, cache); feed_forward: forward(x, ctx); head: forward(x)."""
        c = capi.ImpCall()
        c.x = to_imp(x)
        if cache is not None:
            c.cache = ctypes.cast(cache._ptr, ctypes.POINTER(capi.ImpCacheView))
        return as_torch(self._call(c, ctx).out, self.device)

    def embed(self, ctx: Optional[StepContext] = None):
        return as_torch(self._call(capi.ImpCall(), ctx).h, self.device)

    def block_forward(self, h, pending, ctx: Optional[StepContext] = None, cache: Optional[LayerCache] = None):
        c = capi.ImpCall()
        c.h, c.branch = to_imp(h), to_imp(pending)
        if cache is not None:
            c.cache = ctypes.cast(cache._ptr, ctypes.POINTER(capi.ImpCacheView))
        self._call(c, ctx)
        return as_torch(c.out, self.device) if c.has_out else None

    def apply(self, q, k, ctx: Optional[StepContext] = None):
        c = capi.ImpCall()
        c.q, c.k = to_imp(q), to_imp(k)
        self._call(c, ctx)


# ------------------------------------------------------------------------------- registration
_instances: Dict[int, Any] = {}
_next_instance = [1]
_registered: Dict[tuple, Any] = {}   # (category, kind) -> what must outlive the library's use of it


def _spec_json(spec):
    return spec.to_json() if hasattr(spec, "to_json") else spec


def register_python_part(category: str, kind: str, cls: type, replace: bool = False) -> None:
    """Register `cls` as the part kind `kind` of `category` with the library."""
    lib = capi.load()
    strings = {}

    def returns(name, fn):
        def wrapped(_user, params_json):
            try:
                text = json.dumps(fn(json.loads(params_json.decode()))).encode()
                strings[name] = ctypes.create_string_buffer(text)
                return ctypes.addressof(strings[name])
            except Exception as e:
                lib.imp_part_set_error(f"{type(e).__name__}: {e}".encode())
                return None
        return capi.STRING_FN(wrapped)

    def tensor_specs(params):
        return {k: _spec_json(v) for k, v in cls.tensor_specs(params).items()}

    def cache_spec(params):
        return _spec_json(cls.cache_spec(params))

    def part_slots(params):
        return [{"name": n, "category": c} for n, c in cls.part_slots(params)]

    def create(_user, params_json, n_tensors, names, tensors, n_parts, part_names, parts, compute_dtype, device_id):
        try:
            import torch
            rt = Runtime(compute_dtype, device_id)
            params = json.loads(params_json.decode())
            with torch.cuda.device(device_id):
                if category == "block":
                    handles = {part_names[i].decode(): PartHandle(parts[i], device_id) for i in range(n_parts)}
                    obj = cls(params, handles, rt)
                else:
                    views = {names[i].decode(): as_torch(tensors[i], device_id) for i in range(n_tensors)}
                    obj = cls(params, views, rt)
            key = _next_instance[0]
            _next_instance[0] += 1
            _instances[key] = obj
            return key
        except Exception as e:
            lib.imp_part_set_error(f"{type(e).__name__}: {e}\n{traceback.format_exc()}".encode())
            return None

    def forward(self_key, call_ptr):
        try:
            import torch
            obj = _instances[self_key]
            call = call_ptr.contents
            dev = obj.rt.device_id
            ctx = StepContext(call.batch.contents, ctypes.addressof(call.batch.contents), dev)
            cache = None
            if call.cache:
                cache = LayerCache(call.cache.contents, ctypes.addressof(call.cache.contents), ctx.n_seqs, dev)
            before = getattr(_local, "ctx", None)
            _local.ctx = ctx
            try:
                with torch.cuda.device(dev), torch.cuda.stream(torch.cuda.ExternalStream(ctx.stream, device=obj.rt.device)):
                    out = as_torch(call.out, dev)
                    if category == "norm":
                        rows = int_view(call.rows, call.n_rows, dev) if call.rows else None
                        out.copy_(obj.add_norm(as_torch(call.h, dev), as_torch(call.branch, dev), rows))
                    elif category == "mixer":
                        out.copy_(obj.forward(as_torch(call.x, dev), ctx, cache))
                    elif category == "feed_forward":
                        out.copy_(obj.forward(as_torch(call.x, dev), ctx))
                    elif category == "position":
                        obj.apply(as_torch(call.q, dev), as_torch(call.k, dev), ctx)
                    elif category == "embedding":
                        as_torch(call.h, dev).copy_(obj.forward(ctx.token_ids, ctx))
                    elif category == "head":
                        out.copy_(obj.forward(as_torch(call.x, dev)))
                    elif category == "block":
                        pending = obj.forward(as_torch(call.h, dev), as_torch(call.branch, dev), ctx, cache)
                        call.has_out = 0 if pending is None else 1
                        if pending is not None:
                            out.copy_(pending)
            finally:
                _local.ctx = before
            return 0
        except Exception as e:
            lib.imp_part_set_error(f"{type(e).__name__}: {e}\n{traceback.format_exc()}".encode())
            return 1

    def destroy(self_key):
        _instances.pop(self_key, None)

    vt = capi.ImpPartVTable()
    keep = [returns("tensor_specs", tensor_specs), capi.CREATE_FN(create), capi.FORWARD_FN(forward), capi.DESTROY_FN(destroy)]
    vt.tensor_specs, vt.create, vt.forward, vt.destroy = keep
    if category == "mixer":
        keep.append(returns("cache_spec", cache_spec))
        vt.cache_spec = keep[-1]
    if category == "block":
        keep.append(returns("part_slots", part_slots))
        vt.part_slots = keep[-1]
    if (category, kind) in _registered and replace:
        capi.check(lib.imp_unregister_part(category.encode(), kind.encode()))
    capi.check(lib.imp_register_part(category.encode(), kind.encode(), ctypes.byref(vt)))
    _registered[(category, kind)] = (vt, keep, strings, cls)
