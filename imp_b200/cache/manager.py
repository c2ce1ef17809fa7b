"""The library's cache manager (csrc/host/cache.cpp) as a Python object, without a device.

Pages of keys and values with a block table per request, one pool per group of
layers with the same needs, and slots of fixed-size state.  The bookkeeping
runs in the library; this wrapper maps the caller's request ids to integers
and reads the state back as JSON.  `PagedKVSpec` and `StateSpec` are what a
mixer class returns from `cache_spec(params)`.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from .. import capi
from ..capi import CacheError, OutOfPages  # noqa: F401  (re-exported)


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values per token: [kv_heads, head_dim] each.  window == 0 keeps every token;
    window == W keeps what a query at position p may still see: positions > p - W."""

    num_kv_heads: int
    head_dim: int
    window: int = 0

    kind = "paged"

    def to_json(self):
        return {"kind": "paged", "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim, "window": self.window}


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size per request, zero at a request's start: one tensor of `shape` and `dtype`, or
    several named ones, `tensors` = ((name, shape, dtype), ...)."""

    shape: Tuple[int, ...] = ()
    dtype: str = "float32"
    tensors: Tuple[Tuple[str, Tuple[int, ...], str], ...] = ()

    kind = "state"

    def to_json(self):
        ts = self.tensors or (("state", tuple(self.shape), self.dtype),)
        return {"kind": "state", "tensors": [{"name": n, "shape": list(s), "dtype": d} for n, s, d in ts]}


def spec_json(spec):
    return None if spec is None else spec.to_json() if hasattr(spec, "to_json") else spec


def _check(rc: int) -> None:
    if rc == capi.IMP_SUCCESS:
        return
    msg = capi.load().imp_error_message().decode(errors="replace")
    if rc == capi.IMP_ERROR_OUT_OF_MEMORY:
        raise OutOfPages(rc, msg)
    raise CacheError(rc, msg)


class _Group:
    def __init__(self, mgr: "CacheManager", index: int, kind: str):
        self._mgr, self._index, self._kind = mgr, index, kind

    def _j(self):
        return self._mgr.info()[self._kind][self._index]

    @property
    def layers(self) -> List[int]:
        return self._j()["layers"]

    @property
    def tables(self) -> Dict[Hashable, List[int]]:
        return {self._mgr._names[int(k)]: v for k, v in self._j()["tables"].items()}

    @property
    def n_free(self) -> int:
        return self._j()["free"]

    def first_live_page(self, length: int) -> int:
        w = self._j().get("window", 0)
        return 0 if w <= 0 else max(0, length - w + 1) // self._mgr.page_size


@dataclass
class LayerCacheRef:
    group: int
    index: int
    kind: str


class _Slots:
    def __init__(self, mgr):
        self._mgr = mgr

    @property
    def n_free(self) -> int:
        return self._mgr.info()["free_slots"]

    @property
    def num_pages(self) -> int:
        return self._mgr.info()["slots"]


class CacheManager:
    """`layer_specs[j]` is what run position j asks for (a PagedKVSpec, a StateSpec or None)."""

    def __init__(self, layer_specs: Sequence[Optional[object]], page_size: int, num_pages: int, num_state_slots: int = 1,
                 max_pages_per_seq: Optional[int] = None):
        lib = capi.load()
        self.page_size, self.num_pages = page_size, num_pages
        h = ctypes.c_void_p()
        specs = json.dumps([spec_json(s) for s in layer_specs]).encode()
        rc = lib.imp_cache_create(specs, page_size, num_pages, max(1, num_state_slots), max_pages_per_seq or 0, ctypes.byref(h))
        if rc != capi.IMP_SUCCESS:
            raise ValueError(lib.imp_error_message().decode())
        self.handle = h
        self._ids: Dict[Hashable, int] = {}
        self._names: Dict[int, Hashable] = {}
        self._next = 0
        self.slots = _Slots(self)

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h:
            capi.load().imp_cache_free(h)

    def _id(self, rid: Hashable, create: bool = False) -> int:
        if rid not in self._ids:
            if not create:
                return -1 - abs(hash(rid)) % (1 << 40)   # an id the library does not know
            self._ids[rid] = self._next
            self._names[self._next] = rid
            self._next += 1
        return self._ids[rid]

    def info(self):
        return json.loads(capi.text(capi.load().imp_cache_info_json(self.handle)))

    # ------------------------------------------------------------------ requests
    @property
    def paged(self) -> List[_Group]:
        return [_Group(self, i, "paged") for i in range(len(self.info()["paged"]))]

    @property
    def state(self) -> List[_Group]:
        return [_Group(self, i, "state") for i in range(len(self.info()["state"]))]

    @property
    def layer_ref(self) -> List[Optional[LayerCacheRef]]:
        return [None if r["kind"] == "none" else LayerCacheRef(r["group"], r["index"], r["kind"])
                for r in self.info()["positions"]]

    def live_requests(self):
        return [self._names[int(k)] for k in self.info()["requests"]]

    def has(self, rid: Hashable) -> bool:
        return rid in self._ids and str(self._ids[rid]) in self.info()["requests"]

    def length(self, rid: Hashable) -> int:
        return self.info()["requests"][str(self._ids[rid])]["length"]

    def slot_of(self, rid: Hashable) -> int:
        return self.info()["requests"][str(self._ids[rid])]["slot"]

    def add_request(self, rid: Hashable) -> int:
        slot = ctypes.c_int(-1)
        _check(capi.load().imp_cache_add_request(self.handle, self._id(rid, create=True), ctypes.byref(slot)))
        return slot.value

    def free_pages(self) -> int:
        return self.info()["free_pages"]

    def reserve(self, rid: Hashable, new_len: int) -> None:
        _check(capi.load().imp_cache_reserve(self.handle, self._id(rid), new_len))

    def commit(self, rid: Hashable, new_len: int) -> int:
        n = ctypes.c_int(0)
        _check(capi.load().imp_cache_commit(self.handle, self._id(rid), new_len, ctypes.byref(n)))
        return n.value

    def release(self, rid: Hashable) -> None:
        _check(capi.load().imp_cache_release(self.handle, self._id(rid)))

    def block_table(self, group: int, rid: Hashable) -> List[int]:
        return self.info()["paged"][group]["tables"][str(self._ids[rid])]

    def check_invariants(self) -> None:
        rc = capi.load().imp_cache_check(self.handle)
        assert rc == capi.IMP_SUCCESS, capi.load().imp_error_message().decode()
