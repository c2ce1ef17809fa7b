"""Driving single parts: a device context without a model.

`PartBench` owns what the library's `imp_bench_*` calls give: a stream, a status
word, a workspace, a cache manager built from a list of cache specs (one per
run position), and the batch builder of the step function.  Parts are built
from a spec and device tensors and run against batches the bench prepares:
how the tests drive each part alone, and how a tool can time one.
"""
from __future__ import annotations

import ctypes
import json
from typing import Dict, Hashable, Optional, Sequence

from .. import capi
from ..cache.manager import spec_json
from .base import LayerCache, PartHandle, StepContext, to_imp
from .plan import PartSpec


class PartBench:
    def __init__(self, dtype: str = "bfloat16", cache_specs: Sequence[object] = (), page_size: int = 4, num_pages: int = 64,
                 slots: int = 4, max_tokens: int = 256, max_seq_len: int = 256, device_id: int = 0):
        lib = capi.load()
        h = ctypes.c_void_p()
        c = capi.COMPUTE_FP32 if dtype in ("float32", "fp32") else capi.COMPUTE_BF16
        specs = json.dumps([spec_json(s) for s in cache_specs]).encode()
        capi.check(lib.imp_bench_create(device_id, c, specs, page_size, num_pages, slots, max_tokens, max_seq_len, ctypes.byref(h)))
        self.handle, self.device_id, self.dtype = h, device_id, dtype
        self._ids: Dict[Hashable, int] = {}
        self.ctx: Optional[StepContext] = None

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h:
            capi.load().imp_bench_free(h)

    @property
    def stream(self) -> int:
        return capi.load().imp_bench_stream(self.handle)

    def build(self, category: str, spec: PartSpec, tensors: Optional[Dict[str, object]] = None) -> PartHandle:
        """Build a part from its spec and device tensors by local name (torch tensors; copied)."""
        import torch
        tensors = tensors or {}
        torch.cuda.synchronize()
        names = (ctypes.c_char_p * max(len(tensors), 1))(*[n.encode() for n in tensors])
        views = (capi.ImpTensor * max(len(tensors), 1))(*[to_imp(t.contiguous()) for t in tensors.values()])
        out = ctypes.c_void_p()
        text = json.dumps(spec.to_json() if hasattr(spec, "to_json") else spec).encode()
        capi.check(capi.load().imp_bench_build_part(self.handle, category.encode(), text, len(tensors), names, views,
                                                    ctypes.byref(out)))
        return PartHandle(out.value, self.device_id)

    def build_block(self, kind: str, parts: Dict[str, PartHandle], params: Optional[dict] = None) -> PartHandle:
        """A block of kind `kind` over parts this bench built, by slot name."""
        n = len(parts)
        names = (ctypes.c_char_p * max(n, 1))(*[k.encode() for k in parts])
        ptrs = (ctypes.c_void_p * max(n, 1))(*[h.ptr for h in parts.values()])
        out = ctypes.c_void_p()
        capi.check(capi.load().imp_bench_build_block(self.handle, kind.encode(), json.dumps(params or {}).encode(), n, names,
                                                     ptrs, ctypes.byref(out)))
        return PartHandle(out.value, self.device_id)

    def _rid(self, rid: Hashable) -> int:
        if rid not in self._ids:
            self._ids[rid] = len(self._ids)
        return self._ids[rid]

    def prepare(self, entries) -> StepContext:
        """entries: (rid, tokens, want) triples or StepEntry objects; reserves cache, uploads the batch."""
        import torch
        torch.cuda.synchronize()
        n = len(entries)
        arr = (capi.ImpStepEntry * max(n, 1))()
        keep = []
        for i, e in enumerate(entries):
            rid, tokens, want = (e.rid, e.tokens, e.want) if hasattr(e, "rid") else e
            toks, nt = capi.int32_array([int(t) for t in tokens])
            w, nw = capi.int32_array([int(x) for x in want])
            keep += [toks, w]
            arr[i].id, arr[i].tokens, arr[i].n_tokens, arr[i].want, arr[i].n_want = self._rid(rid), toks, nt, w, nw
        view = ctypes.POINTER(capi.ImpBatchView)()
        capi.check(capi.load().imp_bench_prepare(self.handle, arr, n, ctypes.byref(view)))
        self.ctx = StepContext(view.contents, ctypes.addressof(view.contents), self.device_id)
        return self.ctx

    def cache_view(self, position: int = 0, writes: bool = True) -> LayerCache:
        view = ctypes.POINTER(capi.ImpCacheView)()
        capi.check(capi.load().imp_bench_cache_view(self.handle, position, int(writes), ctypes.byref(view)))
        # the library reuses one view per bench: keep a copy
        copy = capi.ImpCacheView.from_buffer_copy(view.contents)
        lc = LayerCache(copy, ctypes.addressof(copy), self.ctx.n_seqs, self.device_id)
        lc._copy = copy
        return lc

    def commit(self) -> None:
        capi.check(capi.load().imp_bench_commit(self.handle))

    def end(self, rid: Hashable) -> None:
        capi.check(capi.load().imp_bench_end(self.handle, self._rid(rid)))

    def sync(self) -> None:
        """Wait for the bench's stream; raises if a kernel reported a bad index."""
        capi.check(capi.load().imp_bench_sync(self.handle))

    def cache_info(self):
        return json.loads(capi.text(capi.load().imp_bench_cache_info_json(self.handle)))
