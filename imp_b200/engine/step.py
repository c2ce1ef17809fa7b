"""The step function: one batch of (request, its next tokens) through the model.

A batch holds, for each request in it, the tokens that come next for that
request: a portion of its prompt of any length, or a single decoded token.
Everything is one flat list of tokens with, per token, its position and the
index of its sequence in the batch; per sequence, its row of each cache
group's block table, its state slot and its length after the step.  The step
reserves pages, uploads these arrays with one copy from pinned memory, runs
the model once and returns the logits of the wanted rows.

The reference builds two kinds of batches, never mixed: one prompt portion
with a flat block table, or B decode tokens with token i belonging to sequence
i (src/runtime/batch.cpp:86-135, src/runtime/engine.cpp:1203-1258, 1655-1713);
its `seq_offsets` array is uploaded but never read by a kernel
(src/graph/executor.h:122).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, OutOfPages
from ..ops import kernels as K
from ..parts.base import Runtime
from .model import DecoderModel


ATTENTION_TILE = 16   # query tokens per attention tile (the row count of one tensor-core tile)


@dataclass
class StepEntry:
    """The next tokens of one request, and which of them should yield logits."""

    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # indices into `tokens`


class StepContext:
    """Device views of one batch (all int32), plus their host-side sizes."""

    __slots__ = ("n_tokens", "n_seqs", "n_rows", "token_ids", "positions", "seq_of_token", "logit_rows",
                 "q_start", "kv_len", "state_slots", "block_tables", "max_q_len", "max_kv_len", "decode_only",
                 "q_lens", "starts", "rids", "fresh", "tile_tok0", "tile_rows")


class BatchBuffers:
    """Persistent device arrays of a batch at fixed addresses, with pinned staging.

    Layout in int32 words, by capacity (so a view's address does not depend on the
    batch): tokens | positions | seq_of_token | logit_rows | attention tiles (first
    token, rows) | q_start | kv_len | slots | one block table [max_seqs, max_pages]
    per cache group.  An attention tile is a run of up to 16 consecutive tokens of
    one sequence.
    """

    def __init__(self, max_tokens: int, max_seqs: int, max_pages: int, n_groups: int, device):
        self.max_tokens, self.max_seqs, self.max_pages, self.n_groups = max_tokens, max_seqs, max_pages, n_groups
        o = 0
        self.off = {}
        for name, n in (("tok", max_tokens), ("pos", max_tokens), ("seq", max_tokens), ("rows", max_tokens),
                        ("tile0", max_tokens), ("tilen", max_tokens),
                        ("q_start", max_seqs + 1), ("kv_len", max_seqs), ("slots", max_seqs)):
            self.off[name] = o
            o += n
        self.small_words = o
        self.bt_off = []
        for _ in range(n_groups):
            self.bt_off.append(o)
            o += max_seqs * max_pages
        self.words = o
        self.dev = torch.zeros(o, dtype=torch.int32, device=device)
        self.host = [torch.zeros(o, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.host_np = [h.numpy() for h in self.host]
        self.events = [None, None]
        self.turn = 0

    def staging(self):
        """The next staging buffer, once the copy that last used it has finished."""
        i = self.turn
        self.turn ^= 1
        if self.events[i] is not None:
            self.events[i].synchronize()
        return i, self.host_np[i]

    def upload(self, i: int, n_seqs: int) -> None:
        # Small arrays in one copy, then the used rows of each block table.
        self.dev[:self.small_words].copy_(self.host[i][:self.small_words], non_blocking=True)
        for off in self.bt_off:
            n = n_seqs * self.max_pages
            self.dev[off:off + n].copy_(self.host[i][off:off + n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class Stepper:
    """Owns the batch buffers and runs steps of a model against a cache manager."""

    def __init__(self, model: DecoderModel, cache: CacheManager, rt: Runtime, max_tokens: int, max_seqs: int,
                 max_seq_len: int, use_cuda_graphs: bool = False):
        self.model, self.cache, self.rt = model, cache, rt
        self.use_cuda_graphs = use_cuda_graphs
        self._graphs = {}        # batch size -> (graph, static logits)
        self._graph_uses = {}    # batch size -> eager runs so far
        self.max_tokens, self.max_seqs, self.max_seq_len = max_tokens, max_seqs, max_seq_len
        self.max_pages = (max_seq_len + cache.page_size - 1) // cache.page_size
        self.buffers = BatchBuffers(max_tokens, max_seqs, self.max_pages, len(cache.paged), rt.device)
        if rt.status is None:
            rt.status = K.new_status(rt.device)
        model.attach_cache(cache)

    # ------------------------------------------------------------------ checks
    def validate(self, entries: Sequence[StepEntry]) -> None:
        """Host-side checks of a batch before anything is reserved or launched."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        if len(entries) > self.max_seqs:
            raise ValueError(f"{len(entries)} requests in one step; the engine was made for {self.max_seqs}")
        total = 0
        seen = set()
        V = self.model.vocab_size
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.rid!r}: an entry needs at least one token")
            total += n
            for t in e.tokens:
                if not 0 <= int(t) < V:
                    raise ValueError(f"request {e.rid!r}: token id {t} outside the vocabulary of {V}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ValueError(f"request {e.rid!r}: wanted row {w} outside its {n} tokens")
            cur = self.cache.length(e.rid) if self.cache.has(e.rid) else 0
            if cur + n > self.max_seq_len:
                raise ValueError(f"request {e.rid!r}: {cur + n} tokens exceed the maximum sequence length "
                                 f"{self.max_seq_len}")
        if total > self.max_tokens:
            raise ValueError(f"{total} tokens in one step; the engine was made for {self.max_tokens}")

    def pages_short(self, entries: Sequence[StepEntry]) -> int:
        """How many pages the scarcest group lacks for this batch (0 = it fits)."""
        short = 0
        for g in self.cache.paged:
            need = 0
            for e in entries:
                if self.cache.has(e.rid):
                    cur = self.cache.length(e.rid)
                    need += g.pages_needed(g.tables[e.rid], cur, cur + len(e.tokens))
                else:
                    need += g.pages_needed([], 0, len(e.tokens))
            short = max(short, need - g.pool.n_free)
        return short

    # -------------------------------------------------------------------- step
    def prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Reserve cache, fill and upload the batch arrays; returns the device views."""
        self.validate(entries)
        if self.pages_short(entries) > 0:
            raise OutOfPages(f"the batch needs {self.pages_short(entries)} more pages than are free")
        cache = self.cache
        new_slots = sum(1 for e in entries if not cache.has(e.rid))
        if new_slots > cache.slots.n_free:
            raise OutOfPages(f"{new_slots} new requests but only {cache.slots.n_free} free state slots")
        buf = self.buffers
        i, host = buf.staging()
        off = buf.off
        ctx = StepContext()
        t = 0
        rows: List[int] = []
        tiles0: List[int] = []
        tilesn: List[int] = []
        q_lens, starts, rids, fresh = [], [], [], []
        max_kv = 0
        for s, e in enumerate(entries):
            if not cache.has(e.rid):
                slot = cache.add_request(e.rid)
                cache.zero_state(slot)
            start = cache.length(e.rid)
            n = len(e.tokens)
            cache.reserve(e.rid, start + n)
            host[off["tok"] + t: off["tok"] + t + n] = np.asarray(e.tokens, dtype=np.int32)
            host[off["pos"] + t: off["pos"] + t + n] = np.arange(start, start + n, dtype=np.int32)
            host[off["seq"] + t: off["seq"] + t + n] = s
            host[off["q_start"] + s] = t
            host[off["kv_len"] + s] = start + n
            host[off["slots"] + s] = cache.slot_of(e.rid)
            for g, bo in enumerate(buf.bt_off):
                table = cache.block_table(g, e.rid)
                row = host[bo + s * buf.max_pages: bo + (s + 1) * buf.max_pages]
                row[:len(table)] = table
                row[len(table):] = -1
            rows.extend(t + int(w) for w in e.want)
            for a in range(0, n, ATTENTION_TILE):
                tiles0.append(t + a)
                tilesn.append(min(ATTENTION_TILE, n - a))
            q_lens.append(n)
            starts.append(start)
            rids.append(e.rid)
            fresh.append(start == 0)
            max_kv = max(max_kv, start + n)
            t += n
        B = len(entries)
        host[off["q_start"] + B] = t
        R = len(rows)
        host[off["rows"]: off["rows"] + R] = np.asarray(rows, dtype=np.int32) if R else 0
        n_tiles = len(tiles0)
        host[off["tile0"]: off["tile0"] + n_tiles] = np.asarray(tiles0, dtype=np.int32)
        host[off["tilen"]: off["tilen"] + n_tiles] = np.asarray(tilesn, dtype=np.int32)
        buf.upload(i, B)

        d = buf.dev
        ctx.n_tokens, ctx.n_seqs, ctx.n_rows = t, B, R
        ctx.token_ids = d[off["tok"]: off["tok"] + t]
        ctx.positions = d[off["pos"]: off["pos"] + t]
        ctx.seq_of_token = d[off["seq"]: off["seq"] + t]
        ctx.logit_rows = d[off["rows"]: off["rows"] + R]
        ctx.tile_tok0 = d[off["tile0"]: off["tile0"] + n_tiles]
        ctx.tile_rows = d[off["tilen"]: off["tilen"] + n_tiles]
        ctx.q_start = d[off["q_start"]: off["q_start"] + B + 1]
        ctx.kv_len = d[off["kv_len"]: off["kv_len"] + B]
        ctx.state_slots = d[off["slots"]: off["slots"] + B]
        ctx.block_tables = [d[bo: bo + B * buf.max_pages].view(B, buf.max_pages) for bo in buf.bt_off]
        ctx.max_q_len, ctx.max_kv_len = max(q_lens), max_kv
        ctx.decode_only = all(n == 1 for n in q_lens)
        ctx.q_lens, ctx.starts, ctx.rids, ctx.fresh = q_lens, starts, rids, fresh
        return ctx

    def commit(self, ctx: StepContext) -> None:
        """Record the new lengths; pages behind a window return to their pool."""
        for rid, start, n in zip(ctx.rids, ctx.starts, ctx.q_lens):
            self.cache.commit(rid, start + n)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch.  Returns float32 logits [wanted rows, vocab] on the device, in the
        order of the entries and of each entry's `want`."""
        ctx = self.prepare(entries)
        if self.use_cuda_graphs and ctx.decode_only and ctx.n_rows == ctx.n_seqs:
            logits = self._forward_decode_graph(ctx)
        else:
            logits = self.model.forward(ctx)
        self.commit(ctx)
        return logits

    def _forward_decode_graph(self, ctx: StepContext) -> torch.Tensor:
        """Decode-only batches of a given size replay one captured CUDA graph.

        The batch arrays live at fixed addresses, so a graph captured for B sequences serves
        every later step of B sequences; only the arrays' contents change.  The first step of a
        size runs eagerly (it also warms the library GEMM up), the second is captured.
        The returned logits are the graph's own buffer: read them before the next step.
        """
        B = ctx.n_seqs
        hit = self._graphs.get(B)
        if hit is None:
            uses = self._graph_uses.get(B, 0)
            self._graph_uses[B] = uses + 1
            if uses == 0:
                return self.model.forward(ctx)
            graph = torch.cuda.CUDAGraph()
            torch.cuda.current_stream().synchronize()
            with torch.cuda.graph(graph):
                static_logits = self.model.forward(ctx)
            hit = self._graphs[B] = (graph, static_logits)
        hit[0].replay()
        return hit[1]

    def finish(self, rid: Hashable) -> None:
        """The request is over: its pages and its slot go back."""
        self.cache.release(rid)

    def check_device_status(self, what: str = "step") -> None:
        K.check_status(self.rt.status, what)
