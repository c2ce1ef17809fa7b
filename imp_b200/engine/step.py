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


ATTENTION_TILE = 32   # query tokens per attention tile (two 16-row tensor-core tiles share staged keys)
ATTENTION_WIDE_TILE = 128   # query tokens per tile of the tensor-memory prefill kernel
ATTENTION_WIDE_MIN = 64     # portions at least this long are cut into wide tiles as well


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
                 "q_lens", "starts", "rids", "fresh", "slots", "tile_tok0", "tile_rows",
                 "wide_tile_tok0", "wide_tile_rows", "rest_tile_tok0", "rest_tile_rows")


class BatchBuffers:
    """Persistent device arrays of a batch at fixed addresses, with pinned staging.

    Layout in int32 words, by capacity (so a view's address does not depend on the
    batch): tokens | positions | seq_of_token | logit_rows | attention tiles (first
    token, rows) | q_start | kv_len | slots | one block table [max_seqs, max_pages]
    per cache group.  An attention tile is a run of up to 32 consecutive tokens of
    one sequence.
    """

    def __init__(self, max_tokens: int, max_seqs: int, max_pages: int, n_groups: int, device):
        self.max_tokens, self.max_seqs, self.max_pages, self.n_groups = max_tokens, max_seqs, max_pages, n_groups
        o = 0
        self.off = {}
        for name, n in (("tok", max_tokens), ("pos", max_tokens), ("seq", max_tokens), ("rows", max_tokens),
                        ("tile0", max_tokens), ("tilen", max_tokens), ("wtile0", max_tokens), ("wtilen", max_tokens),
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

    # -------------------------------------------------------------------- step
    def pages_short(self, entries: Sequence[StepEntry]) -> int:
        """How many pages the scarcest group lacks for this batch (0 = it fits)."""
        cache = self.cache
        short = 0
        for g in cache.paged:
            need = 0
            for e in entries:
                if cache.has(e.rid):
                    cur = cache.length(e.rid)
                    need += g.pages_needed_n(int(g.n_entries[cache.slot_of(e.rid)]), cur, cur + len(e.tokens))
                else:
                    need += g.pages_needed_n(0, 0, len(e.tokens))
            short = max(short, need - g.pool.n_free)
        return short

    def prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Check the batch on the host, reserve cache, fill and upload the batch arrays."""
        cache, buf = self.cache, self.buffers
        B = len(entries)
        if B == 0:
            raise ValueError("a step needs at least one entry")
        if B > self.max_seqs:
            raise ValueError(f"{B} requests in one step; the engine was made for {self.max_seqs}")
        rids = [e.rid for e in entries]
        if len(set(rids)) != B:
            raise ValueError("a request appears twice in one step")
        q_lens = [len(e.tokens) for e in entries]
        if min(q_lens) == 0:
            raise ValueError("an entry needs at least one token")
        T = sum(q_lens)
        if T > self.max_tokens:
            raise ValueError(f"{T} tokens in one step; the engine was made for {self.max_tokens}")
        flat = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=T)
        V = self.model.vocab_size
        if flat.min() < 0 or flat.max() >= V:
            bad = int(flat[(flat < 0) | (flat >= V)][0])
            raise ValueError(f"token id {bad} outside the vocabulary of {V}")
        starts = [cache.length(r) if cache.has(r) else 0 for r in rids]
        for e, st, n in zip(entries, starts, q_lens):
            if st + n > self.max_seq_len:
                raise ValueError(f"request {e.rid!r}: {st + n} tokens exceed the maximum sequence length "
                                 f"{self.max_seq_len}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ValueError(f"request {e.rid!r}: wanted row {w} outside its {n} tokens")
        short = self.pages_short(entries)
        if short > 0:
            raise OutOfPages(f"the batch needs {short} more pages than are free")
        new_slots = sum(1 for r in rids if not cache.has(r))
        if new_slots > cache.slots.n_free:
            raise OutOfPages(f"{new_slots} new requests but only {cache.slots.n_free} free state slots")

        for r, st, n in zip(rids, starts, q_lens):
            if not cache.has(r):
                cache.zero_state(cache.add_request(r))
            cache.reserve(r, st + n)
        slots = np.fromiter((cache.slot_of(r) for r in rids), dtype=np.int64, count=B)

        i, host = buf.staging()
        off = buf.off
        ql = np.asarray(q_lens, dtype=np.int64)
        st_np = np.asarray(starts, dtype=np.int64)
        q_start = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(ql, out=q_start[1:])
        decode_only = T == B
        host[off["tok"]: off["tok"] + T] = flat
        if decode_only:
            host[off["pos"]: off["pos"] + T] = st_np
            host[off["seq"]: off["seq"] + T] = np.arange(B)
        else:
            host[off["pos"]: off["pos"] + T] = np.arange(T) + np.repeat(st_np - q_start[:-1], ql)
            host[off["seq"]: off["seq"] + T] = np.repeat(np.arange(B), ql)
        host[off["q_start"]: off["q_start"] + B + 1] = q_start
        host[off["kv_len"]: off["kv_len"] + B] = st_np + ql
        host[off["slots"]: off["slots"] + B] = slots
        for g, bo in zip(cache.paged, buf.bt_off):
            view = host[bo: bo + B * buf.max_pages].reshape(B, buf.max_pages)
            width = min(g.table_np.shape[1], buf.max_pages)
            view[:, :width] = g.table_np[slots, :width]
            view[:, width:] = -1
        rows = [int(q_start[s]) + int(w) for s, e in enumerate(entries) for w in e.want]
        R = len(rows)
        if R:
            host[off["rows"]: off["rows"] + R] = rows
        n_tiles = n_wide = n_rest = 0
        if not decode_only:
            # Every portion in tiles of ATTENTION_TILE tokens; and, for kernels with wide tiles, the same
            # tokens again as wide tiles of the long portions followed by narrow tiles of the short ones.
            tiles0, tilesn, wide0, widen, rest0, restn = [], [], [], [], [], []
            for s, n in enumerate(q_lens):
                t0 = int(q_start[s])
                for a in range(0, n, ATTENTION_TILE):
                    tiles0.append(t0 + a)
                    tilesn.append(min(ATTENTION_TILE, n - a))
                if n >= ATTENTION_WIDE_MIN:
                    for a in range(0, n, ATTENTION_WIDE_TILE):
                        wide0.append(t0 + a)
                        widen.append(min(ATTENTION_WIDE_TILE, n - a))
                else:
                    k = (n + ATTENTION_TILE - 1) // ATTENTION_TILE
                    rest0.extend(tiles0[-k:])
                    restn.extend(tilesn[-k:])
            n_tiles, n_wide, n_rest = len(tiles0), len(wide0), len(rest0)
            host[off["tile0"]: off["tile0"] + n_tiles] = tiles0
            host[off["tilen"]: off["tilen"] + n_tiles] = tilesn
            host[off["wtile0"]: off["wtile0"] + n_wide + n_rest] = wide0 + rest0
            host[off["wtilen"]: off["wtilen"] + n_wide + n_rest] = widen + restn
        buf.upload(i, B)

        d = buf.dev
        ctx = StepContext()
        ctx.n_tokens, ctx.n_seqs, ctx.n_rows = T, B, R
        ctx.token_ids = d[off["tok"]: off["tok"] + T]
        ctx.positions = d[off["pos"]: off["pos"] + T]
        ctx.seq_of_token = d[off["seq"]: off["seq"] + T]
        ctx.logit_rows = d[off["rows"]: off["rows"] + R]
        ctx.tile_tok0 = d[off["tile0"]: off["tile0"] + n_tiles]
        ctx.tile_rows = d[off["tilen"]: off["tilen"] + n_tiles]
        ctx.wide_tile_tok0 = d[off["wtile0"]: off["wtile0"] + n_wide]
        ctx.wide_tile_rows = d[off["wtilen"]: off["wtilen"] + n_wide]
        ctx.rest_tile_tok0 = d[off["wtile0"] + n_wide: off["wtile0"] + n_wide + n_rest]
        ctx.rest_tile_rows = d[off["wtilen"] + n_wide: off["wtilen"] + n_wide + n_rest]
        ctx.q_start = d[off["q_start"]: off["q_start"] + B + 1]
        ctx.kv_len = d[off["kv_len"]: off["kv_len"] + B]
        ctx.state_slots = d[off["slots"]: off["slots"] + B]
        ctx.block_tables = [d[bo: bo + B * buf.max_pages].view(B, buf.max_pages) for bo in buf.bt_off]
        ctx.max_q_len, ctx.max_kv_len = max(q_lens), int((st_np + ql).max())
        ctx.decode_only = decode_only
        ctx.q_lens, ctx.starts, ctx.rids = q_lens, starts, rids
        ctx.fresh = [st == 0 for st in starts]
        ctx.slots = [int(x) for x in slots]
        return ctx

    def commit(self, ctx: StepContext) -> None:
        """Record the new lengths; pages behind a window return to their pool."""
        for rid, start, n in zip(ctx.rids, ctx.starts, ctx.q_lens):
            self.cache.commit(rid, start + n)

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run one batch.  Returns float32 logits [wanted rows, vocab] on the device, in the
        order of the entries and of each entry's `want`.

        `device_tokens` (int32, one per token of the batch, on the device) replaces the entries'
        token ids: the ids of a step whose tokens were sampled on the device and have not come
        back to the host yet.  The entries then carry placeholders."""
        ctx = self.prepare(entries)
        if device_tokens is not None:
            if device_tokens.numel() != ctx.n_tokens or device_tokens.dtype != torch.int32:
                raise ValueError("device_tokens must hold one int32 id per token of the batch")
            ctx.token_ids.copy_(device_tokens)
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
