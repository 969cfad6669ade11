"""The step function: one batch of (request, its next tokens) through the model.

The reference builds two groups per step, prompt portions and single decoded tokens,
and runs the whole model once for each (pulsar-core/src/model/paged_forward.cpp:96-105;
pulsar-core/src/runtime/engine.cpp:573-702 builds the groups, with several small
host-device copies each).  Here a step is one ragged batch: a decoded token is a
portion of length one, the projections see all tokens at once, the index arrays of the
step travel in one pinned buffer and one copy, and logits come back only for the
positions that were asked for.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager, OutOfPages
from ..parts.base import CacheView, HostBatch, StepContext


@dataclass
class StepEntry:
    """The next ``tokens`` of request ``rid``; ``want`` lists the indices among these
    tokens whose logits are returned (in this order).  ``token_src`` (for an entry of one
    token) says that the token is not known on the host yet: it is element ``token_src`` of
    the device tensor of sampled ids that the step is given, and ``tokens`` holds a stand-in."""
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    token_src: Optional[int] = None


class StepError(ValueError):
    pass


def _align(n: int, to: int = 4) -> int:
    return (n + to - 1) // to * to


class ModelRunner:
    """Owns the scratch memory and the per-step index arrays; drives the model over the cache."""

    N_STAGING = 4
    TABLE_BUCKET = 64          # block-table width of decode steps is rounded up to this many pages

    def __init__(self, model, cache: CacheManager, device, cuda_graphs: bool = True):
        self.model, self.cache = model, cache
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError(f"the engine runs on a CUDA device only (asked for '{device}'); there is no CPU path")
        self.dtype = model.dtype
        self.vocab = model.spec.vocab_size
        self._scratch: Dict[str, torch.Tensor] = {}
        self.scratch_epoch = 0
        self._staging: List[Optional[torch.Tensor]] = [None] * self.N_STAGING
        self._staging_events: List[Optional[torch.cuda.Event]] = [None] * self.N_STAGING
        self._staging_next = 0
        self._index_buf: Optional[torch.Tensor] = None
        self._views: Dict[tuple, list] = {}
        self.steps_run = 0
        # Decode steps (one token per request) are launch-bound: their kernel sequence is
        # captured once per (batch size, block-table width) and replayed.
        self.cuda_graphs = bool(cuda_graphs)
        self._graphs: Dict[tuple, Tuple[torch.cuda.CUDAGraph, torch.Tensor, int]] = {}
        self._graph_seen: Dict[tuple, int] = {}
        self._graph_epoch = -1
        self.graph_replays = 0
        self._capturing = False
        self.h2d_bytes = 0          # bytes of index arrays copied to the device so far

    # ------------------------------------------------------------------ memory
    def scratch(self, tag: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= s
        key = f"{tag}|{dtype}"
        buf = self._scratch.get(key)
        if buf is None or buf.numel() < numel:
            if self._capturing:
                raise RuntimeError(f"scratch '{tag}' would be allocated during graph capture")
            grow = max(numel, 1) if buf is None else max(numel, 2 * buf.numel())
            buf = torch.empty(grow, dtype=dtype, device=self.device)
            self._scratch[key] = buf
            self.scratch_epoch += 1
        return buf[:numel].view(shape)

    def cache_view(self, ctx: StepContext, entry: int) -> CacheView:
        need = self.cache.needs[entry]
        if need.kind == "paged_kv":
            g = self.cache.group_of_entry[entry]
            k, v = self.cache.kv_pools(entry)
            return CacheView("paged_kv", k, v, ctx.group_tables[g], ctx.group_slots[g], self.cache.page_size, group=g)
        if need.kind == "state":
            return CacheView("state", state=self.cache.state[entry], page_size=self.cache.page_size)
        return CacheView("none", page_size=self.cache.page_size)

    def _stage(self, n_ints: int) -> torch.Tensor:
        i = self._staging_next
        self._staging_next = (i + 1) % self.N_STAGING
        if self._staging_events[i] is not None:
            self._staging_events[i].synchronize()
        buf = self._staging[i]
        if buf is None or buf.numel() < n_ints:
            buf = torch.empty(max(n_ints, 4096), dtype=torch.int32, pin_memory=True)
            self._staging[i] = buf
        self._staging_slot = i
        return buf

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: Sequence[StepEntry], sampled_ids: Optional[torch.Tensor] = None) -> StepContext:
        """Grow the requests in the cache, build the step's index arrays and copy them
        to the device.  Raises OutOfPages before changing anything if the pages do not
        suffice for the whole batch.  ``sampled_ids``: the device tensor that entries with
        ``token_src`` take their token from."""
        cache = self.cache
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            n_tok = len(e.tokens)
            if n_tok == 0:
                raise StepError(f"request {e.rid!r}: a step entry needs at least one token")
            if min(e.tokens) < 0 or max(e.tokens) >= self.vocab:
                bad = [t for t in e.tokens if not (0 <= int(t) < self.vocab)][0]
                raise StepError(f"request {e.rid!r}: token id {bad} outside the vocabulary [0, {self.vocab})")
            if e.token_src is not None and (n_tok != 1 or sampled_ids is None or not (0 <= e.token_src < sampled_ids.numel())):
                raise StepError(f"request {e.rid!r}: a token taken from the device needs an entry of one token and "
                                f"a tensor of sampled ids that has element {e.token_src}")
            if len(e.want) and (min(e.want) < 0 or max(e.want) >= n_tok):
                bad = [w for w in e.want if not (0 <= int(w) < n_tok)][0]
                raise StepError(f"request {e.rid!r}: wanted index {bad} outside its {n_tok} tokens")
        # Page check for the whole batch before any change.
        fresh = [e for e in entries if not cache.has(e.rid)]
        if len(fresh) > cache.n_free_slots():
            raise OutOfPages(f"{len(fresh)} new requests but {cache.n_free_slots()} free state slots")
        n_groups = len(cache.groups)
        need = [0] * n_groups
        for e in entries:
            if cache.has(e.rid):
                cache.release_passed(e.rid)      # pages a window has passed serve this very step
                want_pages = cache.pages_to_append(e.rid, len(e.tokens))
            else:
                want_pages = [-(-len(e.tokens) // cache.page_size)] * n_groups
            for g in range(n_groups):
                need[g] += want_pages[g]
        free = cache.n_free_pages()
        if any(need[g] > free[g] for g in range(n_groups)):
            raise OutOfPages(f"step needs {need} new pages per group, {free} are free")

        q_lens, kv_lens, starts, state_slots = [], [], [], []
        for e in entries:
            if not cache.has(e.rid):
                cache.open(e.rid)
            starts.append(cache.append(e.rid, len(e.tokens)))
            q_lens.append(len(e.tokens))
            kv_lens.append(starts[-1] + len(e.tokens))
            state_slots.append(cache.state_slot(e.rid))
        host = HostBatch(q_lens, kv_lens, state_slots)
        n, s = sum(q_lens), len(entries)
        ctx = StepContext(self, n, s, host)

        # Lengths of the step's index arrays, each padded to 16 bytes, in one pinned buffer:
        # token_ids, positions, seq_of_token [N]; cu_q [S+1]; kv_len, state_slots [S]; logit_rows [R];
        # per group slots [N] and the block table [S, width].
        widths = []
        for g in range(n_groups):
            w = max(1, max(len(cache.table(e.rid, g)) for e in entries))
            if ctx.all_decode:      # few distinct widths, so that captured steps are reused as contexts grow
                w = -(-w // self.TABLE_BUCKET) * self.TABLE_BUCKET
            widths.append(w)
        ctx.table_widths = tuple(widths)
        n_rows = sum(len(e.want) for e in entries)
        lengths = [n, n, n, s + 1, s, s, n_rows]
        for g in range(n_groups):
            lengths += [n, s * widths[g]]
        moved = [(i, e.token_src) for i, e in enumerate(entries) if e.token_src is not None]
        if moved:                 # last, so that the other arrays lie where they lie without them
            lengths += [len(moved), len(moved)]
        offsets, total = [], 0
        for ln in lengths:
            offsets.append(total)
            total += _align(max(ln, 1))
        stage = self._stage(total)
        buf = stage.numpy()
        o_tok, o_pos, o_seq, o_cu, o_kv, o_slot, o_rows = offsets[:7]
        at, row_at = 0, 0
        buf[o_cu] = 0
        for i, e in enumerate(entries):
            q = q_lens[i]
            buf[o_tok + at:o_tok + at + q] = e.tokens
            if q == 1:
                buf[o_pos + at] = starts[i]
            else:
                buf[o_pos + at:o_pos + at + q] = np.arange(starts[i], starts[i] + q, dtype=np.int32)
            buf[o_seq + at:o_seq + at + q] = i
            for w in e.want:
                buf[o_rows + row_at] = at + int(w)
                row_at += 1
            at += q
            buf[o_cu + i + 1] = at
        buf[o_kv:o_kv + s] = kv_lens
        buf[o_slot:o_slot + s] = state_slots
        if moved:
            o_dst, o_src = offsets[-2], offsets[-1]
            for k, (i, src) in enumerate(moved):
                buf[o_dst + k] = buf[o_cu + i]          # the entry's one token sits at its cu_q
                buf[o_src + k] = src
        ps = cache.page_size
        for g in range(n_groups):
            o_s, o_t = offsets[7 + 2 * g], offsets[8 + 2 * g]
            w = widths[g]
            buf[o_t:o_t + s * w] = -1
            at = 0
            for i, e in enumerate(entries):
                row = cache.table(e.rid, g)
                q = q_lens[i]
                if q == 1:
                    p = starts[i]
                    page = row[p // ps]
                    if page < 0:
                        raise StepError(f"request {e.rid!r}: position {p} lies in a released page")
                    buf[o_s + at] = page * ps + p % ps
                else:
                    buf[o_s + at:o_s + at + q] = cache.slots(e.rid, g, starts[i], q)
                buf[o_t + i * w:o_t + i * w + len(row)] = row
                at += q
        if self._index_buf is None or self._index_buf.numel() < total:
            self._index_buf = torch.empty(max(total, 4096) * 2, dtype=torch.int32, device=self.device)
            self.scratch_epoch += 1
            self._views.clear()
        dev = self._index_buf
        dev[:total].copy_(stage[:total], non_blocking=True)
        self.h2d_bytes += total * 4
        ev = self._staging_events[self._staging_slot]
        if ev is None:
            ev = self._staging_events[self._staging_slot] = torch.cuda.Event()
        ev.record()

        # Views of the device buffer; steady decoding has the same layout every step, so they are kept.
        key = (tuple(lengths), tuple(widths))
        views = self._views.get(key)
        if views is None:
            if len(self._views) > 64:
                self._views.clear()
            views = [dev[o:o + ln] for o, ln in zip(offsets, lengths)]
            for g in range(n_groups):
                views[8 + 2 * g] = views[8 + 2 * g].view(s, widths[g])
            self._views[key] = views
        (ctx.token_ids, ctx.positions, ctx.seq_of_token, ctx.cu_q, ctx.kv_len, ctx.state_slots, ctx.logit_rows) = views[:7]
        for g in range(n_groups):
            ctx.group_slots.append(views[7 + 2 * g])
            ctx.group_tables.append(views[8 + 2 * g])
        if moved:
            ops.move_ids(ctx.token_ids, views[-2], views[-1], sampled_ids)
        return ctx

    def step(self, entries: Sequence[StepEntry], sampled_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run the given tokens as one batch from the cache that earlier steps left and
        return float32 logits ``[wanted, vocab]`` in the order of the entries and of their
        ``want`` lists.  The tensor is scratch memory: it is valid until the next step."""
        ctx = self.prepare(entries, sampled_ids)
        with torch.cuda.device(self.device):
            logits = self._forward(ctx)
        self.steps_run += 1
        return logits

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        if not (self.cuda_graphs and ctx.all_decode):
            return self.model.forward(ctx)
        if self._graph_epoch != self.scratch_epoch:       # a buffer moved: every captured address is stale
            self._graphs.clear()
            self._graph_seen.clear()
            self._graph_epoch = self.scratch_epoch
        key = (ctx.n_tokens, ctx.n_seqs, int(ctx.logit_rows.numel()), ctx.table_widths,
               tuple(int(t.data_ptr()) for t in (ctx.token_ids, ctx.logit_rows)))
        hit = self._graphs.get(key)
        if hit is not None:
            hit[0].replay()
            self.graph_replays += 1
            ops.LAUNCHES += hit[2]
            return hit[1]
        seen = self._graph_seen.get(key, 0)
        self._graph_seen[key] = seen + 1
        if seen < 2:                                      # run eagerly first: buffers reach their final size
            return self.model.forward(ctx)
        epoch = self.scratch_epoch
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize(self.device)
        launches = ops.LAUNCHES
        self._capturing = True
        try:
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx)
        finally:
            self._capturing = False
        launches = ops.LAUNCHES - launches            # kernels of this library inside the captured step
        if self.scratch_epoch != epoch:                   # grew during capture: do not keep it
            self._graph_epoch = -1
            return self.model.forward(ctx)
        self._graphs[key] = (graph, logits, launches)
        graph.replay()
        self.graph_replays += 1
        return logits

    def finish(self, rid: Hashable) -> None:
        """The request is over: everything it holds goes back to the pools."""
        self.cache.close(rid)
