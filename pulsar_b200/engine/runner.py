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

import ctypes
import gc
import os

import torch

from .. import host, ops, profiling
from ..cache.manager import CacheManager, OutOfPages
from ..parts.base import CacheView, HostBatch, StepContext


@dataclass
class StepEntry:
    """The next ``tokens`` of request ``rid``; ``want`` lists the indices among these
    tokens whose logits are returned (in this order).  ``token_src`` (for an entry of one
    token) says that the token is not known on the host yet: it is element ``token_src`` of
    the device tensor of sampled ids that the step is given, and ``tokens`` holds a stand-in.
    ``positions`` (only for a model whose positions have more than one axis): one list per further
    axis, each as long as ``tokens``; axis 0 is always the token's index in its sequence, and an axis
    that is not given repeats it."""
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    token_src: Optional[int] = None
    positions: Optional[Sequence[Sequence[int]]] = None


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
        self.position_axes = int(getattr(model.spec, "position_axes", 1))
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
        self.cuda_graphs = bool(cuda_graphs) and bool(getattr(model, "graph_safe", True)) and not profiling.ENABLED
        self._graphs: Dict[tuple, Tuple[torch.cuda.CUDAGraph, torch.Tensor, int]] = {}
        self._graph_seen: Dict[tuple, int] = {}
        self._graph_epoch = -1
        self.graph_replays = 0
        self._capturing = False
        self.h2d_bytes = 0          # bytes of index arrays copied to the device so far
        # The block tables stay on the device, one row per state slot; a step brings only the page ids its requests
        # gained (a few hundred bytes for a decode step instead of the whole [sequences, width] table).
        # PULSAR_RESIDENT_TABLES=0: every step brings whole tables.
        self.resident_tables = os.environ.get("PULSAR_RESIDENT_TABLES", "1") != "0"
        cache.set_resident_tables(self.resident_tables)

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
            return CacheView("paged_kv", self.cache.pools(entry), ctx.group_tables[g], ctx.group_slots[g],
                             self.cache.page_size, group=g)
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
            if e.positions is not None and (len(e.positions) != self.position_axes - 1
                                            or any(len(axis) != n_tok for axis in e.positions)):
                raise StepError(f"request {e.rid!r}: positions must give {self.position_axes - 1} further axes of "
                                f"{n_tok} values each (the model's positions have {self.position_axes} axes)")
            if len(e.want) and (min(e.want) < 0 or max(e.want) >= n_tok):
                bad = [w for w in e.want if not (0 <= int(w) < n_tok)][0]
                raise StepError(f"request {e.rid!r}: wanted index {bad} outside its {n_tok} tokens")
        # The host runtime checks the whole step's pages and slots before anything changes, grows the
        # requests, and writes the step's index arrays into one pinned buffer:
        # token_ids, positions, seq_of_token [N]; cu_q [S+1]; kv_len, state_slots [S]; logit_rows [R];
        # per group slots [N] and the block table [S, width]; move_dst, move_src if tokens come from the device.
        s = len(entries)
        n_groups = len(cache.groups)
        fresh = [e.rid for e in entries if not cache.has(e.rid)]
        rids = host.longs([cache.native_id(e.rid, create=True) for e in entries])
        q_lens = [len(e.tokens) for e in entries]
        n = sum(q_lens)
        flat_tokens = [int(t) for e in entries for t in e.tokens]
        flat_wants = [int(w) for e in entries for w in e.want]
        n_tok, want_n = host.ints(q_lens), host.ints([len(e.want) for e in entries])
        tokens, wants = host.ints(flat_tokens), host.ints(flat_wants or [0])
        token_src = host.ints([-1 if e.token_src is None else int(e.token_src) for e in entries])
        starts, slots = (ctypes.c_int * s)(), (ctypes.c_int * s)()
        widths_c, bad = (ctypes.c_int * max(1, n_groups))(), ctypes.c_int(-1)
        lib, handle = cache._lib, cache._h
        total = lib.ph_step_plan(handle, s, rids, n_tok, tokens, want_n, wants, token_src,
                                 0 if sampled_ids is None else int(sampled_ids.numel()), self.vocab, self.TABLE_BUCKET,
                                 starts, slots, widths_c, ctypes.byref(bad))
        if total < 0:
            for rid in fresh:
                cache._forget_if_idle(rid)
            if total == host.OUT_OF_SLOTS:
                raise OutOfPages(f"{len(fresh)} new requests but {cache.n_free_slots()} free state slots")
            if total == host.OUT_OF_PAGES:
                raise OutOfPages(f"the step's {n} tokens need more pages than the {cache.n_free_pages()} free ones")
            who = entries[bad.value].rid if 0 <= bad.value < s else None
            if total == host.RELEASED_PAGE:
                raise StepError(f"request {who!r}: a position of the step lies in a released page")
            raise StepError(f"the host runtime refused the step (code {total}, entry of request {who!r})")
        for rid in fresh:
            cache.opened_by_runtime(rid)
        starts, state_slots = list(starts), list(slots)
        kv_lens = [st + q for st, q in zip(starts, q_lens)]
        host_batch = HostBatch(q_lens, kv_lens, state_slots)
        ctx = StepContext(self, n, s, host_batch)
        widths = list(widths_c[:n_groups])
        ctx.table_widths = tuple(widths)
        moved = any(e.token_src is not None for e in entries)
        n_arrays = 7 + 2 * n_groups + (2 if moved else 0)
        offsets_c, lengths_c = (ctypes.c_int * n_arrays)(), (ctypes.c_int * n_arrays)()
        stage = self._stage(total)
        rc = lib.ph_step_pack(handle, s, rids, n_tok, tokens, want_n, wants, token_src, (ctypes.c_int * s)(*starts),
                              (ctypes.c_int * s)(*state_slots), widths_c, stage.data_ptr(), stage.numel(), offsets_c, lengths_c)
        if rc == host.RELEASED_PAGE:
            raise StepError("a position of the step lies in a released page")
        if rc != total:
            raise StepError(f"the host runtime packed {rc} words where {total} were planned")
        offsets, lengths = list(offsets_c), list(lengths_c)
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
            if not self.resident_tables:
                for g in range(n_groups):
                    views[8 + 2 * g] = views[8 + 2 * g].view(s, widths[g])
            self._views[key] = views
        (ctx.token_ids, ctx.positions, ctx.seq_of_token, ctx.cu_q, ctx.kv_len, ctx.state_slots, ctx.logit_rows) = views[:7]
        for g in range(n_groups):
            ctx.group_slots.append(views[7 + 2 * g])
            if self.resident_tables:
                resident, fresh = cache.resident_table(g, widths[g])
                if fresh:
                    self.scratch_epoch += 1
                table = self.scratch(f"table.{g}", (s, widths[g]), torch.int32)
                ops.table_update(resident, views[8 + 2 * g], ctx.state_slots, table)
                ctx.group_tables.append(table)
            else:
                ctx.group_tables.append(views[8 + 2 * g])
        if moved:
            ops.move_ids(ctx.token_ids, views[-2], views[-1], sampled_ids)
        if self.position_axes > 1:
            # Further axes of the positions travel in a copy of their own (no architecture of this package has them).
            axes = torch.empty((self.position_axes, n), dtype=torch.int32, pin_memory=True)
            at = 0
            for e, start, q in zip(entries, starts, q_lens):
                own = torch.arange(start, start + q, dtype=torch.int32)
                axes[0, at:at + q] = own
                for a in range(1, self.position_axes):
                    axes[a, at:at + q] = own if e.positions is None else torch.tensor(list(e.positions[a - 1]), dtype=torch.int32)
                at += q
            ctx.position_axes = axes.to(self.device, non_blocking=True)
        return ctx

    def step(self, entries: Sequence[StepEntry], sampled_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run the given tokens as one batch from the cache that earlier steps left and
        return float32 logits ``[wanted, vocab]`` in the order of the entries and of their
        ``want`` lists.  The tensor is scratch memory: it is valid until the next step."""
        with profiling.scope("pack (index arrays, pages, one copy)"):
            ctx = self.prepare(entries, sampled_ids)
        with profiling.scope("launch (the model's kernels)"), torch.cuda.device(self.device):
            logits = self._forward(ctx)
        self.steps_run += 1
        return logits

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        if not (self.cuda_graphs and ctx.all_decode) or self.position_axes > 1:
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
        # No garbage collection while the stream captures: an object that is collected then (an engine of an earlier
        # test, say) frees pinned memory, events or graphs of its own, and some of those calls are not allowed
        # during a capture and spoil it.
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx)
        finally:
            self._capturing = False
            if collecting:
                gc.enable()
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
