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

import torch

from .. import ops
from ..cache.manager import CacheManager, OutOfPages
from ..parts.base import CacheView, HostBatch, StepContext


@dataclass
class StepEntry:
    """The next ``tokens`` of request ``rid``; ``want`` lists the indices among these
    tokens whose logits are returned (in this order)."""
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


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
    def prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Grow the requests in the cache, build the step's index arrays and copy them
        to the device.  Raises OutOfPages before changing anything if the pages do not
        suffice for the whole batch."""
        cache = self.cache
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.rid!r}: a step entry needs at least one token")
            for t in e.tokens:
                if not (0 <= int(t) < self.vocab):
                    raise StepError(f"request {e.rid!r}: token id {t} outside the vocabulary [0, {self.vocab})")
            for w in e.want:
                if not (0 <= int(w) < len(e.tokens)):
                    raise StepError(f"request {e.rid!r}: wanted index {w} outside its {len(e.tokens)} tokens")
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

        token_ids, positions, seq_of_token, logit_rows, cu_q = [], [], [], [], [0]
        for i, e in enumerate(entries):
            base = cu_q[-1]
            token_ids.extend(int(t) for t in e.tokens)
            positions.extend(range(starts[i], starts[i] + q_lens[i]))
            seq_of_token.extend([i] * q_lens[i])
            logit_rows.extend(base + int(w) for w in e.want)
            cu_q.append(base + q_lens[i])
        widths = []
        for g in range(n_groups):
            w = max(1, max(len(cache.table(e.rid, g)) for e in entries))
            if ctx.all_decode:      # few distinct widths, so that captured steps are reused as contexts grow
                w = -(-w // self.TABLE_BUCKET) * self.TABLE_BUCKET
            widths.append(w)
        ctx.table_widths = tuple(widths)
        segments: List[Tuple[str, List[int]]] = [
            ("token_ids", token_ids), ("positions", positions), ("seq_of_token", seq_of_token), ("cu_q", cu_q),
            ("kv_len", kv_lens), ("state_slots", state_slots), ("logit_rows", logit_rows)]
        for g in range(n_groups):
            slots: List[int] = []
            table: List[int] = []
            for i, e in enumerate(entries):
                slots.extend(cache.slots(e.rid, g, starts[i], q_lens[i]))
                row = cache.table(e.rid, g)
                table.extend(row)
                table.extend([-1] * (widths[g] - len(row)))
            segments.append((f"slots{g}", slots))
            segments.append((f"table{g}", table))
        offsets, total = {}, 0
        for name, values in segments:
            offsets[name] = (total, len(values))
            total += _align(max(len(values), 1))
        stage = self._stage(total)
        flat: List[int] = []
        for name, values in segments:
            flat.extend(values)
            flat.extend([0] * (_align(max(len(values), 1)) - len(values)))
        stage[:total] = torch.tensor(flat, dtype=torch.int32)
        if self._index_buf is None or self._index_buf.numel() < total:
            self._index_buf = torch.empty(max(total, 4096) * 2, dtype=torch.int32, device=self.device)
            self.scratch_epoch += 1
        dev = self._index_buf
        dev[:total].copy_(stage[:total], non_blocking=True)
        self.h2d_bytes += total * 4
        ev = torch.cuda.Event()
        ev.record()
        self._staging_events[self._staging_slot] = ev

        def seg(name: str) -> torch.Tensor:
            o, ln = offsets[name]
            return dev[o:o + ln]
        ctx.token_ids, ctx.positions, ctx.seq_of_token = seg("token_ids"), seg("positions"), seg("seq_of_token")
        ctx.cu_q, ctx.kv_len, ctx.state_slots, ctx.logit_rows = seg("cu_q"), seg("kv_len"), seg("state_slots"), seg("logit_rows")
        for g in range(n_groups):
            ctx.group_slots.append(seg(f"slots{g}"))
            ctx.group_tables.append(seg(f"table{g}").view(s, widths[g]))
        return ctx

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the given tokens as one batch from the cache that earlier steps left and
        return float32 logits ``[wanted, vocab]`` in the order of the entries and of their
        ``want`` lists.  The tensor is scratch memory: it is valid until the next step."""
        ctx = self.prepare(entries)
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
