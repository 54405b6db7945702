"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step takes, for each participating request, its next tokens — a portion of a prompt of
any length, or a single decoded token — and the places among them whose logits are wanted.
All entries run as one flat batch; only the tokens given are computed, everything earlier
comes from the cache.  Lengths are committed after the model ran, so a step that fails
leaves the cache as it was (the reference commits the same way,
crates/model/src/qwen3/gpu.rs:374-375).  The reference's forward takes one sequence per
pass (crates/runtime/src/lib.rs:67-100); the mixed batch is this engine's own design.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import ctypes
import gc

import numpy as np
import torch

from ..cache.manager import DROPPED, CacheManager, PagedView, StateView
from ..cache.pages import CONTEXT_FULL, OK, OUT_OF_PAGES, OutOfPages
from ..kernels import ops
from ..models.model import Model
from ..parts.base import Runtime
from .context import Span, StepContext, Workspace


class StepError(ValueError):
    """A step that cannot run as asked: unknown request, bad token id, context full."""


@dataclass
class StepEntry:
    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


class CacheViews:
    """Hands each schedule entry its view of the cache for the current step."""

    def __init__(self, cache: CacheManager):
        self.cache = cache

    def view(self, index: int, ctx: StepContext):
        cache = self.cache
        owner_index = cache.cache_of[index] if cache.cache_of[index] is not None else index
        if owner_index in cache.place:
            g, j = cache.place[owner_index]
            group = cache.groups[g]
            return PagedView(group.k[j], group.v[j], ctx.group_block_tables[g], ctx.group_slot_mappings[g],
                             cache.page_size, owner=owner_index == index)
        if owner_index in cache.state:
            return StateView(cache.state[owner_index], ctx.state_slots, owner=owner_index == index)
        return None


class Runner:
    """Owns the model, the cache manager and the workspace; ``step`` is the only way tokens run."""

    def __init__(self, model: Model, cache: CacheManager, rt: Runtime, max_seq_len: int):
        self.model, self.cache, self.rt = model, cache, rt
        self.max_seq_len = int(max_seq_len)
        self.max_pages_per_seq = -(-self.max_seq_len // cache.page_size)
        self.workspace = Workspace(rt.device)
        self.views = CacheViews(cache)
        self.vocab = model.spec.vocab_size
        #: the kernels' scratch memory, error flag and result buffer of this runner alone (see ``ops.Scratch``)
        self.scratch = None
        if rt.device.type == "cuda":
            self.scratch = ops.Scratch(rt.device)
        #: where a replayed graph's arg-max leaves the step's ids for the host (pinned memory the kernel writes itself,
        #: two rows in turn) and the events behind the last two replays: the host waits for the event and reads,
        #: with no copy of its own in the stream (``read_graph_ids``)
        self._mirror: Optional[torch.Tensor] = None
        self._mirror_done: List[object] = []
        self._which = self._ran = 0
        self._pinned: Optional[torch.Tensor] = None           # host side of the packed inputs of steps run without a graph
        self._pinned_free = None                               # the event after which it may be written again
        self.steps_run = 0
        self._longest = 1
        #: after a step replayed from a graph: int32 ids of the largest logit of each returned row (lowest id among
        #: equals), computed inside the graph; None after any other step
        self.greedy_ids: Optional[torch.Tensor] = None
        self._replayed: Optional[dict] = None      # the graph the last step was replayed from, if it was
        self._prepared: Optional[dict] = None      # the next step's inputs, packed ahead (see prepare_next)

    # ---- requests ----------------------------------------------------------------------------------
    def begin(self, req_id: Hashable) -> None:
        self.cache.admit(req_id)

    def end(self, req_id: Hashable) -> None:
        self.cache.release(req_id)

    def length(self, req_id: Hashable) -> int:
        return self.cache.length(req_id)

    # ---- the step ------------------------------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.req_id in seen:
                raise StepError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            if e.req_id not in self.cache.requests:
                raise StepError(f"request {e.req_id!r} is not live")
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.req_id!r} brings no tokens")
            if n == 1:
                low = high = int(e.tokens[0])
            else:
                ids = np.asarray(e.tokens)
                if ids.dtype.kind not in "iu":
                    raise StepError(f"request {e.req_id!r}: token ids must be integers")
                low, high = int(ids.min()), int(ids.max())
            if low < 0 or high >= self.vocab:
                bad = next(t for t in e.tokens if not 0 <= int(t) < self.vocab)
                raise StepError(f"request {e.req_id!r}: token id {bad} is outside the vocabulary of {self.vocab}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"request {e.req_id!r}: wanted place {w} is outside its {n} tokens")

    def build_context(self, entries: Sequence[StepEntry], pad_to: int = 0, static=None, refresh_only: bool = False,
                      pack_only: bool = False):
        """Flattens the entries (single tokens first) into the arrays the kernels read, and copies
        them to the device in one transfer.  ``pad_to`` (decode batches only) pads the batch with empty
        requests up to a fixed size; ``static`` is then the device buffer a captured graph reads, and with
        ``refresh_only`` nothing but that buffer is wanted (a replay follows): no context is built; with ``pack_only``
        the pinned host buffer is filled and not copied (the device buffer may still be read by the step that runs)."""
        cache = self.cache
        n = len(entries)
        counts = np.fromiter((len(e.tokens) for e in entries), np.int32, n)
        want_counts = np.fromiter((len(e.want) for e in entries), np.int32, n)
        tokens = np.concatenate([np.asarray(e.tokens, np.int32) for e in entries]) if n > 1 else np.asarray(entries[0].tokens, np.int32)
        wants = np.fromiter((w for e in entries for w in e.want), np.int32, int(want_counts.sum()))
        handles = np.fromiter((cache.requests[e.req_id].handle for e in entries), np.int64, n)
        real_T = int(counts.sum())
        R, T = (pad_to, pad_to) if pad_to else (n, real_T)
        W = pad_to if pad_to else int(want_counts.sum())
        maxb = self.max_pages_per_seq
        G = len(cache.groups)
        sizes = [T, T, T, R + 1, R, R, W, G * R * maxb, G * T]
        total = sum(sizes)
        if static is not None:
            host, dev, copied = static
            copied.synchronize()                 # the last step's copy has left the pinned buffer
            packed = host.numpy()
        elif self.rt.device.type == "cuda":
            # one pinned buffer serves every step that runs without a graph; it grows when a step needs more
            if self._pinned is None or self._pinned.numel() < total:
                self._pinned = torch.empty(max(total, 1 << 16), dtype=torch.int32).pin_memory()
                self._pinned_free = torch.cuda.Event()
            else:
                self._pinned_free.synchronize()
            packed = self._pinned.numpy()[:total]
        else:
            packed = np.empty(total, np.int32)
        info = np.zeros(8, np.int32)
        span_rows = np.zeros((n, 5), np.int32)
        # the C++ side walks the block tables and writes the arrays in place (csrc/host/cache_core.cpp)
        wrote = cache._lib.mbh_pack_step(cache._core(), n, handles.ctypes.data, counts.ctypes.data, tokens.ctypes.data,
                                        want_counts.ctypes.data, wants.ctypes.data, int(pad_to), maxb, packed.ctypes.data,
                                        int(packed.size), info.ctypes.data, span_rows.ctypes.data)
        if wrote != total:
            raise StepError(f"packing the step failed (code {wrote}, {total} values expected)")
        num_decode, max_query_len, max_seq_len = int(info[3]), int(info[4]), int(info[5])
        num_rows = W
        if static is not None:
            self._which ^= 1
            packed[total] = self._which          # the row of the ids' mirror this step's arg-max writes (see _graph_for)
            if pack_only:
                return None
            dev.copy_(host, non_blocking=True)
            copied.record()
            if refresh_only:
                return None
        elif self.rt.device.type == "cuda":
            dev = self._pinned[:total].to(self.rt.device, non_blocking=True)
            self._pinned_free.record()
        else:
            dev = torch.from_numpy(packed)
        spans = [Span(row, entries[int(i)].req_id, int(at), int(cnt), int(first), int(slot))
                 for row, (i, at, cnt, first, slot) in enumerate(span_rows.tolist())]
        views, at = [], 0
        for size in sizes:
            views.append(dev[at:at + size])
            at += size
        d_tok, d_pos, d_req, d_cu, d_lens, d_slots, d_rows, d_tables, d_maps = views
        return StepContext(
            num_tokens=T, num_requests=R, num_decode=R if pad_to else num_decode, num_logit_rows=num_rows,
            max_query_len=max_query_len, max_seq_len=max_seq_len,
            token_ids=d_tok, positions=d_pos, req_index=d_req, cu_tokens=d_cu, seq_lens=d_lens,
            state_slots=d_slots, logit_rows=d_rows,
            group_block_tables=[d_tables.view(G, R, maxb)[g] for g in range(G)] if G else [],
            group_slot_mappings=[d_maps.view(G, T)[g] for g in range(G)] if G else [],
            spans=spans, workspace=self.workspace,
        )

    def packed_size(self, pad_to: int) -> int:
        G = len(self.cache.groups)
        return pad_to * 3 + (pad_to + 1) + pad_to * 2 + pad_to + G * pad_to * self.max_pages_per_seq + G * pad_to

    def _replay(self, g: dict) -> None:
        g["graph"].replay()
        self._mirror_done[self._which].record()
        self._ran = self._which                  # the mirror's row the replay writes (packing ahead moves _which on)
        ops.launches_extra(g["launches"])
        self._replayed = g

    def read_graph_ids(self, rows: int, which: Optional[int] = None) -> List[int]:
        """The ids the arg-max of a replayed graph left in the host's mirror (-1: that row's logits were not finite), for
        the last replay or the one before (``which``): waits for the event behind that replay, not for anything
        launched since.  Raises ``KernelError`` if a kernel's wait gave up."""
        w = self._ran if which is None else which
        self._mirror_done[w].synchronize()
        both = self._mirror[w, :4 + rows].tolist()
        if both[0]:
            torch.cuda.synchronize()
            self.scratch.clear()
            raise ops.KernelError(f"a tensor-core kernel's wait on an mbarrier gave up (code {both[0]})")
        return both[4:]

    # ---- decode steps as CUDA graphs -----------------------------------------------------------------------
    def enable_graphs(self, batch_sizes: Sequence[int] = (1, 2, 4, 8, 16, 32, 64)) -> None:
        """Steps in which every request brings exactly one token are replayed from a CUDA graph captured per
        padded batch size: the kernels' arguments live in one static device buffer that each step overwrites.
        Whether a model's single-token steps can be captured is its parts' answer (``Mixer.capturable``,
        ``FeedForward.capturable``); if one of them says no, graphs are left off."""
        capturable = getattr(self.model, "capturable", None)
        if capturable is None or not capturable():
            return
        self.graph_sizes = sorted(set(int(b) for b in batch_sizes))
        self.graphs: Dict[tuple, dict] = {}

    #: sequences up to this long share the shortest graph; longer ones take the next power of two
    GRAPH_MIN_SPAN = 1024

    def _span_of(self, longest: int) -> int:
        span = self.GRAPH_MIN_SPAN
        while span < longest:
            span *= 2
        return min(span, self.max_seq_len)

    def _graph_for(self, bucket: int, entries: Sequence[StepEntry]) -> dict:
        # A graph is captured per padded batch size and per span of sequence lengths (a power of two, at most the
        # context capacity): the split of the keys over CTAs is part of the captured grid, and a split made for the
        # whole capacity would leave short sequences to one CTA each.
        key = (bucket, self._span_of(self._longest))
        span = key[1]
        g = self.graphs.get(key)
        if g is not None:
            return g
        size = self.packed_size(bucket)
        host = torch.zeros(size + 1, dtype=torch.int32).pin_memory()       # one int more: which row of the ids' mirror
        dev = torch.zeros(size + 1, dtype=torch.int32, device=self.rt.device)
        if self._mirror is None:
            self._mirror = torch.zeros(2, 4 + self.scratch.RESULT_ROWS, dtype=torch.int32).pin_memory()
            self._mirror_done = [torch.cuda.Event(), torch.cuda.Event()]
        # what each kind of mixer fixes ahead for this batch size and span (for attention: the split of the keys, which
        # is part of the captured grid, and scratch of the capture's own), asked of the mixers themselves
        shared = next((o for (b, _), o in self.graphs.items() if b == bucket), None)
        g = {"key": key, "static": (host, dev, torch.cuda.Event()), "workspace": shared["workspace"] if shared else Workspace(self.rt.device),
             "graph": None, "logits": None, "plans": self.model.decode_plans(bucket, span)}
        self.graphs[key] = g

        def run():
            ctx = self.build_context(entries, pad_to=bucket, static=g["static"])
            ctx.workspace = g["workspace"]
            ctx.decode_plans = g["plans"]
            return self.model.forward(ctx, self.views)

        # Warm up: builds kernels, sizes the workspace.  The step runs for real here and once more when the captured
        # graph is first replayed.  Keys and values are written to the same places with the same values both times;
        # per-request state is not like that (a recurrence would advance twice), so it is put back after the warm-up.
        kept = {i: t.clone() for i, t in self.cache.state.items()}
        with ops.using(self.scratch):
            run()
        torch.cuda.synchronize()
        for i, t in kept.items():
            self.cache.state[i].copy_(t)
        graph = torch.cuda.CUDAGraph()
        ctx = self.build_context(entries, pad_to=bucket, static=g["static"])
        ctx.workspace = g["workspace"]
        ctx.decode_plans = g["plans"]
        torch.cuda.synchronize()
        launches = ops.launches
        g["best"] = self.scratch.ids(bucket)     # behind the scratch's report: the host reads both in one copy
        # No garbage collection while the stream is capturing: an engine or a tensor dropped earlier that is freed now
        # (pinned memory, events, older graphs) would make a CUDA call that a capture does not allow, and the capture
        # would be lost.  (torch.cuda.graph collects once before it begins.)
        collecting = gc.isenabled()
        gc.disable()
        logging, ops.launch_log = ops.launch_log, []      # what the graph's kernels are, in order (engine/profile.py)
        try:
            with ops.using(self.scratch), torch.cuda.graph(graph):
                g["logits"] = self.model.forward(ctx, self.views)
                ops.stage_name = "sampling"
                # greedy sampling rides in the same graph; the ids also go where the next step reads its token ids
                # (a step launched ahead is fed there) and, written by the kernel itself, to the host's mirror
                ops.argmax(g["logits"], self.vocab, g["best"], feed=dev[:bucket], mirror=self._mirror, which=dev[size:size + 1])
        finally:
            g["labels"], ops.launch_log = ops.launch_log, logging
            if collecting:
                gc.enable()
        g["launches"] = ops.launches - launches
        g["graph"] = graph
        return g

    def _step_graph(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        sizes = getattr(self, "graph_sizes", None)
        if not sizes or any(len(e.tokens) != 1 for e in entries):
            return None
        bucket = next((b for b in sizes if b >= len(entries)), None)
        if bucket is None:
            return None
        g = self._graph_for(bucket, entries)
        self.build_context(entries, pad_to=bucket, static=g["static"], refresh_only=True)
        self._replay(g)
        rows = [i for i, e in enumerate(entries) for _ in e.want]
        if rows == list(range(len(entries))):
            self.greedy_ids = g["best"][: len(entries)]      # the largest logit of each returned row, already found
            return g["logits"][: len(entries)]
        return g["logits"][torch.as_tensor(rows, device=self.rt.device, dtype=torch.long)]

    def step(self, entries: Sequence[StepEntry], observe=None) -> torch.Tensor:
        """Runs the entries as one batch; returns float32 logits ``[wanted, vocab]`` on the device,
        in the order of the entries and of each entry's ``want``.  ``observe`` (see ``Model.forward``) turns
        graph replay off for this step."""
        self._validate(entries)
        self.greedy_ids = None
        prepared, self._prepared, self._replayed = self._prepared, None, None
        if prepared is not None and observe is None and self._is_the_prepared_step(prepared, entries):
            return self._run_prepared(prepared, entries)
        cache, n = self.cache, len(entries)
        handles = np.fromiter((cache.requests[e.req_id].handle for e in entries), np.int64, n)
        counts = np.fromiter((len(e.tokens) for e in entries), np.int32, n)
        # one call checks the context capacity and takes every entry's pages, or takes none
        info = (ctypes.c_int * 2)()
        rc = cache._lib.mbh_step_reserve(cache._core(), n, handles.ctypes.data, counts.ctypes.data, self.max_seq_len, info)
        self._longest = int(info[1])
        if rc == CONTEXT_FULL:
            e = entries[info[0]]
            raise StepError(f"request {e.req_id!r}: context full ({cache.length(e.req_id) + len(e.tokens)} positions needed, "
                            f"capacity {self.max_seq_len})")
        if rc == OUT_OF_PAGES:
            raise OutOfPages(f"the step needs more pages than are free ({cache.free_pages()} free per group)")
        if rc != OK:
            raise StepError(f"reserving the step's pages failed (code {rc})")
        logits = self._step_graph(entries) if observe is None else None
        if logits is None:
            ctx = self.build_context(entries)
            with ops.using(self.scratch):
                logits = self.model.forward(ctx, self.views, observe) if observe is not None else self.model.forward(ctx, self.views)
        rc = cache._lib.mbh_step_commit(cache._core(), n, handles.ctypes.data, counts.ctypes.data)
        if rc != OK:
            raise StepError(f"recording the step failed (code {rc})")
        self.steps_run += 1
        return logits

    # ---- the next step, packed while this one runs -------------------------------------------------------------
    def prepare_next(self, entries: Sequence[StepEntry]) -> bool:
        """To be called right after a step that was replayed from a graph, while the GPU runs it.  Supposes that the
        same requests bring one token each to the next step too (no request ends, none joins): takes their pages and
        packs that step's inputs, all but the token ids, into the graph's pinned buffer.  If the next call of
        ``step`` brings exactly that, only the ids are filled in and copied; if it brings anything else the packed
        buffer is forgotten (the pages taken are the requests' own either way).  Returns whether it prepared."""
        g, self._prepared = self._replayed, None
        if g is None or any(len(e.tokens) != 1 for e in entries):
            return False
        cache, n = self.cache, len(entries)
        try:
            handles = np.fromiter((cache.requests[e.req_id].handle for e in entries), np.int64, n)
        except KeyError:
            return False
        counts = np.ones(n, np.int32)
        info = (ctypes.c_int * 2)()
        if cache._lib.mbh_step_reserve(cache._core(), n, handles.ctypes.data, counts.ctypes.data, self.max_seq_len, info) != OK:
            return False                          # full context or no pages: the step itself will say so
        longest = int(info[1])
        if (g["key"][0], self._span_of(longest)) != g["key"]:
            return False                          # the sequences grow into the next graph
        ahead = [StepEntry(e.req_id, [0], [0]) for e in entries]
        self.build_context(ahead, pad_to=g["key"][0], static=g["static"], pack_only=True)
        self._prepared = {"graph": g, "ids": [e.req_id for e in entries], "handles": handles, "counts": counts, "longest": longest}
        return True

    # ---- the next step, launched before this one's tokens are known ------------------------------------------------
    def launch_ahead(self, entries: Sequence[StepEntry]) -> Optional[dict]:
        """To be called right after a step of single tokens that was replayed from a graph, with the same entries.
        Supposes that the same requests go on with the tokens this step is about to produce, and launches that next
        step now: the ids the graph's arg-max leaves on the device are copied into the next step's inputs on the device,
        so the GPU goes from one step into the next while the host still waits for, reads and books the first one's
        tokens.  Returns a handle for ``read_ahead`` / ``commit_ahead``, or None if the step could not be prepared (no
        pages, context full, the sequences grow into another graph): then nothing was launched.

        The launched step's lengths are NOT committed here: the caller commits them for the requests that turn out to
        go on (``commit_ahead``) once it knows; a request that ended meanwhile has computed one token for nothing."""
        g = self._replayed
        if g is None or self.scratch is None or not self.prepare_next(entries):
            return None
        prepared, self._prepared = self._prepared, None
        n, bucket = len(entries), g["key"][0]
        before = self._ran                                     # the running step's row of the ids' mirror
        host, dev, copied = g["static"]
        # positions, lengths, tables and places of the next step; its token ids are on the device already: the running
        # step's arg-max puts them there, never seen by the host
        dev[bucket:].copy_(host[bucket:], non_blocking=True)
        copied.record()
        self._replay(g)
        self._longest = prepared["longest"]
        self.greedy_ids = g["best"][:n]
        return {"before": before, "which": self._which, "rows": n, "req_ids": prepared["ids"], "handles": prepared["handles"], "graph": g}

    def read_ahead(self, ahead: dict) -> List[int]:
        """The ids of the step BEFORE the one ``launch_ahead`` launched: waits for that step only, not for the one that runs."""
        return self.read_graph_ids(ahead["rows"], ahead["before"])

    def commit_ahead(self, ahead: dict, live: Sequence[Hashable]) -> None:
        """Books the step ``launch_ahead`` launched, for the requests of it that are still live (in ``live``)."""
        keep = [i for i, rid in enumerate(ahead["req_ids"]) if rid in live and rid in self.cache.requests
                and self.cache.requests[rid].handle == int(ahead["handles"][i])]
        if keep:
            handles = np.ascontiguousarray(ahead["handles"][keep])
            counts = np.ones(len(keep), np.int32)
            rc = self.cache._lib.mbh_step_commit(self.cache._core(), len(keep), handles.ctypes.data, counts.ctypes.data)
            if rc != OK:
                raise StepError(f"recording the step launched ahead failed (code {rc})")
        self.steps_run += 1

    def _is_the_prepared_step(self, prepared: dict, entries: Sequence[StepEntry]) -> bool:
        ids, handles, requests = prepared["ids"], prepared["handles"], self.cache.requests
        if len(entries) != len(ids):
            return False
        for e, rid, handle in zip(entries, ids, handles.tolist()):
            if e.req_id != rid or len(e.tokens) != 1 or list(e.want) != [0] or requests[e.req_id].handle != handle:
                return False
        return True

    def _run_prepared(self, prepared: dict, entries: Sequence[StepEntry]) -> torch.Tensor:
        g, n = prepared["graph"], len(entries)
        host, dev, copied = g["static"]
        host.numpy()[:n] = [e.tokens[0] for e in entries]      # the token ids lead the packed buffer
        dev.copy_(host, non_blocking=True)
        copied.record()
        self._replay(g)
        self._longest = prepared["longest"]
        rc = self.cache._lib.mbh_step_commit(self.cache._core(), n, prepared["handles"].ctypes.data, prepared["counts"].ctypes.data)
        if rc != OK:
            raise StepError(f"recording the step failed (code {rc})")
        self.steps_run += 1
        self.greedy_ids = g["best"][:n]
        return g["logits"][:n]
