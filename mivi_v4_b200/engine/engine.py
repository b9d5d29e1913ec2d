"""The engine: a model, its cache, the step function, and generation on top.

``step`` is the one function that runs the model: a batch of sequences with
unequal numbers of next tokens - whole prompts, then one token each, or any
cut in between - from the cache that earlier steps left, returning the logits
at the wanted places.  The generation loop, the trace replay program and the
benchmark all drive this function.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..cache import CacheError, SequenceCache
from ..ops import kernels as K
from ..sampling import Sampler, SamplingParams
from .generate import Request, run_generation
from .model import Model
from .step import StepContext, Workspace

Want = Union[None, str, Sequence[Sequence[int]]]


class StepError(ValueError):
    """A step that cannot run: an unknown slot, a token id outside the
    vocabulary, a wanted place outside the step's tokens, a full cache."""


class _Recorded:
    """A decode step of one shape (sequences, page-table widths), recorded as a CUDA graph over the
    engine's decode workspace: the graph, where its logits land, and the host copy of the step's
    integer arrays with the place of each array in it."""
    __slots__ = ("graph", "logits", "n_kernels", "flat", "spans", "generation")

    def __init__(self, graph, logits, n_kernels, flat, spans, generation):
        self.graph, self.logits, self.n_kernels = graph, logits, n_kernels
        self.flat, self.spans, self.generation = flat, spans, generation


def _width_for(blocks: int) -> int:
    """Page-table width of a recorded decode step: the next power of two, at least 8 pages, so that a
    sequence that grows to n pages passes through about log2(n) recordings."""
    w = 8
    while w < blocks:
        w *= 2
    return w


class Engine:
    def __init__(self, model: Model, *, max_tokens: int, max_batch: Optional[int] = None,
                 page_size: int = 64, max_step_tokens: int = 8192, cuda_graphs: bool = True,
                 max_graphs: int = 64, profile: bool = False):
        if model.dtype is None:
            raise ValueError("the model has no weights yet; use load_model()")
        if model.device.type != "cuda":
            raise RuntimeError(f"the engine runs on CUDA devices only, the model is on {model.device}")
        self.model = model
        self.dtype, self.device = model.dtype, model.device
        self.page_size = page_size
        n_pages = -(-int(max_tokens) // page_size)
        self.total_pages = n_pages
        # every live sequence holds at least one page, so there are never more sequences than pages
        n_slots = max_batch if max_batch is not None else min(n_pages, 256)
        self.max_batch = max(1, n_slots)
        self.plan = model.cache_plan()
        self.cache = SequenceCache(self.plan, n_slots=self.max_batch, n_pages=n_pages, page_size=page_size,
                                   dtype=self.dtype, device=self.device)
        self.ws = Workspace(self.device)
        self.max_step_tokens = int(max_step_tokens)
        self.max_positions = model.spec.max_positions
        self.steps_run = 0
        self.h2d_bytes = 0
        # Decode steps (one token per sequence, last logits wanted) replay a recorded CUDA graph, one per
        # shape (sequences, page-table widths).  All recordings work in ONE workspace and allocate from
        # one graph memory pool, so a recording costs its launch records only; the least recently used
        # go when there are more than ``max_graphs``.  When the workspace has to move a buffer (a
        # larger batch than any before), the recordings made before name stale addresses and are dropped.
        # ``profile``: every launch of every step is timed by stage and kernel (``profile_report``); steps
        # then run launch by launch, never from a recording
        self.profile = K.KernelProfile() if profile else None
        # (a build with index checks declares its bounds by host copies that cannot be recorded)
        self.cuda_graphs = bool(cuda_graphs) and model.graph_safe and not profile and not K.DEBUG_CHECKS
        self.max_graphs = max(1, int(max_graphs))
        self._graphs: "OrderedDict[tuple, _Recorded]" = OrderedDict()
        self._gws = Workspace(self.device)
        self._graph_pool = None
        self.graph_replays = 0
        self.graphs_recorded = 0
        self._launches_last_step = 0

    # ---- sequences ------------------------------------------------------------
    def open(self) -> int:
        """Start a sequence; returns its slot."""
        if self.cache.slots.free_count == 0 and self.cache.n_slots < self.total_pages:
            self.cache.grow_slots(min(self.total_pages, max(2 * self.cache.n_slots, 1)))
            self._graphs.clear()                          # the state storage moved
        return self.cache.assign()

    def close(self, slot: int) -> None:
        """The sequence is over; what it holds goes back to the cache."""
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def graph_keys(self) -> List[tuple]:
        """The decode-step shapes recorded so far: (sequences, ((cache group, page-table width), ...), whether
        the recording ends with the copy of the error flag)."""
        return list(self._graphs)

    def check_errors(self) -> None:
        """Raise ``KernelError`` if a kernel of a step that the host has waited for reported a fault
        (a bounded wait that ran out).  Costs nothing; call it where the host has just read a step's
        results.  ``generate`` does so with every step's tokens."""
        K.raise_seen_device_errors(self.device)

    def profile_report(self, reset: bool = True) -> dict:
        """Where the time of the steps since the last report went (an engine made with ``profile=True``):
        per stage of the model and per kernel its launches, device time, share, and where the wrapper
        knows them the bytes it had to move per second and its floating-point operations per second."""
        if self.profile is None:
            raise RuntimeError("this engine was not made with profile=True")
        return self.profile.report(reset)

    # ---- the step function -----------------------------------------------------
    def step(self, items: Sequence[Tuple[int, Sequence[int]]], want: Want = "last",
             copy: bool = True) -> Optional[torch.Tensor]:
        """Run ``items`` = [(slot, next tokens), ...] as one batch.

        ``want``: "last" (the last token of every sequence), "all", None, or
        one list of places per item (indices into that item's tokens).
        Returns float32 logits [wanted, vocab] on the device, in the order of the items and,
        within an item, of its places; None if nothing is wanted.  With ``copy=False`` the
        result is the engine's own buffer, valid until the next step.
        """
        K.raise_seen_device_errors(self.device)
        if self.cuda_graphs and isinstance(want, str) and want == "last":
            logits = self._try_decode(items)
            if logits is not None:
                return logits.clone() if copy else logits
        try:
            items = [(int(s), np.asarray(toks, dtype=np.int64).ravel()) for s, toks in items]
        except (TypeError, ValueError):
            raise StepError("a step is a list of (slot, token ids) with integer token ids") from None
        V = self.model.vocab_size
        seen = set()
        for slot, toks in items:
            if slot in seen:
                raise StepError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if toks.size == 0:
                raise StepError(f"slot {slot} brings no tokens")
            if toks.min() < 0 or toks.max() >= V:
                bad = toks[(toks < 0) | (toks >= V)]
                raise StepError(f"slot {slot}: token id {int(bad[0])} is outside the vocabulary of {V}")
            try:
                start = self.cache.length(slot)
            except CacheError as e:
                raise StepError(str(e)) from None
            if self.max_positions is not None and start + len(toks) > self.max_positions:
                raise StepError(f"slot {slot}: {start} + {len(toks)} tokens exceed the context of "
                                f"{self.max_positions}")
        if want is None:
            places: List[List[int]] = [[] for _ in items]
        elif isinstance(want, str):
            if want == "last":
                places = [[len(t) - 1] for _, t in items]
            elif want == "all":
                places = [list(range(len(t))) for _, t in items]
            else:
                raise StepError(f'want={want!r}: known are "last", "all", None or one list of places per item')
        else:
            try:
                places = [[int(i) for i in w] for w in want]
            except (TypeError, ValueError):
                raise StepError('want must be "last", "all", None or one list of integer places per item') from None
            if len(places) != len(items):
                raise StepError(f"{len(places)} lists of wanted places for {len(items)} items")
            for (slot, toks), w in zip(items, places):
                if any(not 0 <= i < len(toks) for i in w):
                    raise StepError(f"slot {slot}: a wanted place is outside its {len(toks)} tokens")
        # room for everything, or nothing is touched
        for g in self.cache.kv_groups:
            need = sum(max(0, -(-(self.cache.length(s) + len(t)) // self.page_size)
                           - len(self.cache._get(s).pages[g])) for s, t in items)
            if need > self.cache.pages[g].free_count:
                raise StepError(f"the cache is full: this step needs {need} more pages of {self.page_size} "
                                f"tokens, {self.cache.pages[g].free_count} of {self.total_pages} are free")

        n_out = sum(len(w) for w in places)
        total = sum(len(t) for _, t in items)
        if total <= self.max_step_tokens:
            logits = self._run(items, places)
            if logits is not None and copy:
                logits = logits.clone()
            return logits
        # a step larger than the workspace is cut into pieces; the cache makes the cut invisible
        out = torch.empty((n_out, V), dtype=torch.float32, device=self.device) if n_out else None
        out_base = []
        acc = 0
        for w in places:
            out_base.append(acc)
            acc += len(w)
        chunk_items: List[Tuple[int, List[int]]] = []
        chunk_places: List[List[int]] = []
        chunk_dst: List[int] = []
        room = self.max_step_tokens

        def flush():
            nonlocal chunk_items, chunk_places, chunk_dst, room
            if chunk_items:
                lg = self._run(chunk_items, chunk_places)
                if lg is not None:
                    # the rows' places go up like the step's other integers: no copy that the host waits for
                    out.index_copy_(0, self.ws.stage("chunk_rows", chunk_dst).long(), lg)
            chunk_items, chunk_places, chunk_dst, room = [], [], [], self.max_step_tokens

        for idx, ((slot, toks), w) in enumerate(zip(items, places)):
            done = 0
            while done < len(toks):
                if room == 0:
                    flush()
                take = min(room, len(toks) - done)
                sub = [(j, i - done) for j, i in enumerate(w) if done <= i < done + take]
                chunk_items.append((slot, toks[done:done + take]))
                chunk_places.append([i for _, i in sub])
                chunk_dst.extend(out_base[idx] + j for j, _ in sub)
                room -= take
                done += take
                if done < len(toks):
                    flush()                               # the same slot cannot be twice in one piece
        flush()
        return out

    def _run(self, items, places) -> Optional[torch.Tensor]:
        """One step of at most ``max_step_tokens`` tokens, already checked."""
        if self.cuda_graphs and all(len(t) == 1 for _, t in items) and all(w == [0] for w in places):
            slots = np.fromiter((s for s, _ in items), dtype=np.int64, count=len(items))
            toks = np.fromiter((int(t[0]) for _, t in items), dtype=np.int64, count=len(items))
            logits = self._decode(slots, toks, None)
            if logits is not None:
                return logits
        slots = [s for s, _ in items]
        starts = [self.cache.length(s) for s in slots]
        for s, toks in items:
            self.cache.reserve(s, len(toks))
        out_rows: List[int] = []
        row = 0
        for (_, toks), w in zip(items, places):
            out_rows.extend(row + i for i in w)
            row += len(toks)
        page_rows = {g: self.cache.page_rows(g, slots) for g in self.cache.kv_groups}
        lists = [t for _, t in items]
        ctx = StepContext(slots=slots, starts=starts, token_lists=lists, out_rows=out_rows,
                          page_rows=page_rows, dtype=self.dtype, ws=self.ws)
        if self.profile is not None and ctx.n_tokens <= 256:
            # a step of short kernels: let its launches queue up behind a busy stream, so that their times
            # are the device's and not the host's pace of launching (about 40 us a launch with its events)
            K.delay(min(50000, 40 * max(self._launches_last_step, 100)))
        n0 = K.launch_count()
        with K.profiling(self.profile):
            logits = self.model.forward(ctx, self.cache)
        self._launches_last_step = K.launch_count() - n0
        if self.profile is not None:
            self.profile.steps += 1
        K.note_device_errors(self.device)
        for s, toks in zip(slots, lists):
            self.cache.advance(s, len(toks))
        self.steps_run += 1
        self.h2d_bytes += ctx.h2d_bytes
        return logits

    # ---- decode steps: one token for each sequence, every row's logits ------------------------------
    def _try_decode(self, items) -> Optional[torch.Tensor]:
        """``items`` as a decode step if they are one: None sends the caller down the general path,
        which also words the errors."""
        B = len(items)
        try:
            if B == 0 or any(len(t) != 1 for _, t in items):
                return None
            slots = np.fromiter((s for s, _ in items), dtype=np.int64, count=B)
            toks = np.fromiter((t[0] for _, t in items), dtype=np.int64, count=B)
        except (TypeError, ValueError, IndexError):
            return None
        if int(toks.min()) < 0 or int(toks.max()) >= self.model.vocab_size:
            return None
        return self._decode(slots, toks, None)

    def _decode(self, slots: np.ndarray, toks: Optional[np.ndarray],
                device_tokens: Optional[torch.Tensor], note_errors: bool = True) -> Optional[torch.Tensor]:
        """One more token for each of ``slots`` (an array that names each slot once is checked here),
        the token ids from the host (``toks``) or from the device (``device_tokens``, int32).  Works on
        arrays over the sequences; the only per-sequence work is a new page when one crosses a page's
        end.  Returns None, with nothing touched, if the step cannot run as it stands.  ``note_errors``:
        the step ends with the copy of the device's error flag to the host; a caller whose next launch
        carries the flag itself (the sampling kernel, with the tokens) saves the copy."""
        cache = self.cache
        B = int(slots.size)
        if not cache.are_assigned(slots) or (B > 1 and np.unique(slots).size != B):
            return None
        lengths = cache.lengths_of(slots)
        if self.max_positions is not None and int(lengths.max()) + 1 > self.max_positions:
            return None
        widths: tuple = ()
        if cache.kv_groups:
            blocks = lengths // self.page_size + 1
            short = blocks > cache.blocks_of(slots)
            if short.any():
                need = int(short.sum())
                if any(cache.pages[g].free_count < need for g in cache.kv_groups):
                    return None
                for s in slots[short].tolist():
                    cache.reserve(s, 1)
            width = _width_for(int(blocks.max()))
            widths = tuple((g, width) for g in cache.kv_groups)
        key = (B, widths, bool(note_errors))
        rec = self._graphs.get(key)
        if rec is not None and rec.generation != self._gws.generation:
            del self._graphs[key]                         # recorded over buffers that have moved since
            rec = None
        if rec is None:
            logits = self._record(key, slots, lengths, toks, device_tokens)
        else:
            self._graphs.move_to_end(key)
            flat, spans = rec.flat, rec.spans
            if toks is not None:
                o = spans["tokens"][0]
                flat[o:o + B] = toks
            for name, values in (("positions", lengths), ("starts", lengths), ("slots", slots)):
                o = spans[name][0]
                flat[o:o + B] = values
            for g, w in widths:
                o, n = spans[f"pages{g}"]
                flat[o:o + n] = cache.table_rows(g, slots, w).reshape(-1)
            arena = self._gws.stage("step_meta", flat)
            if device_tokens is not None:
                o = spans["tokens"][0]
                arena[o:o + B].copy_(device_tokens, non_blocking=True)
            rec.graph.replay()
            K.add_launches(rec.n_kernels)
            self.graph_replays += 1
            self.h2d_bytes += flat.size * 4
            logits = rec.logits
        cache.advance_each_by_one(slots)
        self.steps_run += 1
        return logits

    def _record(self, key, slots: np.ndarray, lengths: np.ndarray, toks: Optional[np.ndarray],
                device_tokens: Optional[torch.Tensor]) -> torch.Tensor:
        """The first decode step of a shape: run it for real in the decode workspace (which sizes every
        buffer and notes which weights the products read, in order), then record the same launches for
        the steps to come; recorded, each product of few rows asks the L2 cache for its successor's
        weights."""
        from ..ops import linear as L
        gws = self._gws
        B = int(slots.size)
        before = gws.generation
        lists = [[int(t)] for t in toks] if toks is not None else [[0]] * B
        page_rows = {g: self.cache.table_rows(g, slots, w).tolist() for g, w in key[1]}
        ctx = StepContext(slots=slots.tolist(), starts=lengths.tolist(), token_lists=lists, out_rows=list(range(B)),
                          page_rows=page_rows, dtype=self.dtype, ws=gws)
        if device_tokens is not None:
            ctx.tokens.copy_(device_tokens, non_blocking=True)
        with L.recording() as order:
            logits = self.model.forward(ctx, self.cache)
        if gws.generation != before:
            self._graphs.clear()                          # a buffer moved: older recordings name its old place
        settled = gws.generation
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        n0 = K.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, pool=self._graph_pool), L.looking_ahead(order, self.model.weight_extents()):
            captured = self.model.forward(ctx, self.cache)
            if key[2]:
                K.note_device_errors(self.device)
        n_kernels = K.launch_count() - n0
        K.add_launches(-n_kernels)                        # recorded, not run
        if captured.data_ptr() != logits.data_ptr() or gws.generation != settled:
            raise RuntimeError("a decode step allocated while it was recorded; its recording cannot be replayed")
        self._graphs[key] = _Recorded(graph, logits, n_kernels, ctx._flat, ctx.spans, settled)
        self.graphs_recorded += 1
        while len(self._graphs) > self.max_graphs:
            self._graphs.popitem(last=False)
        self.h2d_bytes += ctx.h2d_bytes
        return logits

    def decode_from_device(self, slots: Sequence[int], device_tokens: torch.Tensor,
                           note_errors: bool = True) -> Optional[torch.Tensor]:
        """One more token for each of ``slots``, the token ids being ``device_tokens`` (int32 [len(slots)],
        on the device, e.g. what the sampling kernel just wrote): the step is enqueued without the host
        waiting for them.  Returns the logits of all, or None if the step cannot run now (no room in the
        cache, the context is full): the caller then waits for the tokens and calls ``step``."""
        if not self.cuda_graphs or len(slots) == 0 or device_tokens.numel() != len(slots) \
                or device_tokens.dtype != torch.int32 or not device_tokens.is_cuda:
            return None
        try:
            arr = np.asarray(slots, dtype=np.int64)
        except (TypeError, ValueError):
            return None
        return self._decode(arr, None, device_tokens, note_errors)

    # ---- generation ---------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: Union[int, Sequence[int]] = 256,
                 sampling: Optional[SamplingParams] = None, stop_token_ids: Optional[Sequence[int]] = None,
                 on_token=None, return_requests: bool = False):
        """Token ids in, token ids out: one list of new tokens per prompt.
        ``stop_token_ids`` defaults to the model's end-of-sequence id."""
        sampling = sampling or SamplingParams()
        stops = list(self.model.spec.stop_token_ids) if stop_token_ids is None else list(stop_token_ids)
        backend = _EngineBackend(self, Sampler(sampling, self.model.vocab_size, self.device))
        requests = run_generation(prompts, max_new_tokens, backend, stops, on_token)
        return requests if return_requests else [r.output for r in requests]


class _EngineBackend:
    """What the generation loop asks of the engine."""

    def __init__(self, engine: Engine, sampler: Sampler):
        self.engine, self.sampler = engine, sampler
        self.max_batch, self.page_size = engine.max_batch, engine.page_size
        self.total_pages, self.max_positions = engine.total_pages, engine.max_positions
        self._early = None            # the step after the current one, already enqueued
        self._last = {}               # handle -> the token sampled for it in the last call

    def open(self) -> int:
        self._early, self._last = None, {}        # a new sequence may get the slot of an old one
        return self.engine.open()

    def close(self, handle: int) -> None:
        self._last.pop(handle, None)
        self.engine.close(handle)

    def forward_and_sample(self, requests: Sequence[Request], token_lists) -> List[int]:
        """Forward the given tokens and sample the next one for every request.

        The step AFTER this one is enqueued before the host waits for this one's tokens (the recent
        tokens that penalties look at are kept on the device by the sampling kernel itself): the
        sampling kernel's output is fed to the next step on the device, for every request that can
        go on (it has tokens left to generate).  If a request then turns out to have stopped, its row
        of the early step is simply not used; the other rows do not depend on it.  The next call finds
        its work already running.  The sampler has two sets of buffers; a step and the one enqueued
        early after it always use different ones."""
        sampler, eng = self.sampler, self.engine
        handles = [r.handle for r in requests]
        early, self._early = self._early, None
        if (early is not None and set(handles) <= set(early["handles"])
                and all(len(t) == 1 and self._last.get(h) == t[0] for h, t in zip(handles, token_lists))):
            rows = [early["handles"].index(h) for h in handles]
            out_dev, host, event, cur = early["out"], early["host"], early["event"], early["set"]
        else:
            if early is not None and set(handles) & set(early["handles"]):
                # the early step has already advanced these sequences by the tokens it sampled itself
                raise RuntimeError("the generation loop fed other tokens than the ones sampled for its sequences")
            cur = 1 - early["set"] if early is not None else 0
            logits = eng.step([(r.handle, t) for r, t in zip(requests, token_lists)], "last", copy=False)
            with K.profiling(eng.profile), K.profile_stage("sampling"):
                out_dev = sampler.launch(logits, [r.index for r in requests], [len(r.output) for r in requests],
                                         [r.output for r in requests], slot=cur, states=handles)
            host, event = sampler.read_async(out_dev, slot=cur)
            rows = list(range(len(requests)))
        # the step after this one, for the requests that will still have tokens to generate
        if eng.cuda_graphs:
            goers = [(i, r) for i, r in zip(rows, requests) if len(r.output) + 2 <= r.max_new_tokens]
            if goers:
                picks = [i for i, _ in goers]
                src = out_dev if picks == list(range(out_dev.numel())) else \
                    out_dev[torch.tensor(picks, device=out_dev.device)]
                # the sampling kernel after it carries the error flag to the host with the tokens
                nxt = eng.decode_from_device([r.handle for _, r in goers], src, note_errors=False)
                if nxt is not None:
                    with K.profiling(eng.profile), K.profile_stage("sampling"):
                        out2 = sampler.launch(nxt, [r.index for _, r in goers], [len(r.output) + 1 for _, r in goers],
                                              [[] for _ in goers], slot=1 - cur, states=[r.handle for _, r in goers],
                                              carry_flag=True)
                    host2, event2 = sampler.read_async(out2, slot=1 - cur)
                    self._early = dict(handles=[r.handle for _, r in goers], out=out2, host=host2, event=event2,
                                       set=1 - cur)
        event.synchronize()
        code = sampler.flag(cur)                 # the flag as this step's sampling kernel saw it, if it carried it
        if code:
            K.raise_device_error(eng.device, code)
        eng.check_errors()                       # and the copy that steps of the step function end with
        tokens = host.tolist()
        result = [tokens[i] for i in rows]
        self._last = dict(zip(handles, result))
        return result
