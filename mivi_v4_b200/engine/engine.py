"""The engine: a model, its cache, the step function, and generation on top.

``step`` is the one function that runs the model: a batch of sequences with
unequal numbers of next tokens - whole prompts, then one token each, or any
cut in between - from the cache that earlier steps left, returning the logits
at the wanted places.  The generation loop, the trace replay program and the
benchmark all drive this function.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..cache import CacheError, KVNeed, SequenceCache
from ..sampling import Sampler, SamplingParams
from .generate import Request, run_generation
from .model import Model
from .step import StepContext, Workspace

Want = Union[None, str, Sequence[Sequence[int]]]


class StepError(ValueError):
    """A step that cannot run: an unknown slot, a token id outside the
    vocabulary, a wanted place outside the step's tokens, a full cache."""


class Engine:
    def __init__(self, model: Model, *, max_tokens: int, max_batch: Optional[int] = None,
                 page_size: int = 64, max_step_tokens: int = 8192, cuda_graphs: bool = True):
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
        # decode steps (one token per sequence, last logits wanted) replay a captured CUDA graph;
        # key: (sequences, page-table widths) -> (graph, private workspace, logits, kernels in the graph)
        self.cuda_graphs = bool(cuda_graphs) and model.graph_safe
        self._graphs: Dict[tuple, tuple] = {}
        self.graph_replays = 0
        self._prepared: Optional[dict] = None             # a decode step laid out ahead of its tokens

    # ---- sequences ------------------------------------------------------------
    def open(self) -> int:
        """Start a sequence; returns its slot."""
        if self.cache.slots.free_count == 0 and self.cache.n_slots < self.total_pages:
            self.cache.grow_slots(min(self.total_pages, max(2 * self.cache.n_slots, 1)))
            self._graphs.clear()                          # the state storage moved
            self._prepared = None
        return self.cache.assign()

    def close(self, slot: int) -> None:
        """The sequence is over; what it holds goes back to the cache."""
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step function -----------------------------------------------------
    def step(self, items: Sequence[Tuple[int, Sequence[int]]], want: Want = "last",
             copy: bool = True) -> Optional[torch.Tensor]:
        """Run ``items`` = [(slot, next tokens), ...] as one batch.

        ``want``: "last" (the last token of every sequence), "all", None, or
        one list of places per item (indices into that item's tokens).
        Returns float32 logits [wanted, vocab] in the order of the items and,
        within an item, of its places; None if nothing is wanted.
        """
        try:
            items = [(int(s), np.asarray(toks, dtype=np.int64).ravel()) for s, toks in items]
        except (TypeError, ValueError):
            raise StepError("token ids must be integers") from None
        V = self.model.vocab_size
        prepared, self._prepared = self._prepared, None
        if (prepared is not None and want == "last" and len(items) == len(prepared["slots"])
                and all(s == ps and len(t) == 1 for (s, t), ps in zip(items, prepared["slots"]))
                and self._graphs.get(prepared["key"]) is not None):
            tokens = [int(t[0]) for _, t in items]
            for (slot, _), t in zip(items, tokens):
                if not 0 <= t < V:
                    raise StepError(f"slot {slot}: token id {t} is outside the vocabulary of {V}")
            logits = self._execute(prepared, tokens)
            return logits.clone() if copy else logits
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
        elif want == "last":
            places = [[len(t) - 1] for _, t in items]
        elif want == "all":
            places = [list(range(len(t))) for _, t in items]
        else:
            places = [[int(i) for i in w] for w in want]
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
                    out[torch.tensor(chunk_dst, device=self.device)] = lg
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
        return self._execute(self._plan(items, places))

    def _plan(self, items, places) -> dict:
        """Everything of a step that the host can work out before the token ids matter: room in the
        cache, positions, page tables, and for a decode-shaped step the arrays laid out for its graph."""
        slots = [s for s, _ in items]
        starts = [self.cache.length(s) for s in slots]
        for s, toks in items:
            self.cache.reserve(s, len(toks))
        out_rows: List[int] = []
        row = 0
        for (_, toks), w in zip(items, places):
            out_rows.extend(row + i for i in w)
            row += len(toks)
        decode = self.cuda_graphs and all(len(t) == 1 for _, t in items) and \
            out_rows == list(range(len(items)))
        # page tables of a decode step are padded to 8 pages so that one graph serves 512 tokens of growth
        widths = {g: -(-max(len(self.cache._get(s).pages[g]) for s in slots) // 8) * 8 if decode else None
                  for g in self.cache.kv_groups}
        page_rows = {g: self.cache.page_rows(g, slots, widths[g]) for g in self.cache.kv_groups}
        plan = dict(slots=slots, starts=starts, lists=[t for _, t in items], out_rows=out_rows,
                    page_rows=page_rows, decode=decode, key=None, ctx=None)
        if decode:
            plan["key"] = (len(items), tuple(sorted(widths.items())))
            entry = self._graphs.get(plan["key"])
            if entry is not None:
                plan["ctx"] = StepContext(slots=slots, starts=starts, token_lists=plan["lists"], out_rows=out_rows,
                                          page_rows=page_rows, dtype=self.dtype, ws=entry[1], upload=False)
        return plan

    def _execute(self, plan: dict, tokens: Optional[List[int]] = None,
                 device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run a planned step.  ``tokens`` replaces the token ids of a decode-shaped plan;
        ``device_tokens`` (int32 [B], on the device) does the same without the host ever seeing them:
        they are copied into the step's token array on the stream, after the other arrays went up."""
        slots, starts, lists = plan["slots"], plan["starts"], plan["lists"]
        if tokens is not None:
            lists = [[t] for t in tokens]

        def context(ws, reuse=None):
            ctx = reuse
            if ctx is None or ctx.ws is not ws:
                ctx = StepContext(slots=slots, starts=starts, token_lists=lists, out_rows=plan["out_rows"],
                                  page_rows=plan["page_rows"], dtype=self.dtype, ws=ws, upload=False)
            ctx.upload(np.concatenate([np.asarray(t).ravel() for t in lists]) if ctx is reuse else None)
            if device_tokens is not None:
                ctx.tokens.copy_(device_tokens, non_blocking=True)
            return ctx

        if not plan["decode"]:
            ctx = context(self.ws)
            logits = self.model.forward(ctx, self.cache)
        else:
            from ..ops import kernels as K
            entry = self._graphs.get(plan["key"])
            if entry is None:
                # first time: run the step for real on a workspace of its own (which sizes every
                # buffer), then record the same launches for the steps to come
                # (the real run also notes which weights the products read, in order; recorded, each
                # product of few rows then asks the L2 cache for its successor's weights)
                from ..ops import linear as L
                gws = Workspace(self.device)
                ctx = context(gws)
                with L.recording() as order:
                    logits = self.model.forward(ctx, self.cache)
                n0 = K.launch_count()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph), L.looking_ahead(order, self.model.weight_extents()):
                    captured = self.model.forward(ctx, self.cache)
                n_kernels = K.launch_count() - n0
                K.add_launches(-n_kernels)                # recorded, not run
                assert captured.data_ptr() == logits.data_ptr()
                self._graphs[plan["key"]] = (graph, gws, logits, n_kernels)
            else:
                graph, gws, logits, n_kernels = entry
                ctx = context(gws, plan["ctx"])
                graph.replay()
                K.add_launches(n_kernels)
                self.graph_replays += 1
        for s, toks in zip(slots, lists):
            self.cache.advance(s, len(toks))
        self.steps_run += 1
        self.h2d_bytes += ctx.h2d_bytes
        return logits

    def decode_from_device(self, slots: Sequence[int], device_tokens: torch.Tensor) -> Optional[torch.Tensor]:
        """One more token for each of ``slots``, the token ids being ``device_tokens`` (int32 [len(slots)],
        on the device, e.g. what the sampling kernel just wrote): the step is enqueued without the host
        waiting for them.  Returns the logits of all, or None if the step cannot run now (no room in the
        cache, the context is full): the caller then waits for the tokens and calls ``step``."""
        self._prepared = None
        slots = [int(s) for s in slots]
        if not slots or len(set(slots)) != len(slots) or device_tokens.numel() != len(slots) \
                or device_tokens.dtype != torch.int32 or not device_tokens.is_cuda:
            return None
        try:
            if self.max_positions is not None and any(self.cache.length(s) + 1 > self.max_positions for s in slots):
                return None
            for g in self.cache.kv_groups:
                need = sum(max(0, -(-(self.cache.length(s) + 1) // self.page_size)
                               - len(self.cache._get(s).pages[g])) for s in slots)
                if need > self.cache.pages[g].free_count:
                    return None
            plan = self._plan([(s, [0]) for s in slots], [[0]] * len(slots))
        except CacheError:
            return None
        return self._execute(plan, device_tokens=device_tokens)

    def prepare_decode(self, slots: Sequence[int]) -> None:
        """Lay out the next step - one more token for each of ``slots``, logits of all - while the GPU
        is still busy with the current one.  ``step`` uses the layout if it is then called with
        exactly these slots and one token each; otherwise the layout is dropped."""
        self._prepared = None
        if not self.cuda_graphs:
            return
        try:
            slots = [int(s) for s in slots]
            if self.max_positions is not None and any(self.cache.length(s) + 1 > self.max_positions for s in slots):
                return
            for g in self.cache.kv_groups:
                need = sum(max(0, -(-(self.cache.length(s) + 1) // self.page_size)
                               - len(self.cache._get(s).pages[g])) for s in slots)
                if need > self.cache.pages[g].free_count:
                    return
            self._prepared = self._plan([(s, [0]) for s in slots], [[0]] * len(slots))
        except CacheError:
            self._prepared = None

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
        go on (it has tokens left to generate).  If a request then turns out to have stopped, its row of the early step is simply
        not used; the other rows do not depend on it.  The next call finds its work already running."""
        sampler, eng = self.sampler, self.engine
        handles = [r.handle for r in requests]
        early = self._early
        self._early = None
        if (early is not None and set(handles) <= set(early["handles"])
                and all(len(t) == 1 and self._last.get(h) == t[0] for h, t in zip(handles, token_lists))):
            rows = [early["handles"].index(h) for h in handles]
            out_dev, host, event = early["out"], early["host"], early["event"]
        else:
            logits = eng.step([(r.handle, t) for r, t in zip(requests, token_lists)], "last", copy=False)
            out_dev = sampler.launch(logits, [r.index for r in requests], [len(r.output) for r in requests],
                                     [r.output for r in requests], states=handles)
            host, event = sampler.read_async(out_dev)
            rows = list(range(len(requests)))
        # the step after this one, for the requests that will still have tokens to generate
        if eng.cuda_graphs:
            goers = [(i, r) for i, r in zip(rows, requests) if len(r.output) + 2 <= r.max_new_tokens]
            if goers and len(goers) == len([r for r in requests if len(r.output) + 1 < r.max_new_tokens]):
                src = out_dev if [i for i, _ in goers] == list(range(out_dev.numel())) else \
                    out_dev[torch.tensor([i for i, _ in goers], device=out_dev.device)]
                nxt = eng.decode_from_device([r.handle for _, r in goers], src)
                if nxt is not None:
                    out2 = sampler.launch(nxt, [r.index for _, r in goers], [len(r.output) + 1 for _, r in goers],
                                          [[] for _ in goers], slot=1 - early["slot"] if early else 1,
                                          states=[r.handle for _, r in goers])
                    host2, event2 = sampler.read_async(out2, slot=1 - early["slot"] if early else 1)
                    self._early = dict(handles=[r.handle for _, r in goers], out=out2, host=host2, event=event2,
                                       slot=1 - early["slot"] if early else 1)
        else:
            eng.prepare_decode(handles)
        event.synchronize()
        tokens = host.tolist()
        result = [tokens[i] for i in rows]
        self._last = dict(zip(handles, result))
        return result
