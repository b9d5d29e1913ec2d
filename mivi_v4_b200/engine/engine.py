"""The engine: a model, its cache, the step function, and generation on top.

``step`` is the one function that runs the model: a batch of sequences with
unequal numbers of next tokens - whole prompts, then one token each, or any
cut in between - from the cache that earlier steps left, returning the logits
at the wanted places.  The generation loop, the trace replay program and the
benchmark all drive this function.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple, Union

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
        self.cuda_graphs = bool(cuda_graphs)
        self._graphs: Dict[tuple, tuple] = {}
        self.graph_replays = 0

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

    # ---- the step function -----------------------------------------------------
    def step(self, items: Sequence[Tuple[int, Sequence[int]]], want: Want = "last",
             copy: bool = True) -> Optional[torch.Tensor]:
        """Run ``items`` = [(slot, next tokens), ...] as one batch.

        ``want``: "last" (the last token of every sequence), "all", None, or
        one list of places per item (indices into that item's tokens).
        Returns float32 logits [wanted, vocab] in the order of the items and,
        within an item, of its places; None if nothing is wanted.
        """
        items = [(int(s), [int(t) for t in toks]) for s, toks in items]
        V = self.model.vocab_size
        seen = set()
        for slot, toks in items:
            if slot in seen:
                raise StepError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if not toks:
                raise StepError(f"slot {slot} brings no tokens")
            bad = [t for t in toks if not 0 <= t < V]
            if bad:
                raise StepError(f"slot {slot}: token id {bad[0]} is outside the vocabulary of {V}")
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
        lists = [t for _, t in items]
        if not decode:
            ctx = StepContext(slots=slots, starts=starts, token_lists=lists, out_rows=out_rows,
                              page_rows=page_rows, dtype=self.dtype, ws=self.ws)
            logits = self.model.forward(ctx, self.cache)
        else:
            key = (len(items), tuple(sorted(widths.items())))
            entry = self._graphs.get(key)
            if entry is None:
                # first time: run the step for real on a workspace of its own (which sizes every
                # buffer), then record the same launches for the steps to come
                gws = Workspace(self.device)
                ctx = StepContext(slots=slots, starts=starts, token_lists=lists, out_rows=out_rows,
                                  page_rows=page_rows, dtype=self.dtype, ws=gws)
                logits = self.model.forward(ctx, self.cache)
                from ..ops import kernels as K
                n0 = K.launch_count()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    captured = self.model.forward(ctx, self.cache)
                n_kernels = K.launch_count() - n0
                K.add_launches(-n_kernels)                # recorded, not run
                assert captured.data_ptr() == logits.data_ptr()
                self._graphs[key] = (graph, gws, logits, n_kernels)
            else:
                graph, gws, logits, n_kernels = entry
                ctx = StepContext(slots=slots, starts=starts, token_lists=lists, out_rows=out_rows,
                                  page_rows=page_rows, dtype=self.dtype, ws=gws)
                graph.replay()
                from ..ops import kernels as K
                K.add_launches(n_kernels)
                self.graph_replays += 1
        for s, toks in items:
            self.cache.advance(s, len(toks))
        self.steps_run += 1
        self.h2d_bytes += ctx.h2d_bytes
        return logits

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

    def open(self) -> int:
        return self.engine.open()

    def close(self, handle: int) -> None:
        self.engine.close(handle)

    def forward_and_sample(self, requests: Sequence[Request], token_lists) -> List[int]:
        logits = self.engine.step([(r.handle, t) for r, t in zip(requests, token_lists)], "last", copy=False)
        return self.sampler.sample(logits, [r.index for r in requests], [len(r.output) for r in requests],
                                   [r.output for r in requests])
