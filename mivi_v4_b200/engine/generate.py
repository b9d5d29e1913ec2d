"""The generation loop: which requests form a batch, when a sequence ends, when
its slot goes back, when the next batch starts.  It decides; a backend does
the work (the engine on the device, or a scripted stand-in in tests).

The reference's loop serves one sequence (crates/mivi-model/src/model.rs:
1131-1230): sample from the last logits; a stop token ends the sequence and is
not emitted (1166-1173); else emit, and run the token through the model; stop
at max_tokens or at the end of the context (1135-1137).  Not taken over: the
suppression of end tokens at step 0 and text stop strings (chat heuristics),
and the forward pass of a token after which nothing is sampled (1227).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Protocol, Sequence


@dataclass
class Request:
    index: int                      # place in the caller's list; also its random stream
    prompt: List[int]
    max_new_tokens: int
    output: List[int] = field(default_factory=list)
    handle: Optional[int] = None
    finish_reason: Optional[str] = None    # "stop", "length", "context"


class Backend(Protocol):
    max_batch: int
    page_size: int
    total_pages: int
    max_positions: Optional[int]

    def open(self) -> int: ...
    def close(self, handle: int) -> None: ...
    def forward_and_sample(self, requests: Sequence[Request], token_lists: Sequence[List[int]]) -> List[int]: ...


class GenerationError(RuntimeError):
    pass


def pages_for(n_tokens: int, page_size: int) -> int:
    return -(-n_tokens // page_size)


def plan_batches(requests: Sequence[Request], max_batch: int, total_pages: int, page_size: int) -> List[List[Request]]:
    """Requests in order, cut into batches that the cache can carry to the end:
    a batch holds at most ``max_batch`` sequences, and the pages that its
    sequences can grow to (prompt plus all new tokens) fit the pool."""
    batches: List[List[Request]] = []
    cur: List[Request] = []
    used = 0
    for r in requests:
        need = pages_for(len(r.prompt) + r.max_new_tokens, page_size)
        if need > total_pages:
            raise GenerationError(
                f"request {r.index}: {len(r.prompt)} prompt tokens + {r.max_new_tokens} new tokens need "
                f"{need} pages of {page_size}; the cache has {total_pages}")
        if cur and (len(cur) >= max_batch or used + need > total_pages):
            batches.append(cur)
            cur, used = [], 0
        cur.append(r)
        used += need
    if cur:
        batches.append(cur)
    return batches


def run_batch(batch: List[Request], backend: Backend, stop_ids: Sequence[int],
              on_token: Optional[Callable[[int, int], None]] = None) -> None:
    """Prompts in one step, then one token each; a sequence that ends leaves the
    batch and gives its slot back at once."""
    stop = set(int(s) for s in stop_ids)
    live = [r for r in batch]
    for r in live:
        if not r.prompt:
            raise GenerationError(f"request {r.index} has an empty prompt")
        r.handle = backend.open()
    feed = [list(r.prompt) for r in live]
    lengths = {r.index: len(r.prompt) for r in live}
    try:
        while live:
            done_now = [r for r in live if r.max_new_tokens <= len(r.output)]
            for r in done_now:                          # max_new_tokens == 0: nothing to sample
                r.finish_reason = "length"
            if done_now:
                keep = [i for i, r in enumerate(live) if r not in done_now]
                for r in done_now:
                    backend.close(r.handle)
                    r.handle = None
                live, feed = [live[i] for i in keep], [feed[i] for i in keep]
                if not live:
                    break
            sampled = backend.forward_and_sample(live, feed)
            nxt_live, nxt_feed = [], []
            for r, tok in zip(live, sampled):
                tok = int(tok)
                if backend.max_positions is not None and lengths[r.index] >= backend.max_positions:
                    # the context is full: like the reference (model.rs:1135-1137) nothing more is sampled
                    r.finish_reason = "context"
                elif tok in stop:
                    r.finish_reason = "stop"
                else:
                    r.output.append(tok)
                    if on_token is not None:
                        on_token(r.index, tok)
                    if len(r.output) >= r.max_new_tokens:
                        r.finish_reason = "length"
                if r.finish_reason is None:
                    lengths[r.index] += 1
                    nxt_live.append(r)
                    nxt_feed.append([tok])
                else:
                    backend.close(r.handle)
                    r.handle = None
            live, feed = nxt_live, nxt_feed
    finally:
        for r in batch:
            if r.handle is not None:
                backend.close(r.handle)
                r.handle = None


def run_generation(prompts: Sequence[Sequence[int]], max_new_tokens, backend: Backend,
                   stop_ids: Sequence[int] = (), on_token=None) -> List[Request]:
    """Generate for every prompt, as many batches one after another as it takes."""
    if isinstance(max_new_tokens, int):
        max_new_tokens = [max_new_tokens] * len(prompts)
    if len(max_new_tokens) != len(prompts):
        raise GenerationError("max_new_tokens must be one number or one per prompt")
    requests = [Request(i, [int(t) for t in p], int(m)) for i, (p, m) in enumerate(zip(prompts, max_new_tokens))]
    for r in requests:
        if r.max_new_tokens < 0:
            raise GenerationError(f"request {r.index}: max_new_tokens is negative")
        if backend.max_positions is not None and len(r.prompt) > backend.max_positions:
            raise GenerationError(f"request {r.index}: the prompt has {len(r.prompt)} tokens, the context "
                                  f"holds {backend.max_positions}")
    for batch in plan_batches(requests, backend.max_batch, backend.total_pages, backend.page_size):
        run_batch(batch, backend, stop_ids, on_token)
    return requests
