"""Device-side sampling for a batch of rows of logits."""
from __future__ import annotations

import time
from typing import List, Sequence

import torch

from ..ops import kernels as K
from .params import RECENT_TOKENS_WINDOW, SamplingParams


class Sampler:
    """Draws one token per row.  Row i belongs to random stream ``streams[i]``
    and is that stream's ``steps[i]``-th draw; the result for a row does not
    depend on which other rows are in the batch."""

    def __init__(self, params: SamplingParams, vocab: int, device):
        self.params = params.validate()
        self.vocab = vocab
        self.device = torch.device(device)
        seed = params.seed
        if seed is None:
            seed = time.time_ns()
        self.seed = int(seed) & ((1 << 64) - 1)
        self._work = None
        self._out = None
        from ..engine.step import Workspace
        self._ws = Workspace(self.device)

    def sample(self, logits: torch.Tensor, streams: Sequence[int], steps: Sequence[int],
               recent: Sequence[Sequence[int]]) -> List[int]:
        B, V = logits.shape
        p = self.params
        if self._work is None or self._work.shape[0] < B:
            self._work = torch.empty((max(B, 1), V), dtype=torch.float32, device=self.device)
            self._out = torch.empty((max(B, 1),), dtype=torch.int32, device=self.device)
        meta: List[int] = [int(s) & 0x7fffffff for s in streams] + [int(s) for s in steps]
        use_pen = p.uses_penalties and any(len(r) for r in recent)
        if use_pen:
            meta += [min(len(r), RECENT_TOKENS_WINDOW) for r in recent]
            for r in recent:
                r = list(r)[-RECENT_TOKENS_WINDOW:]
                meta += r + [0] * (RECENT_TOKENS_WINDOW - len(r))
        m = self._ws.stage("sample_meta", meta)
        streams_d, steps_d = m[:B], m[B:2 * B]
        n_recent_d = m[2 * B:3 * B] if use_pen else None
        recent_d = m[3 * B:].view(B, RECENT_TOKENS_WINDOW) if use_pen else None
        out = self._out[:B]
        K.sample(logits, self._work, out, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p,
                 min_p=p.min_p, repetition_penalty=p.repetition_penalty, presence_penalty=p.presence_penalty,
                 frequency_penalty=p.frequency_penalty, recent=recent_d, n_recent=n_recent_d, seed=self.seed,
                 streams=streams_d, steps=steps_d)
        return out.tolist()
