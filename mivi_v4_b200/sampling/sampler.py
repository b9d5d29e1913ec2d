"""Device-side sampling for a batch of rows of logits."""
from __future__ import annotations

import time
from typing import List, Optional, Sequence

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
        self._bufs = {}
        self._pinned = {}
        self._events = {}
        self._done = {}
        self._ring = None             # recent tokens kept on the device: int32 [states, 128]
        self._with_flag = {}          # buffer set -> rows of the launch whose output carries the error flag behind them
        # the sampled tokens go to the host on a stream of their own: the step after this one does not
        # wait behind the copy
        self._copy_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        from ..engine.step import Workspace
        self._ws = Workspace(self.device)

    def launch(self, logits: torch.Tensor, streams: Sequence[int], steps: Sequence[int],
               recent: Sequence[Sequence[int]], slot: int = 0,
               states: Optional[Sequence[int]] = None, carry_flag: bool = False) -> torch.Tensor:
        """Enqueue the sampling kernel; returns the device tensor (int32 [B]) that will hold the
        tokens.  ``slot`` (0 or 1) picks one of two sets of buffers, so that two launches can be in
        flight.  ``states``: a small integer per row that stays with its sequence (the engine's slot);
        with it the recent tokens that the penalties look at are kept on the device, in a ring per
        state that the kernel itself appends to, and ``recent`` is not used: a step can then be
        enqueued before the host knows the token of the step before it.  ``carry_flag``: the kernel
        copies the device's error flag behind the tokens; ``read_async`` brings it to the host with
        them and ``flag(slot)`` reads it there."""
        B, V = logits.shape
        p = self.params
        bufs = self._bufs.get(slot)
        if bufs is None or bufs[0].shape[0] < B:
            bufs = (torch.empty((max(B, 1), K.sample_scratch_width(V)), dtype=torch.float32, device=self.device),
                    torch.zeros((max(B, 1) + 1,), dtype=torch.int32, device=self.device))
            self._bufs[slot] = bufs
        work, out_all = bufs
        on_device = states is not None and p.uses_penalties
        use_pen = p.uses_penalties and not on_device and any(len(r) for r in recent)
        out = out_all[:B]
        ring = rows_d = None
        if on_device:
            need = max(int(x) for x in states) + 1
            if self._ring is None or self._ring.shape[0] < need:
                grown = torch.zeros((max(need, 2 * (0 if self._ring is None else self._ring.shape[0]), 8),
                                     K.RECENT_RING), dtype=torch.int32, device=self.device)
                if self._ring is not None:
                    grown[:self._ring.shape[0]] = self._ring
                self._ring = grown
            ring = self._ring
        if p.temperature <= 0.0 and not use_pen and not on_device:
            # the largest logit: no draw, so no stream and step numbers to send up
            streams_d = steps_d = n_recent_d = recent_d = None
        else:
            meta: List[int] = [int(s) & 0x7fffffff for s in streams] + [int(s) for s in steps]
            if on_device:
                meta += [int(x) for x in states]
            if use_pen:
                meta += [min(len(r), RECENT_TOKENS_WINDOW) for r in recent]
                for r in recent:
                    r = list(r)[-RECENT_TOKENS_WINDOW:]
                    meta += r + [0] * (RECENT_TOKENS_WINDOW - len(r))
            m = self._ws.stage(f"sample_meta{slot}", meta)
            streams_d, steps_d = m[:B], m[B:2 * B]
            rows_d = m[2 * B:3 * B] if on_device else None
            n_recent_d = m[2 * B:3 * B] if use_pen else None
            recent_d = m[3 * B:].view(B, RECENT_TOKENS_WINDOW) if use_pen else None
        K.sample(logits, work, out, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p,
                 min_p=p.min_p, repetition_penalty=p.repetition_penalty, presence_penalty=p.presence_penalty,
                 frequency_penalty=p.frequency_penalty, recent=recent_d, n_recent=n_recent_d, seed=self.seed,
                 streams=streams_d, steps=steps_d, ring=ring, ring_rows=rows_d,
                 flag_to=out_all[B:B + 1] if carry_flag else None)
        self._with_flag[slot] = B if carry_flag else None
        return out

    def read_async(self, out: torch.Tensor, slot: int = 0):
        """Start the copy of sampled tokens to pinned host memory; returns (host tensor, event).  The
        tokens are there once the event has completed, whatever was enqueued after it."""
        B = out.numel()
        pinned = self._pinned.get(slot)
        if pinned is None or pinned.numel() < B + 1:
            pinned = torch.zeros(max(B + 1, 64), dtype=torch.int32).pin_memory()
            self._pinned[slot] = pinned
        if self._with_flag.get(slot) == B:
            # the flag lies behind the tokens in the same buffer: one copy brings both
            out = self._bufs[slot][1][:B + 1]
            host_all = pinned[:B + 1]
        else:
            host_all = pinned[:B]
            pinned[B] = 0
        host = host_all[:B]
        event = self._events.setdefault(slot, torch.cuda.Event())
        if self._copy_stream is None:
            host_all.copy_(out, non_blocking=True)
            event.record()
            return host, event
        done = self._done.setdefault(slot, torch.cuda.Event())
        done.record()                                   # the sampling kernel, on the launching stream
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(done)
            host_all.copy_(out, non_blocking=True)
            event.record()
        return host, event

    def flag(self, slot: int = 0) -> int:
        """The device's error flag as the launch of ``slot`` saw it, once its copy has arrived (0 if that
        launch did not carry it)."""
        pinned = self._pinned.get(slot)
        n = self._with_flag.get(slot)
        return int(pinned[n]) if pinned is not None and n is not None else 0

    def sample(self, logits: torch.Tensor, streams: Sequence[int], steps: Sequence[int],
               recent: Sequence[Sequence[int]], before_sync=None) -> List[int]:
        """One token per row, on the host.  ``before_sync`` is called after the kernel is launched
        and before the host waits for the tokens, for host work that can overlap with the GPU."""
        out = self.launch(logits, streams, steps, recent)
        host, event = self.read_async(out)
        if before_sync is not None:
            before_sync()
        event.synchronize()
        return host.tolist()
