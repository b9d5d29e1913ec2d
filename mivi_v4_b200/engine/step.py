"""One step's batch as the kernels see it: the packed tokens of all sequences
and the small integer arrays that say which token belongs where.

The reference's step is one token of one sequence at one position
(crates/mivi-model/src/model.rs:336-433) or a tile of consecutive tokens of
that sequence (model.rs:670-831).  Here a step is any number of sequences,
each with any number of next tokens, packed without padding: padding never
enters a kernel, so it cannot change a result.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


class Workspace:
    """Named device buffers that live as long as the engine and grow on demand,
    so that steps allocate nothing once sizes have been seen."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        # the views handed out, by (name, dtype, shape): a step asks for the same ones layer after layer
        self._views: Dict[tuple, torch.Tensor] = {}
        # counts the allocations: launches recorded while it had one value name addresses that are
        # still the buffers' addresses for as long as it keeps that value
        self.generation = 0

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        vkey = (name, dtype, tuple(shape))
        view = self._views.get(vkey)
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self.generation += 1
            for k in [k for k in self._views if k[0] == name and k[1] == dtype]:
                del self._views[k]                # views of the buffer that was replaced
        if len(self._views) > 4096:
            self._views.clear()
        view = buf[:n].view(*shape)
        self._views[vkey] = view
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())

    def get_zeroed(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """Like ``get``, but the buffer is zero when it is first handed out (and
        after it had to grow).  For scratch that its kernels leave zeroed."""
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self.generation += 1
            for k in [k for k in self._views if k[0] == name and k[1] == dtype]:
                del self._views[k]
        return buf[:n].view(*shape)

    def stage(self, name: str, values) -> torch.Tensor:
        """Copy integers (a list or a numpy array) to the device buffer ``name``
        (int32) through pinned host memory, one asynchronous copy.  A small ring
        of pinned buffers is reused; a buffer is taken again only after the copy
        that last read it has run."""
        n = len(values)
        dst = self.get(name, (n,), torch.int32)
        if self.device.type != "cuda":
            dst.copy_(torch.from_numpy(np.asarray(values, dtype=np.int32)))
            return dst
        ring = self.__dict__.setdefault("_ring", [])
        if not ring:
            ring.extend([None, None, None, None])
            self._ring_at = 0
        i = self._ring_at
        self._ring_at = (i + 1) % len(ring)
        slot = ring[i]
        if slot is None or slot[0].numel() < n:
            slot = (torch.empty(max(n, 256), dtype=torch.int32).pin_memory(), torch.cuda.Event())
            ring[i] = slot
        else:
            slot[1].synchronize()
        host, event = slot
        host.numpy()[:n] = values
        dst.copy_(host[:n], non_blocking=True)
        event.record()
        return dst


# Steps in which the products around a norm may carry it: every bfloat16 step; which products can is
# theirs to say (``ops.linear.norm_link_ok``: every tensor-core kernel applies a carried norm's scale, the
# weight-streaming kernels, which steps of up to about a thousand tokens use, also emit one).  Measured on
# the 1.2B-parameter shape: 0.85 -> 0.79 ms a step at 8 tokens.


class StepContext:
    """Host and device view of one step.

    Device arrays (int32): tokens[N], positions[N] (absolute position of each
    token in its sequence), seq_of[N] (index of its sequence in this step),
    cu[B+1] (first packed row of each sequence), slots[B], starts[B] (length of
    each sequence before the step), lens[B] (tokens it brings), out_rows[n_out]
    (packed rows whose logits are wanted), page_tables[group] [B, P].
    """

    def __init__(self, *, slots: List[int], starts: List[int], token_lists: List[List[int]],
                 out_rows: List[int], page_rows: Dict[int, List[List[int]]], dtype: torch.dtype,
                 ws: Workspace, upload: bool = True):
        device = ws.device
        self.ws, self.dtype, self.device = ws, dtype, device
        self.host_slots, self.host_starts = list(slots), list(starts)
        self.host_lens = [len(t) for t in token_lists]
        self.n_seqs = len(slots)
        self.n_tokens = sum(self.host_lens)
        self.n_out = len(out_rows)
        self.out_rows_all = list(out_rows) == list(range(self.n_tokens))     # every row's logits, in order
        self.is_decode = all(n == 1 for n in self.host_lens)
        self.max_len = max(self.host_lens, default=0)
        self.max_context = max((s + n for s, n in zip(starts, self.host_lens)), default=0)
        # steps of few tokens in bfloat16 let the products around a norm carry it (MIVI_CARRY_NORMS=0: never)
        self.carry_norms = (dtype == torch.bfloat16 and self.n_tokens >= 1
                            and os.environ.get("MIVI_CARRY_NORMS", "1") != "0")
        self._link = None

        parts: List[np.ndarray] = []
        spans: Dict[str, Tuple[int, int]] = {}
        total = 0

        def put(name: str, values) -> None:
            nonlocal total
            arr = np.asarray(values, dtype=np.int32).ravel()
            spans[name] = (total, arr.size)
            pad = -arr.size % 4                           # 16-byte starts
            parts.append(arr)
            if pad:
                parts.append(np.zeros(pad, dtype=np.int32))
            total += arr.size + pad

        lens = np.asarray(self.host_lens, dtype=np.int64)
        starts_a = np.asarray(starts, dtype=np.int64)
        cu = np.zeros(self.n_seqs + 1, dtype=np.int64)
        np.cumsum(lens, out=cu[1:])
        seq_of = np.repeat(np.arange(self.n_seqs, dtype=np.int64), lens)
        # position of a packed row = start of its sequence + its place in the sequence's run
        positions = np.arange(self.n_tokens, dtype=np.int64) - cu[:-1][seq_of] + starts_a[seq_of] if self.n_tokens \
            else np.zeros(0, dtype=np.int64)
        tokens = np.concatenate([np.asarray(t, dtype=np.int64).ravel() for t in token_lists]) if token_lists \
            else np.zeros(0, dtype=np.int64)
        put("tokens", tokens)
        put("positions", positions)
        put("seq_of", seq_of)
        put("cu", cu)
        put("slots", list(slots))
        put("starts", starts_a)
        put("lens", lens)
        put("out_rows", list(out_rows))
        widths: Dict[int, int] = {}
        for g, rows in page_rows.items():
            widths[g] = len(rows[0]) if rows else 1
            put(f"pages{g}", rows if rows else [])
        flat = np.concatenate(parts) if parts else np.zeros(0, dtype=np.int32)
        # the arrays live in one device buffer whose place depends only on the workspace; they are
        # filled by upload(), which may come later (a step can be laid out before its tokens are known)
        arena = ws.get("step_meta", (len(flat),), torch.int32)
        self._flat = flat
        self.spans = spans                                   # name -> (first element, elements) in the arena
        self.h2d_bytes = len(flat) * 4

        def view(name: str) -> torch.Tensor:
            o, n = spans[name]
            return arena[o:o + n]

        self.tokens, self.positions, self.seq_of = view("tokens"), view("positions"), view("seq_of")
        self.cu, self.slots, self.starts, self.lens = view("cu"), view("slots"), view("starts"), view("lens")
        self.out_rows: Optional[torch.Tensor] = view("out_rows") if self.n_out else None
        if upload:
            self.upload()
        self.page_tables: Dict[int, torch.Tensor] = {
            g: view(f"pages{g}").view(max(self.n_seqs, 1) if rows else 1, widths[g]) if rows else view(f"pages{g}")
            for g, rows in page_rows.items()}

    def leave_link(self, link) -> None:
        """A block's last product has written the rows of the next block's first norm (or None)."""
        self._link = link

    def take_link(self, norm):
        """The link left for this norm part, if the block before left one."""
        link, self._link = self._link, None
        return link if link is not None and link.norm is norm else None

    def upload(self, tokens: Optional[List[int]] = None) -> None:
        """One host-to-device copy of the step's arrays; ``tokens`` replaces the token ids first."""
        if tokens is not None:
            if len(tokens) != self.n_tokens:
                raise ValueError(f"{len(tokens)} token ids for a step of {self.n_tokens} tokens")
            self._flat[:self.n_tokens] = tokens
        self.ws.stage("step_meta", self._flat)
