"""The cache of a running batch: a slot for each sequence with its own length,
keys and values in pages for the layers that keep them, state of fixed size
for the layers that keep that.

Layers with the same need form a group with storage of its own:
  * a KV group: pool[layer, page, 2 (K, V), kv head, row, head_dim] in the
    model's dtype, pages of ``page_size`` tokens handed out on demand; a group
    with a window gives pages back as they fall out of it;
  * a state group: state[layer, slot, ...] in the need's dtype (float32 unless it
    says otherwise), zeroed when the slot is assigned.
The reference allocates keys and values only for its attention layers through
a layer map (crates/mivi-kv/src/cache.rs:109-141) and keeps the convolution
state per layer in its run state (crates/mivi-core/src/arena.rs:56,82,105);
both have one sequence.  Slots, pages and groups are this library's own.

All bookkeeping is on the host; only the storage lives on the device.  Nothing
here launches a kernel except zeroing a slot's state.  Beside the page lists of
each sequence the cache keeps the same facts as arrays over all slots (lengths,
page tables), so that a decode step of many sequences reads and advances them
without a loop over the sequences.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .allocator import CacheError, IndexPool
from .needs import KVNeed, StateNeed

Need = Union[KVNeed, StateNeed, None]


@dataclass
class GroupPlan:
    need: Union[KVNeed, StateNeed]
    n_layers: int = 0


@dataclass
class CachePlan:
    """Which group and which layer of it each position of the schedule uses."""
    groups: List[GroupPlan]
    binding: List[Optional[Tuple[int, int]]]      # schedule position -> (group, layer in group) of its first need, or None
    owner: List[bool]                             # False: the position reads another position's cache
    bindings: List[List[Tuple[int, int]]]         # schedule position -> (group, layer in group) of each of its needs
    several: List[bool]                           # the position gave a list of needs and gets a list of views


def plan_cache(needs: Sequence[Union[Need, Sequence[Need]]], cache_of: Sequence[Optional[int]]) -> CachePlan:
    """Layers with equal needs share a group.  A position's need is one need, None, or a list of needs."""
    groups: List[GroupPlan] = []
    index: Dict[Need, int] = {}
    bindings: List[List[Tuple[int, int]]] = []
    owner: List[bool] = []
    several: List[bool] = []
    for pos, (need, src) in enumerate(zip(needs, cache_of)):
        is_list = isinstance(need, (list, tuple))
        wanted = [n for n in need if n is not None] if is_list else ([] if need is None else [need])
        several.append(is_list)
        if src is not None:
            if not (0 <= src < pos):
                raise CacheError(f"schedule position {pos} reads the cache of position {src}, "
                                 f"which is not an earlier position")
            if not bindings[src] or not owner[src]:
                raise CacheError(f"schedule position {pos} reads the cache of position {src}, "
                                 f"which keeps none of its own")
            kept = [groups[g].need for g, _ in bindings[src]]
            if kept != wanted:
                raise CacheError(f"schedule position {pos} needs {need} but position {src} keeps "
                                 f"{kept[0] if len(kept) == 1 else kept}")
            bindings.append(list(bindings[src]))
            owner.append(False)
            continue
        mine = []
        for n in wanted:
            if n not in index:
                index[n] = len(groups)
                groups.append(GroupPlan(n))
            g = index[n]
            mine.append((g, groups[g].n_layers))
            groups[g].n_layers += 1
        bindings.append(mine)
        owner.append(True)
    return CachePlan(groups, [b[0] if b else None for b in bindings], owner, bindings, several)


@dataclass
class KVView:
    """What an attention-like mixer gets: its layer's pool, and the page table
    of the step's sequences (device int32 [B, P])."""
    pool: torch.Tensor                 # [pages, 2, kv heads, page_size, head_dim]
    page_table: torch.Tensor
    page_size: int
    writable: bool
    need: KVNeed


@dataclass
class StateView:
    """What a mixer with fixed-size state gets: state[slot, ...] of its layer;
    the step's slots are in the step context."""
    state: torch.Tensor
    writable: bool
    need: StateNeed


class _Slot:
    __slots__ = ("pages",)

    def __init__(self, n_groups: int):
        # per KV group: page of each page-sized block of the sequence (None once given back)
        self.pages: List[List[Optional[int]]] = [[] for _ in range(n_groups)]


class SequenceCache:
    def __init__(self, plan: CachePlan, *, n_slots: int, n_pages: int, page_size: int = 64,
                 dtype: torch.dtype = torch.bfloat16, device: Union[str, torch.device] = "cuda"):
        if page_size < 1 or page_size & (page_size - 1):
            raise CacheError(f"page size {page_size} is not a power of two")
        self.plan = plan
        self.page_size = page_size
        self.dtype = dtype
        self.device = torch.device(device)
        self.slots = IndexPool(n_slots, "slot")
        self._seq: Dict[int, _Slot] = {}
        self.n_pages = n_pages
        self.kv_groups: List[int] = [i for i, g in enumerate(plan.groups) if isinstance(g.need, KVNeed)]
        self.state_groups: List[int] = [i for i, g in enumerate(plan.groups) if isinstance(g.need, StateNeed)]
        self.pages: Dict[int, IndexPool] = {g: IndexPool(n_pages, "page") for g in self.kv_groups}
        self.windowed: List[int] = [g for g in self.kv_groups if plan.groups[g].need.window > 0]
        # the same bookkeeping as arrays over all slots: length, assigned or not, blocks that have a page
        # entry, and per KV group the page of each block (0 where there is none)
        self._len = np.zeros(max(n_slots, 1), dtype=np.int64)
        self._assigned = np.zeros(max(n_slots, 1), dtype=bool)
        self._nblk = np.zeros(max(n_slots, 1), dtype=np.int64)
        self._table: Dict[int, np.ndarray] = {g: np.zeros((max(n_slots, 1), 8), dtype=np.int32) for g in self.kv_groups}
        self.storage: Dict[int, torch.Tensor] = {}
        for gi, g in enumerate(plan.groups):
            if isinstance(g.need, KVNeed):
                shape = (g.n_layers, max(n_pages, 1), 2, g.need.n_kv_heads, page_size, g.need.head_dim)
                self.storage[gi] = torch.zeros(shape, dtype=dtype, device=self.device)
            else:
                shape = (g.n_layers, max(n_slots, 1)) + tuple(g.need.shape)
                self.storage[gi] = torch.zeros(shape, dtype=g.need.dtype, device=self.device)

    # ---- sizes ------------------------------------------------------------
    @property
    def n_slots(self) -> int:
        return self.slots.n

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.storage.values())

    def grow_slots(self, n_slots: int) -> None:
        """More sequences than planned: widen the per-slot state storage."""
        if n_slots <= self.slots.n:
            return
        for gi in self.state_groups:
            old = self.storage[gi]
            new = torch.zeros((old.shape[0], n_slots) + tuple(old.shape[2:]), dtype=old.dtype, device=old.device)
            new[:, :old.shape[1]] = old
            self.storage[gi] = new
        add = n_slots - self._len.shape[0]
        if add > 0:
            self._len = np.concatenate([self._len, np.zeros(add, dtype=np.int64)])
            self._assigned = np.concatenate([self._assigned, np.zeros(add, dtype=bool)])
            self._nblk = np.concatenate([self._nblk, np.zeros(add, dtype=np.int64)])
            for g, t in self._table.items():
                self._table[g] = np.concatenate([t, np.zeros((add, t.shape[1]), dtype=np.int32)])
        self.slots.grow(n_slots)

    # ---- slots --------------------------------------------------------------
    def assign(self) -> int:
        """A fresh sequence: a slot of length 0 with zeroed state."""
        s = self.slots.take()
        self._seq[s] = _Slot(len(self.plan.groups))
        self._len[s], self._nblk[s], self._assigned[s] = 0, 0, True
        for t in self._table.values():
            t[s] = 0
        for gi in self.state_groups:
            self.storage[gi][:, s].zero_()
        return s

    def release(self, slot: int) -> None:
        """The sequence is over: its pages and its slot go back."""
        seq = self._seq.get(slot)
        if seq is None:
            raise CacheError(f"slot {slot} is released but is not assigned")
        for gi in self.kv_groups:
            for p in seq.pages[gi]:
                if p is not None:
                    self.pages[gi].give(p)
        del self._seq[slot]
        self._len[slot], self._nblk[slot], self._assigned[slot] = 0, 0, False
        self.slots.give(slot)

    def length(self, slot: int) -> int:
        self._get(slot)
        return int(self._len[slot])

    def active_slots(self) -> List[int]:
        return sorted(self._seq)

    def _get(self, slot: int) -> _Slot:
        seq = self._seq.get(slot)
        if seq is None:
            raise CacheError(f"slot {slot} is not assigned")
        return seq

    # ---- growth ---------------------------------------------------------------
    def pages_needed(self, slot: int, n_tokens: int) -> int:
        """Most pages that any KV group must add for ``n_tokens`` more tokens."""
        seq = self._get(slot)
        blocks = -(-(int(self._len[slot]) + n_tokens) // self.page_size)
        return max((blocks - len(seq.pages[gi]) for gi in self.kv_groups), default=0)

    def reserve(self, slot: int, n_tokens: int) -> None:
        """Make room for ``n_tokens`` more tokens of this sequence in every KV
        group.  Takes all pages or none."""
        seq = self._get(slot)
        length = int(self._len[slot])
        blocks = -(-(length + n_tokens) // self.page_size)
        for gi in self.kv_groups:
            want = blocks - len(seq.pages[gi])
            if want > self.pages[gi].free_count:
                raise CacheError(
                    f"the cache is full: slot {slot} needs {want} more page(s) of {self.page_size} tokens "
                    f"for {length}+{n_tokens} tokens, {self.pages[gi].free_count} of "
                    f"{self.n_pages} are free")
        for gi in self.kv_groups:
            table = self._table[gi]
            if blocks > table.shape[1]:
                table = np.concatenate([table, np.zeros((table.shape[0], max(blocks, 2 * table.shape[1]) - table.shape[1]),
                                                        dtype=np.int32)], axis=1)
                self._table[gi] = table
            while len(seq.pages[gi]) < blocks:
                page = self.pages[gi].take()
                table[slot, len(seq.pages[gi])] = page
                seq.pages[gi].append(page)
        if self.kv_groups:
            self._nblk[slot] = blocks

    def advance(self, slot: int, n_tokens: int) -> None:
        """The step's kernels are enqueued: the sequence is ``n_tokens`` longer.
        Groups with a window give back the pages that no later token reads."""
        seq = self._get(slot)
        self._len[slot] += n_tokens
        self._give_back(slot, seq)

    def _give_back(self, slot: int, seq: _Slot) -> None:
        length = int(self._len[slot])
        for gi in self.windowed:
            window = self.plan.groups[gi].need.window
            first_needed = max(0, length - window + 1)     # the next token reads keys from here on
            for blk in range(min(first_needed // self.page_size, len(seq.pages[gi]))):
                if seq.pages[gi][blk] is not None:
                    self.pages[gi].give(seq.pages[gi][blk])
                    seq.pages[gi][blk] = None
                    self._table[gi][slot, blk] = 0

    # ---- the same for many sequences at once (arrays of slots) ---------------------------
    def are_assigned(self, slots: np.ndarray) -> bool:
        return bool(slots.size) and 0 <= int(slots.min()) and int(slots.max()) < self._assigned.shape[0] \
            and bool(self._assigned[slots].all())

    def lengths_of(self, slots: np.ndarray) -> np.ndarray:
        return self._len[slots]

    def blocks_of(self, slots: np.ndarray) -> np.ndarray:
        """Blocks of each sequence that have an entry in its page table (the same in every KV group)."""
        return self._nblk[slots]

    def table_rows(self, group: int, slots: np.ndarray, width: int) -> np.ndarray:
        """``page_rows`` as an array [len(slots), width]."""
        table = self._table[group]
        if width > table.shape[1]:
            table = np.concatenate([table, np.zeros((table.shape[0], width - table.shape[1]), dtype=np.int32)], axis=1)
            self._table[group] = table
        return table[slots, :width]

    def advance_each_by_one(self, slots: np.ndarray) -> None:
        """``advance(slot, 1)`` for every slot of the array (which names each slot once)."""
        self._len[slots] += 1
        if self.windowed:
            for s in slots.tolist():
                self._give_back(s, self._seq[s])

    def page_rows(self, group: int, slots: Sequence[int], width: Optional[int] = None) -> List[List[int]]:
        """Page table of these sequences for one KV group, padded with page 0
        (a valid page: a stray read cannot fault, and no kernel reads past a
        sequence's length)."""
        rows = [[0 if p is None else p for p in self._get(s).pages[group]] for s in slots]
        width = max([width or 1] + [len(r) for r in rows])
        return [r + [0] * (width - len(r)) for r in rows]

    # ---- views ------------------------------------------------------------------
    def view(self, position: int, page_tables: Dict[int, torch.Tensor]):
        """The cache as schedule position ``position`` sees it in this step: one view, None, or (for a
        position that gave a list of needs) a list of views in the order of its needs."""
        writable = self.plan.owner[position]
        views = []
        for gi, layer in self.plan.bindings[position]:
            need = self.plan.groups[gi].need
            if isinstance(need, KVNeed):
                views.append(KVView(self.storage[gi][layer], page_tables[gi], self.page_size, writable, need))
            else:
                views.append(StateView(self.storage[gi][layer], writable, need))
        if self.plan.several[position]:
            return views
        return views[0] if views else None

    # ---- inspection ---------------------------------------------------------------
    def dump_slot(self, slot: int) -> Dict[int, torch.Tensor]:
        """Contents of a sequence for tests: per KV group [layers, 2, length, kv heads, head_dim]
        (rows of pages that were given back are zero), per state group [layers, ...]."""
        seq = self._get(slot)
        out: Dict[int, torch.Tensor] = {}
        for gi, g in enumerate(self.plan.groups):
            st = self.storage[gi]
            if isinstance(g.need, KVNeed):
                L = int(self._len[slot])
                rows = torch.zeros((g.n_layers, 2, L, g.need.n_kv_heads, g.need.head_dim), dtype=st.dtype,
                                   device=st.device)
                for blk, page in enumerate(seq.pages[gi]):
                    lo, hi = blk * self.page_size, min(L, (blk + 1) * self.page_size)
                    if page is None or lo >= hi:
                        continue
                    rows[:, :, lo:hi] = st[:, page, :, :, :hi - lo].permute(0, 1, 3, 2, 4)
                out[gi] = rows
            else:
                out[gi] = st[:, slot].clone()
        return out

    def check(self) -> None:
        """No slot or page lost, held twice or freed twice."""
        self.slots.check()
        if sorted(self._seq) != [i for i in range(self.slots.n) if self.slots.is_held(i)]:
            raise CacheError("assigned sequences and held slots disagree")
        for gi in self.kv_groups:
            self.pages[gi].check()
            held = [p for s in self._seq.values() for p in s.pages[gi] if p is not None]
            if len(set(held)) != len(held):
                raise CacheError("a page belongs to two sequences")
            if len(held) != self.pages[gi].held_count:
                raise CacheError(f"{self.pages[gi].held_count} pages are held but sequences own {len(held)}")
            for s, seq in self._seq.items():
                row = [0 if p is None else p for p in seq.pages[gi]]
                if self._table[gi][s, :len(row)].tolist() != row or int(self._nblk[s]) != len(row):
                    raise CacheError(f"the page table of slot {s} and its page list disagree")
        if [i for i in range(self.slots.n) if self._assigned[i]] != sorted(self._seq):
            raise CacheError("the array of assigned slots and the assigned sequences disagree")
