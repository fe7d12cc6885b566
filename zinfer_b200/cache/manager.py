"""The cache: a slot per sequence, paged keys and values per group of layers, fixed-size state.

The reference holds exactly one sequence per `State`: a position counter, one K and one V byte
array with a region per (attention layer, kv head) indexed by `kv_slot` which counts attention
layers only, and `conv_state [n_conv][K-1][D]` zeroed at reset (src/model.zig:1403-1465,
1537-1574, 1617-1621, 733-744).  Here:

* a *slot* is one sequence of a batch: its length, its pages in every group, its row in every
  state tensor.  Slots are handed out by `alloc_slots` and given back by `free_slots`; a freed
  slot's pages return to their pools and are reused by later batches.
* layers whose mixers ask for the same kind of growing cache (same KV heads, widths and
  window) form a *group* with storage of its own: two tensors
  [layers of the group, pages, kv heads, page_size, width] (keys and values for attention; a
  mixer may ask for another width of the second, or for one tensor only) and one page table
  [slots, pages per sequence] shared by the group's layers.  A group with a window gives pages
  back as soon as every position in them has left the window.
* a mixer that asks for fixed-size state gets a row per slot in a tensor
  [calls with that state shape, slots, *shape], zeroed when the slot is handed out.

Storage belongs to *calls* (entries of the model's schedule), not to layers, so a layer named
twice in the schedule has two caches, and a call may read the cache another call owns.
All bookkeeping is host-side Python on NumPy tables; only `sync()` touches the device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..parts.base import KVRequest, StateRequest


class CacheError(RuntimeError):
    pass


class NoFreeSlot(CacheError):
    pass


class OutOfPages(CacheError):
    pass


class ContextFull(CacheError):
    """A sequence would grow past the longest sequence the cache was built for
    (reference: error.ContextFull, src/model.zig:2520)."""


@dataclass
class CallCacheSpec:
    """What one schedule entry needs: `kv` if its mixer has a growing cache, `kv_owner` = the
    call whose storage it uses (itself unless it reads another call's cache), `state` if its
    mixer keeps fixed-size state."""

    kv: Optional[KVRequest] = None
    kv_owner: Optional[int] = None
    state: Optional[StateRequest] = None


@dataclass
class KVView:
    """One call's growing cache: k [pages, kv heads, page_size, head_dim], v [pages, kv heads,
    page_size, value_dim] (None if the mixer asked for one tensor only) and the group's page table
    [slots, pages per sequence] (int32, -1 = no page)."""

    k: torch.Tensor
    v: Optional[torch.Tensor]
    page_table: torch.Tensor
    page_size: int
    window: int
    group: int


class KVGroup:
    def __init__(self, request: KVRequest, n_layers: int, num_pages: int, page_size: int, max_slots: int,
                 max_pages_per_seq: int, dtype: torch.dtype, device):
        self.request, self.n_layers, self.num_pages, self.page_size = request, n_layers, num_pages, page_size
        shape = (n_layers, num_pages, request.n_kv_heads, page_size)
        self.k = torch.zeros((*shape, request.head_dim), dtype=dtype, device=device)
        # the second tensor has the width the mixer asked for, or is absent (one vector per token)
        self.v = torch.zeros((*shape, request.v_dim), dtype=dtype, device=device) if request.v_dim > 0 else None
        self.table_host = np.full((max_slots, max_pages_per_seq), -1, dtype=np.int32)
        self.table_dev = torch.full((max_slots, max_pages_per_seq), -1, dtype=torch.int32, device=device)
        self.free_pages = list(range(num_pages - 1, -1, -1))      # pop() hands out page 0 first
        self.n_pages_of = np.zeros(max_slots, dtype=np.int64)     # logical pages a slot has reached
        self.first_page_of = np.zeros(max_slots, dtype=np.int64)  # pages below it were given back
        self.dirty = False

    def pages_needed(self, slot: int, new_len: int) -> int:
        return max(0, -(-new_len // self.page_size) - int(self.n_pages_of[slot]))

    def grow(self, slot: int, new_len: int) -> None:
        for _ in range(self.pages_needed(slot, new_len)):
            page = self.free_pages.pop()
            self.table_host[slot, self.n_pages_of[slot]] = page
            self.n_pages_of[slot] += 1
            self.dirty = True

    def trim(self, slot: int, length: int) -> None:
        """Gives back pages whose positions all lie more than `window` behind the next query
        (position `length`, which sees keys [length + 1 - window, length])."""
        w = self.request.window
        if w <= 0:
            return
        first_needed = max(0, length + 1 - w) // self.page_size
        while self.first_page_of[slot] < min(first_needed, self.n_pages_of[slot]):
            i = int(self.first_page_of[slot])
            self.free_pages.append(int(self.table_host[slot, i]))
            self.table_host[slot, i] = -1
            self.first_page_of[slot] += 1
            self.dirty = True

    def release(self, slot: int) -> None:
        for i in range(int(self.first_page_of[slot]), int(self.n_pages_of[slot])):
            self.free_pages.append(int(self.table_host[slot, i]))
        if self.n_pages_of[slot]:
            self.table_host[slot, :self.n_pages_of[slot]] = -1
            self.dirty = True
        self.n_pages_of[slot] = 0
        self.first_page_of[slot] = 0

    def pages_held(self, slot: int) -> list[int]:
        return [int(p) for p in self.table_host[slot, int(self.first_page_of[slot]):int(self.n_pages_of[slot])]]

    def sync(self) -> None:
        if self.dirty:
            self.table_dev.copy_(torch.from_numpy(self.table_host), non_blocking=False)
            self.dirty = False


class CacheManager:
    def __init__(self, calls: Sequence[CallCacheSpec], max_slots: int, max_tokens: int, max_seq_len: int,
                 page_size: int, dtype: torch.dtype, device):
        if page_size <= 0 or page_size % 16:
            raise CacheError(f"page_size {page_size} must be a positive multiple of 16")
        if max_slots <= 0 or max_tokens <= 0 or max_seq_len <= 0:
            raise CacheError("max_slots, max_tokens and max_seq_len must be positive")
        self.max_slots, self.max_seq_len, self.page_size = max_slots, max_seq_len, page_size
        self.dtype, self.device = dtype, device
        self.num_pages = -(-max_tokens // page_size)
        self.max_pages_per_seq = min(-(-max_seq_len // page_size), self.num_pages)
        self.lengths = np.zeros(max_slots, dtype=np.int64)
        self.active = np.zeros(max_slots, dtype=bool)
        self.free_slot_list = list(range(max_slots - 1, -1, -1))

        # groups of growing caches
        self.groups: list[KVGroup] = []
        self._kv_place: dict[int, tuple[int, int]] = {}          # owning call -> (group, layer in group)
        self._kv_of_call: dict[int, int] = {}                    # call -> owning call
        by_request: dict[KVRequest, list[int]] = {}
        for c, spec in enumerate(calls):
            if spec.kv is None:
                continue
            owner = c if spec.kv_owner is None else spec.kv_owner
            self._kv_of_call[c] = owner
            if owner == c:
                by_request.setdefault(spec.kv, []).append(c)
        for c, owner in self._kv_of_call.items():
            if owner != c:
                if owner not in self._kv_of_call or self._kv_of_call[owner] != owner:
                    raise CacheError(f"call {c} reads the cache of call {owner}, which owns none")
                if calls[owner].kv != calls[c].kv:
                    raise CacheError(f"call {c} reads the cache of call {owner} but asks for a different layout")
        for request, owners in by_request.items():
            g = len(self.groups)
            self.groups.append(KVGroup(request, len(owners), self.num_pages, page_size, max_slots,
                                       self.max_pages_per_seq, dtype, device))
            for i, c in enumerate(owners):
                self._kv_place[c] = (g, i)

        # fixed-size state, one tensor per distinct request
        self.state_tensors: list[torch.Tensor] = []
        self._state_place: dict[int, tuple[int, int]] = {}
        by_state: dict[StateRequest, list[int]] = {}
        for c, spec in enumerate(calls):
            if spec.state is not None:
                by_state.setdefault(spec.state, []).append(c)
        for request, cs in by_state.items():
            s = len(self.state_tensors)
            self.state_tensors.append(torch.zeros((len(cs), max_slots, *request.shape), dtype=request.dtype,
                                                  device=device))
            for i, c in enumerate(cs):
                self._state_place[c] = (s, i)

    # ------------------------------------------------------------------ views for the calls
    def kv_view(self, call: int) -> Optional[KVView]:
        if call not in self._kv_of_call:
            return None
        g, i = self._kv_place[self._kv_of_call[call]]
        grp = self.groups[g]
        return KVView(grp.k[i], None if grp.v is None else grp.v[i], grp.table_dev, self.page_size,
                      grp.request.window, g)

    def writes_kv(self, call: int) -> bool:
        return self._kv_of_call.get(call) == call

    def state_view(self, call: int) -> Optional[torch.Tensor]:
        if call not in self._state_place:
            return None
        s, i = self._state_place[call]
        return self.state_tensors[s][i]

    # ------------------------------------------------------------------ slots
    def free_slot_count(self) -> int:
        return len(self.free_slot_list)

    def free_page_count(self) -> list[int]:
        return [len(g.free_pages) for g in self.groups]

    def alloc_slots(self, n: int) -> list[int]:
        """Hands out `n` empty slots (length 0, no pages, zero state) or raises NoFreeSlot."""
        if n > len(self.free_slot_list):
            raise NoFreeSlot(f"{n} sequences asked for, {len(self.free_slot_list)} of {self.max_slots} slots free")
        slots = [self.free_slot_list.pop() for _ in range(n)]
        for s in slots:
            self.active[s] = True
            self.lengths[s] = 0
        if slots and self.state_tensors:
            idx = torch.tensor(slots, dtype=torch.int64, device=self.device)
            for st in self.state_tensors:
                st.index_fill_(1, idx, 0)
        return slots

    def free_slots(self, slots: Sequence[int]) -> None:
        """Gives slots and their pages back.  Freeing a slot that is not held raises."""
        for s in slots:
            if not (0 <= s < self.max_slots) or not self.active[s]:
                raise CacheError(f"slot {s} is not held: it cannot be given back")
        if len(set(slots)) != len(slots):
            raise CacheError(f"slots {list(slots)} name a slot twice")
        for s in slots:
            for g in self.groups:
                g.release(s)
            self.active[s] = False
            self.lengths[s] = 0
            self.free_slot_list.append(s)

    # ------------------------------------------------------------------ growth
    def reserve(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        """Makes room for `new_tokens[i]` more tokens in `slots[i]`, in every group, or raises
        ContextFull / OutOfPages with nothing changed."""
        need = [0] * len(self.groups)
        for s, n in zip(slots, new_tokens):
            if not self.active[s]:
                raise CacheError(f"slot {s} is not held")
            new_len = int(self.lengths[s]) + int(n)
            if new_len > self.max_seq_len:
                raise ContextFull(f"slot {s}: {new_len} tokens exceed the longest sequence {self.max_seq_len}")
            for gi, g in enumerate(self.groups):
                need[gi] += g.pages_needed(s, new_len)
        for gi, g in enumerate(self.groups):
            if need[gi] > len(g.free_pages):
                raise OutOfPages(f"cache group {gi}: {need[gi]} pages needed, {len(g.free_pages)} of {g.num_pages} free")
        for s, n in zip(slots, new_tokens):
            for g in self.groups:
                g.grow(s, int(self.lengths[s]) + int(n))

    def advance(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        """Lengths move on after a step ran (src/model.zig:2480); windowed groups drop old pages."""
        for s, n in zip(slots, new_tokens):
            self.lengths[s] += int(n)
            for g in self.groups:
                g.trim(s, int(self.lengths[s]))

    def sync(self) -> None:
        """Uploads page tables that changed since the last step."""
        for g in self.groups:
            g.sync()

    def check_consistency(self) -> None:
        """Every page is free or held by exactly one slot; every slot is free or active."""
        for gi, g in enumerate(self.groups):
            held = [p for s in range(self.max_slots) for p in g.pages_held(s)]
            allp = held + g.free_pages
            if sorted(allp) != list(range(g.num_pages)):
                raise CacheError(f"group {gi}: pages lost or held twice")
        if sorted(self.free_slot_list + [s for s in range(self.max_slots) if self.active[s]]) != list(range(self.max_slots)):
            raise CacheError("slots lost or held twice")
