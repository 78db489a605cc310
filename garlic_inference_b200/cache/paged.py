"""The cache on the device: paged keys and values per group of layers, and a
fixed-size state row per slot.

Each mixer says what it needs of the cache (`KVRequirement`: all keys or a
window of them; `StateRequirement`: a tensor of fixed shape per sequence).
Cache entries with the same key/value needs form a *group* with storage, a
page pool and a block table of its own; within a group a page id means the
same page in every layer, so one table row serves all its layers.  Lengths
live on the host; the step function writes per-token positions and slots for
the kernels.

Pools are `[n_pages, n_kv_heads, page_size, head_dim]` per layer, keys and
values apart (upstream: src/kvcache.h:49-50, page size fixed to 32 at
kvcache.h:7, one table per layer).  Pools start zeroed and only ever hold
finite numbers, so a kernel may read a page's unused rows and mask them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Union

import numpy as np
import torch

from .allocator import CacheError, GroupTable, SlotAllocator

TOKEN_UNIT = 64     # capacities are counted per sequence in units of this many tokens


@dataclass(frozen=True)
class KVRequirement:
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: every earlier key; w: the last w keys


@dataclass(frozen=True)
class StateRequirement:
    shape: tuple
    dtype: torch.dtype = torch.float32


Requirement = Union[KVRequirement, StateRequirement, None]


@dataclass
class KVView:
    """What a mixer gets for one cache entry in one step."""
    k_pool: torch.Tensor          # [n_pages, n_kv, page_size, d]
    v_pool: torch.Tensor
    block_table: torch.Tensor     # int32 [max_slots, max_pages_per_seq], -1 = no page
    page_size: int
    window: Optional[int]


@dataclass
class EntryView:
    """Everything one cache entry holds: paged keys/values and/or a state tensor [max_slots, ...]."""
    kv: Optional[KVView] = None
    state: Optional[torch.Tensor] = None


class _KVGroup:
    def __init__(self, req: KVRequirement, entries: list[int], n_pages: int, page_size: int, max_slots: int,
                 max_pages_per_seq: int, dtype: torch.dtype, device):
        self.req = req
        self.entries = entries
        self.host = GroupTable(n_pages, page_size, max_slots, max_pages_per_seq, req.window)
        self.storage = torch.zeros((len(entries), 2, n_pages, req.n_kv_heads, page_size, req.head_dim),
                                   dtype=dtype, device=device)
        self.table = torch.full((max_slots, max_pages_per_seq), -1, dtype=torch.int32, device=device)

    def upload(self) -> None:
        if not self.host.dirty:
            return
        rows = sorted(self.host.dirty)
        self.host.dirty.clear()
        idx = torch.as_tensor(rows, dtype=torch.long)
        src = torch.from_numpy(self.host.table[rows])
        if self.table.is_cuda:                   # pinned, so that neither copy waits for the steps in flight
            idx, src = idx.pin_memory(), src.pin_memory()
        self.table.index_copy_(0, idx.to(self.table.device, non_blocking=True),
                               src.to(self.table.device, non_blocking=True))


class PagedCache:
    """Slots, pages and state for one model.

    `requirements[e]` is what cache entry `e` needs (None for a mixer that keeps nothing).
    `max_tokens` is the most tokens that live sequences hold at any time, each sequence counted
    in units of 64 tokens."""

    def __init__(self, requirements: Sequence[Requirement], max_tokens: int, max_positions: int,
                 dtype: torch.dtype, device, page_size: int = 64, max_slots: Optional[int] = None):
        if page_size <= 0:
            raise CacheError(f"page_size must be positive, not {page_size}")
        if max_tokens <= 0:
            raise CacheError(f"max_tokens must be positive, not {max_tokens}")
        units = -(-max_tokens // TOKEN_UNIT)
        self.page_size = page_size
        self.max_tokens = units * TOKEN_UNIT
        self.max_positions = max_positions
        self.max_slots = max_slots or units
        self.n_pages = units * (-(-TOKEN_UNIT // page_size)) if page_size <= TOKEN_UNIT else units
        longest = min(max_positions, self.max_tokens)
        self.max_pages_per_seq = -(-longest // page_size)
        self.dtype, self.device = dtype, torch.device(device)
        self.slots = SlotAllocator(self.max_slots)
        self.lengths = np.zeros(self.max_slots, dtype=np.int64)

        self.groups: list[_KVGroup] = []
        self._kv_of_entry: dict[int, tuple[_KVGroup, int]] = {}
        self._state_of_entry: dict[int, torch.Tensor] = {}
        by_req: dict[KVRequirement, list[int]] = {}
        for e, req in enumerate(requirements):
            if isinstance(req, KVRequirement):
                by_req.setdefault(req, []).append(e)
            elif isinstance(req, StateRequirement):
                # one row per slot and a spare last row: a padding row of a recorded step carries slot -1,
                # which as an index is that spare, so it reads and writes nothing a sequence owns
                self._state_of_entry[e] = torch.zeros((self.max_slots + 1, *req.shape), dtype=req.dtype,
                                                      device=self.device)
            elif req is not None:
                raise CacheError(f"cache entry {e}: unknown requirement {req!r}")
        for req, entries in by_req.items():
            g = _KVGroup(req, entries, self.n_pages, page_size, self.max_slots, self.max_pages_per_seq,
                         dtype, self.device)
            self.groups.append(g)
            for i, e in enumerate(entries):
                self._kv_of_entry[e] = (g, i)
        # set by the kernels when an index they were given is out of range (0 = all well)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    # ---- slots -------------------------------------------------------------------
    def alloc_slot(self) -> int:
        s = self.slots.alloc()
        self.lengths[s] = 0
        for st in self._state_of_entry.values():
            st[s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)
        for g in self.groups:
            g.host.release(slot)
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        return int(self.lengths[slot])

    @property
    def state_bytes_per_slot(self) -> int:
        return sum(int(np.prod(st.shape[1:])) * st.element_size() for st in self._state_of_entry.values())

    # ---- one step ------------------------------------------------------------------
    def prepare(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        """Give every listed slot room for `n_new` more positions, or raise before anything changed."""
        seen = set()
        for s, n in zip(slots, n_new):
            if not self.slots.is_live(s):
                raise CacheError(f"slot {s} is not in use")
            if s in seen:
                raise CacheError(f"slot {s} appears twice in one step")
            seen.add(s)
            if n < 0:
                raise CacheError("a step cannot bring a negative number of tokens")
            if self.lengths[s] + n > self.max_positions:
                raise CacheError(f"slot {s} would reach {self.lengths[s] + n} positions; the model's "
                                 f"limit is {self.max_positions}")
            if -(-(int(self.lengths[s]) + n) // self.page_size) > self.max_pages_per_seq:
                raise CacheError(f"slot {s} would reach {self.lengths[s] + n} positions; the cache was "
                                 f"sized for {self.max_pages_per_seq * self.page_size} per sequence")
        for g in self.groups:
            need = sum(g.host.pages_needed(s, int(self.lengths[s]) + n) for s, n in zip(slots, n_new))
            if need > g.host.pool.n_free:
                raise CacheError(f"the cache is full: this step needs {need} more pages of "
                                 f"{self.page_size} tokens, {g.host.pool.n_free} of {g.host.pool.n_pages} are free")
        for g in self.groups:
            for s, n in zip(slots, n_new):
                g.host.reserve(s, int(self.lengths[s]) + n)
            g.upload()

    def commit(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        """The step ran: lengths grow, windowed groups drop what no later query can see."""
        for s, n in zip(slots, n_new):
            self.lengths[s] += n
            for g in self.groups:
                g.host.trim(s, int(self.lengths[s]))

    # ---- views -----------------------------------------------------------------------
    def kv_view(self, entry: int) -> Optional[KVView]:
        if entry not in self._kv_of_entry:
            return None
        g, i = self._kv_of_entry[entry]
        return KVView(g.storage[i, 0], g.storage[i, 1], g.table, self.page_size, g.req.window)

    def state_view(self, entry: int) -> Optional[torch.Tensor]:
        return self._state_of_entry.get(entry)

    def view(self, entry: int) -> EntryView:
        return EntryView(self.kv_view(entry), self.state_view(entry))

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise CacheError(f"a kernel was given an index outside the cache (code {code}): "
                             "1 position beyond the block table, 2/5 unmapped page, 3 position beyond "
                             "the rotary table, 4 query position beyond the block table")

    def bytes_per_token(self) -> int:
        return sum(2 * len(g.entries) * g.req.n_kv_heads * g.req.head_dim * g.storage.element_size()
                   for g in self.groups)
