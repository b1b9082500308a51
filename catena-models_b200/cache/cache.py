"""The cache: a slot for each sequence, per-layer state in groups with storage of their own.

`CacheBook` is the host-side ledger (which slot is live, how long each sequence is, which
pages it holds in which group); it needs no device and is what the CPU tests exercise.
`Cache` adds the device storage:

* a group of key/value layers with equal `KVStateSpec`:
  `storage[layer, k|v, page, kv_head, PAGE_TOKENS, head_dim]` and a page table
  `[slot, page index] -> page`; a growing group holds position p in entry p, a ring group
  in entry p % ring, so a sliding-window layer never holds more than its window;
* a group of layers with equal `FixedStateSpec`: `storage[layer, slot, *shape]`.

Sizing follows one number, `max_tokens`: the most tokens that live sequences hold at any
time, each sequence rounded up to whole pages.  Slots and pages are given back by `release`
and used again by the next batch; nothing is cleared on release, because every kernel reads
only entries below the sequence's own length.  Fixed-size states are cleared when a slot is
admitted (`zero_slots`).
"""
from __future__ import annotations

import dataclasses

import torch

from .. import kernels
from .allocators import CacheError, CacheFull, IndexAllocator
from .spec import PAGE_TOKENS, FixedStateSpec, KVStateSpec

DEFAULT_MAX_SEQS = 4096


def _ceil_div(a, b):
    return (a + b - 1) // b


class CacheBook:
    """Slots, lengths and pages of the live sequences (host only)."""

    def __init__(self, kv_specs, max_tokens, max_seqs=None, max_len=None):
        if max_tokens < 1:
            raise CacheError(f"max_tokens {max_tokens}")
        self.page_budget = _ceil_div(max_tokens, PAGE_TOKENS)
        self.max_seqs = max_seqs or min(self.page_budget, DEFAULT_MAX_SEQS)
        self.max_len = max_len or self.page_budget * PAGE_TOKENS
        self.kv_specs = list(kv_specs)
        self.slots = IndexAllocator(self.max_seqs, "slot")
        self.group_pages, self.pages_per_seq, self.page_alloc = [], [], []
        for spec in self.kv_specs:
            if spec.window > 0:
                per_seq = spec.ring // PAGE_TOKENS
                total = min(self.page_budget, self.max_seqs * per_seq)
            else:
                per_seq = min(self.page_budget, _ceil_div(self.max_len, PAGE_TOKENS))
                total = self.page_budget
            self.group_pages.append(total)
            self.pages_per_seq.append(per_seq)
            self.page_alloc.append(IndexAllocator(total, "page"))
        self.length = {}          # slot -> tokens held
        self.pages = {}           # slot -> [pages of group 0, pages of group 1, ...]

    def admit(self):
        (slot,) = self.slots.take(1)
        self.length[slot] = 0
        self.pages[slot] = [[] for _ in self.kv_specs]
        return slot

    def reserve(self, slot, new_length):
        """Make room for positions below `new_length`.  Returns the new page-table entries as
        (group, page index within the sequence, page).  Takes nothing if any group is short."""
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not live")
        if new_length > self.max_len:
            raise CacheFull(f"sequence of {new_length} tokens exceeds the longest allowed ({self.max_len})")
        need = []
        for g, spec in enumerate(self.kv_specs):
            extra = spec.pages(new_length) - len(self.pages[slot][g])
            if extra > self.page_alloc[g].free_count:
                raise CacheFull(f"group {g}: {extra} page(s) wanted, {self.page_alloc[g].free_count} free "
                                f"(cache sized for {self.page_budget * PAGE_TOKENS} tokens)")
            need.append(max(0, extra))
        updates = []
        for g, extra in enumerate(need):
            for page in self.page_alloc[g].take(extra):
                updates.append((g, len(self.pages[slot][g]), page))
                self.pages[slot][g].append(page)
        return updates

    def advance(self, slot, new_length):
        self.length[slot] = new_length

    def release(self, slot):
        if slot not in self.length:
            raise CacheError(f"slot {slot} released but not live")
        for g, pages in enumerate(self.pages[slot]):
            self.page_alloc[g].give_back(pages)
        del self.length[slot], self.pages[slot]
        self.slots.give_back([slot])

    @property
    def live(self):
        return sorted(self.length)

    def tokens_held(self):
        return sum(_ceil_div(n, PAGE_TOKENS) * PAGE_TOKENS for n in self.length.values())


@dataclasses.dataclass
class KVView:
    """What an attention-like mixer gets for one layer."""
    spec: KVStateSpec
    pool: torch.Tensor          # [2, pages, kv_heads, PAGE_TOKENS, head_dim]
    pages: int
    ptab: torch.Tensor          # [slots, pages per sequence] int32
    group: int
    owned: bool = True          # False: this layer reads a state that another layer writes
    unit: int = -1              # the state unit of the plan this view belongs to

    @property
    def ring(self):
        return self.spec.ring


@dataclasses.dataclass
class FixedView:
    """What a mixer with fixed-size state gets for one layer: `tensor[slot]` is its state."""
    spec: FixedStateSpec
    tensor: torch.Tensor        # [slots, *shape]
    owned: bool = True
    unit: int = -1


class Cache:
    """Device storage for a list of state specs (one per state unit of the model's plan)."""

    def __init__(self, state_specs, max_tokens, dtype, device, max_seqs=None, max_len=None):
        self.dtype, self.device = dtype, torch.device(device)
        self.state_specs = list(state_specs)
        kv_groups, fixed_groups = [], []
        self._where = []                                   # state unit -> (kind, group, index)
        counts = {}
        for spec in self.state_specs:
            if spec is None:
                self._where.append(None)
                continue
            table = kv_groups if isinstance(spec, KVStateSpec) else fixed_groups
            if spec not in table:
                table.append(spec)
            g = table.index(spec)
            kind = "kv" if isinstance(spec, KVStateSpec) else "fixed"
            idx = counts.get((kind, g), 0)
            counts[(kind, g)] = idx + 1
            self._where.append((kind, g, idx))
        self.book = CacheBook(kv_groups, max_tokens, max_seqs, max_len)
        self.kv_storage, self.ptabs, self._ptab_offset = [], [], []
        total_entries = sum(self.book.max_seqs * p for p in self.book.pages_per_seq)
        self.ptab_all = torch.zeros(max(1, total_entries), dtype=torch.int32, device=self.device)
        off = 0
        for g, spec in enumerate(kv_groups):
            layers = counts[("kv", g)]
            self.kv_storage.append(torch.empty(
                (layers, 2, self.book.group_pages[g], spec.kv_heads, PAGE_TOKENS, spec.head_dim),
                dtype=dtype, device=self.device))
            n = self.book.max_seqs * self.book.pages_per_seq[g]
            self.ptabs.append(self.ptab_all[off:off + n].view(self.book.max_seqs, self.book.pages_per_seq[g]))
            self._ptab_offset.append(off)
            off += n
        self.fixed_storage = []
        for g, spec in enumerate(fixed_groups):
            layers = counts[("fixed", g)]
            fdtype = torch.float32 if spec.dtype == "float32" else dtype
            self.fixed_storage.append(torch.zeros((layers, self.book.max_seqs, *spec.shape),
                                                  dtype=fdtype, device=self.device))
        self.kv_specs, self.fixed_specs = kv_groups, fixed_groups

    # ------------------------------------------------------------------ views for mixers
    def view(self, unit):
        where = self._where[unit]
        if where is None:
            return None
        kind, g, idx = where
        if kind == "kv":
            return KVView(self.kv_specs[g], self.kv_storage[g][idx], self.book.group_pages[g], self.ptabs[g], g)
        return FixedView(self.fixed_specs[g], self.fixed_storage[g][idx])

    # ------------------------------------------------------------------ bookkeeping
    def admit(self):
        """A fresh slot; its fixed-size states are cleared on the device."""
        return self.admit_many(1)[0]

    def admit_many(self, count):
        """`count` fresh slots; their fixed-size states are cleared by one launch per group."""
        slots = [self.book.admit() for _ in range(count)]
        for store in self.fixed_storage:
            kernels.zero_slots(store, slots)
        return slots

    def release(self, slot):
        self.book.release(slot)

    def copy_slot(self, src, dst):
        """Give the fresh slot `dst` a copy of everything slot `src` holds: its pages (new pages,
        same contents), its fixed-size states and its length.  All or nothing."""
        book = self.book
        if src not in book.length or dst not in book.length:
            raise CacheError("copy_slot: both slots must be live")
        if book.length[dst] != 0 or any(book.pages[dst]):
            raise CacheError(f"copy_slot: slot {dst} already holds tokens")
        length = book.length[src]
        updates = book.reserve(dst, length)                  # raises CacheFull and takes nothing if short
        flat = self.flat_updates(dst, updates)
        if flat:
            index = torch.tensor([i for i, _ in flat], dtype=torch.int32, device=self.device)
            value = torch.tensor([p for _, p in flat], dtype=torch.int32, device=self.device)
            count = torch.tensor([len(flat)], dtype=torch.int32, device=self.device)
            kernels.scatter_i32(self.ptab_all, index, value, count, len(flat))
        for g in range(len(self.kv_specs)):
            n = len(book.pages[dst][g])
            if n:
                s_ids = torch.tensor(book.pages[src][g][:n], dtype=torch.int32, device=self.device)
                d_ids = torch.tensor(book.pages[dst][g], dtype=torch.int32, device=self.device)
                kernels.copy_pages(self.kv_storage[g], s_ids, d_ids)
        for store in self.fixed_storage:
            store[:, dst].copy_(store[:, src])
        book.advance(dst, length)

    def flat_updates(self, slot, updates):
        """(index into ptab_all, page) pairs for the entries `CacheBook.reserve` returned."""
        return [(self._ptab_offset[g] + slot * self.book.pages_per_seq[g] + j, page) for g, j, page in updates]

    def bytes(self):
        n = self.ptab_all.numel() * 4
        for t in self.kv_storage + self.fixed_storage:
            n += t.numel() * t.element_size()
        return n

    def live_bytes(self):
        """Bytes of cache that a decode step over all live sequences has to read."""
        total = 0
        for slot, length in self.book.length.items():
            for g, spec in enumerate(self.kv_specs):
                layers = self.kv_storage[g].shape[0]
                visible = min(length, spec.window) if spec.window > 0 else length
                total += layers * 2 * visible * spec.kv_heads * spec.head_dim * self.kv_storage[g].element_size()
            for store in self.fixed_storage:
                total += store[:, slot].numel() * store.element_size()
        return total
