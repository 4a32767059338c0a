"""Host side of the paged KV cache: page allocator, per-slot block tables, prefix sharing.

The reference keeps one ring buffer per batch slot and, when a request arrives, puts it in
the FREE slot whose previous request shares the longest token prefix, so that the shared
chunks need no prefill (g4b/scheduler.py:96-125).  With pages the same idea becomes page
sharing: the new request's block table points at the donor's full pages (reference counted,
never written again), the donor may be any slot, free or still running, and a retired
slot's pages stay cached until the pool runs short.

``PagedKVManager`` produces what the kernels read: ``block_tables [B, max_pages] int32``,
``cache_offsets [B] int32``, ``time_dim_sizes [B] int32`` and ``user_phase [B] uint8``, through
methods with the signature of the reference's ``Model.prepare_prefill_inputs`` /
``prepare_decode_inputs`` (g4b/models/model.py:15-31, g4b/models/gemma4e.py:224-248).  Pure
host code; device tensors are written with one asynchronous copy each from pinned memory.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

PHASE_UNALLOCATED, PHASE_PREFILL, PHASE_DECODE = 0, 1, 2   # g4b/kernels/fa2.py:29-31


class OutOfPages(RuntimeError):
    """The pool cannot cover a request even after dropping every cached (retired) page."""


def shared_prefix_length(a, b) -> int:
    """Number of leading tokens a and b have in common (g4b/utils.py:94-98)."""
    n = min(len(a), len(b))
    for i in range(n):
        if a[i] != b[i]:
            return i
    return n


class PageAllocator:
    """Free list + reference counts over ``num_pages`` page ids."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("num_pages must be positive")
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages - 1, -1, -1))   # pop() hands out 0, 1, 2, ...
        self._refs = np.zeros(self.num_pages, dtype=np.int32)

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def refcount(self, page: int) -> int:
        return int(self._refs[page])

    def alloc(self, n: int) -> list[int]:
        if n > len(self._free):
            raise OutOfPages(f"need {n} pages, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        self._refs[out] = 1
        return out

    def retain(self, pages) -> None:
        for p in pages:
            if self._refs[p] <= 0:
                raise RuntimeError(f"page {p} is not allocated")
            self._refs[p] += 1

    def release(self, pages) -> None:
        for p in pages:
            if self._refs[p] <= 0:
                raise RuntimeError(f"page {p} released more often than retained")
            self._refs[p] -= 1
            if self._refs[p] == 0:
                self._free.append(p)


@dataclass
class _Slot:
    pages: list[int] = field(default_factory=list)   # page ids in sequence order
    tokens: list[int] = field(default_factory=list)  # tokens whose K/V those pages hold (or will, once prefilled)
    filled: int = 0                                  # leading tokens whose K/V a launched step has written
    active: bool = False
    retired_at: int = -1                             # tick of retirement, for eviction order


class PagedKVManager:
    """Block tables for ``max_batch`` slots over one page pool shared by all of them."""

    def __init__(self, *, num_pages: int, max_batch: int, max_context: int, page_size: int = 16,
                 prefill_chunk: int = 1, decode_reserve_pages: int = 1):
        if page_size < 16 or page_size & (page_size - 1):
            raise ValueError("page_size must be a power of two >= 16")
        self.page_size = int(page_size)
        self.max_batch = int(max_batch)
        self.max_pages = (int(max_context) + self.page_size - 1) // self.page_size
        self.prefill_chunk = int(prefill_chunk)
        self.decode_reserve_pages = int(decode_reserve_pages)
        self.alloc = PageAllocator(num_pages)
        self.slots = [_Slot() for _ in range(self.max_batch)]
        self.block_tables = np.full((self.max_batch, self.max_pages), -1, dtype=np.int32)
        self.cache_offsets = np.zeros(self.max_batch, dtype=np.int32)
        self.time_dim_sizes = np.zeros(self.max_batch, dtype=np.int32)
        self.user_phase = np.zeros(self.max_batch, dtype=np.uint8)
        self.tables_dirty = True
        self._tick = 0
        self._device = None

    # ------------------------------------------------------------------ requests
    def free_slots(self) -> list[int]:
        return [i for i, s in enumerate(self.slots) if not s.active]

    def place_request(self, tokens: list[int]) -> tuple[int, int]:
        """Puts a new request into a free slot.  Returns ``(slot, prefill_pos)``: the first
        ``prefill_pos`` tokens already have their K/V in pages shared with a donor slot.

        ``prefill_pos`` follows the reference's rule -- whole prefill chunks only, and never the
        chunk that holds the last prompt token, which must run to sample
        (g4b/scheduler.py:118-122) -- rounded down to whole pages."""
        free = self.free_slots()
        if not free:
            raise RuntimeError("no free slot")
        # only K/V that an already launched step wrote can be shared (launches are stream ordered)
        shared = [min(shared_prefix_length(s.tokens, tokens), s.filled) for s in self.slots]
        donor = max(range(self.max_batch), key=lambda i: shared[i])
        n = max(0, (shared[donor] - 1) // self.prefill_chunk * self.prefill_chunk)
        n = n // self.page_size * self.page_size
        n_pages = n // self.page_size
        # the donor itself if it is free (its tail pages are dropped), else the emptiest free slot
        if n_pages > 0 and not self.slots[donor].active:
            slot = donor
            s = self.slots[slot]
            self.alloc.release(s.pages[n_pages:])
            s.pages = s.pages[:n_pages]
        else:
            slot = min(free, key=lambda i: len(self.slots[i].pages))
            s = self.slots[slot]
            self.alloc.release(s.pages)
            s.pages = []
            s.filled = 0
            if n_pages > 0:
                s.pages = list(self.slots[donor].pages[:n_pages])
                self.alloc.retain(s.pages)
        s.tokens = list(tokens)
        s.filled = n
        s.active = True
        s.retired_at = -1
        self._write_row(slot)
        return slot, n

    def retire(self, slot: int, processed_tokens: list[int] | None = None) -> None:
        """The slot's request ended.  Its pages stay as a prefix cache (``processed_tokens``:
        what they hold, default the prompt given at placement) until the pool needs them."""
        s = self.slots[slot]
        s.active = False
        if processed_tokens is not None:
            s.tokens = list(processed_tokens)
        # only tokens whose K/V sits in the pages can be shared later
        s.filled = min(s.filled, len(s.tokens), len(s.pages) * self.page_size)
        s.tokens = s.tokens[: s.filled]
        self._tick += 1
        s.retired_at = self._tick

    def ensure(self, slot: int, n_tokens: int) -> bool:
        """Makes the slot's table cover ``n_tokens`` tokens.  Returns True if pages were added."""
        if n_tokens > self.max_pages * self.page_size:
            raise ValueError(f"{n_tokens} tokens exceed the context capacity {self.max_pages * self.page_size}")
        s = self.slots[slot]
        need = (n_tokens + self.page_size - 1) // self.page_size - len(s.pages)
        if need <= 0:
            return False
        self._make_room(need, keep=slot)
        s.pages += self.alloc.alloc(need)
        self._write_row(slot)
        return True

    def _make_room(self, need: int, keep: int) -> None:
        """Drops cached pages of retired slots, oldest first, until ``need`` pages are free."""
        if self.alloc.free_pages >= need:
            return
        retired = sorted((i for i, s in enumerate(self.slots) if not s.active and s.pages and i != keep),
                         key=lambda i: self.slots[i].retired_at)
        for i in retired:
            s = self.slots[i]
            self.alloc.release(s.pages)
            s.pages, s.tokens, s.filled = [], [], 0
            self._write_row(i)
            if self.alloc.free_pages >= need:
                return
        if self.alloc.free_pages < need:
            raise OutOfPages(f"need {need} pages, {self.alloc.free_pages} free after dropping the prefix cache")

    def _write_row(self, slot: int) -> None:
        row = self.block_tables[slot]
        pages = self.slots[slot].pages
        row[: len(pages)] = pages
        row[len(pages):] = -1
        self.tables_dirty = True

    # ------------------------------------------------------------------ model-facing
    def prepare_prefill_inputs(self, token_cols, cache_offsets, time_sizes_after, sample_positions=None):
        """Same arguments as the reference's ``Model.prepare_prefill_inputs``.  A slot takes part
        iff ``time_sizes_after[b] > 0`` (the scheduler passes zeros for idle slots,
        g4b/scheduler.py:141-147); its table is grown to ``time_sizes_after[b]`` tokens, which
        counts the whole padded chunk (g4b/scheduler.py:166-172)."""
        return self._prepare(cache_offsets, time_sizes_after, PHASE_PREFILL, reserve=0)

    def prepare_decode_inputs(self, token_cols, cache_offsets, time_sizes_after, sample_positions=None):
        """Same arguments as ``Model.prepare_decode_inputs``.  The reference uploads decode state
        once and then advances it on the device (g4b/scheduler.py:205-210), so pages are reserved
        ahead: ``decode_reserve_pages`` beyond the one the next token falls in."""
        return self._prepare(cache_offsets, time_sizes_after, PHASE_DECODE, reserve=self.decode_reserve_pages)

    def _prepare(self, cache_offsets, time_sizes_after, phase, reserve):
        for b in range(self.max_batch):
            live = time_sizes_after[b] > 0
            self.cache_offsets[b] = cache_offsets[b]
            self.time_dim_sizes[b] = time_sizes_after[b]
            self.user_phase[b] = phase if live else PHASE_UNALLOCATED
            if live:
                want = min(int(time_sizes_after[b]) + reserve * self.page_size, self.max_pages * self.page_size)
                self.ensure(b, max(want, int(time_sizes_after[b])))
                s = self.slots[b]
                s.filled = max(s.filled, int(time_sizes_after[b]))
        return self.block_tables, self.cache_offsets, self.time_dim_sizes, self.user_phase

    def decode_steps_covered(self, slot: int) -> int:
        """How many more tokens the slot can append on the device before it needs a new page."""
        return len(self.slots[slot].pages) * self.page_size - int(self.time_dim_sizes[slot])

    def advance_decode(self) -> bool:
        """Mirrors ``advance_decode_state`` on the host (g4b/kernels/advance_decode_state.py:52-63)
        and tops up reservations.  Returns True when a block table changed, i.e. the caller must
        upload before the next step (the reference's ``needs_upload``)."""
        changed = False
        for b in range(self.max_batch):
            if self.user_phase[b] != PHASE_DECODE:
                continue
            self.cache_offsets[b] += 1
            self.time_dim_sizes[b] += 1
            self.slots[b].filled = max(self.slots[b].filled, int(self.time_dim_sizes[b]))
            if self.decode_steps_covered(b) < 0:
                raise RuntimeError(f"slot {b} ran past its reserved pages")
            if self.decode_steps_covered(b) == 0 and int(self.time_dim_sizes[b]) < self.max_pages * self.page_size:
                want = min(int(self.time_dim_sizes[b]) + 1 + self.decode_reserve_pages * self.page_size,
                           self.max_pages * self.page_size)
                changed |= self.ensure(b, want)
        return changed

    # ------------------------------------------------------------------ device mirror
    def bind_device(self, device) -> None:
        """Allocates the device tensors and their pinned staging buffers once."""
        import torch

        self._device = torch.device(device)
        pin = self._device.type == "cuda"
        self._host = {
            "block_tables": torch.from_numpy(self.block_tables),
            "cache_offsets": torch.from_numpy(self.cache_offsets),
            "time_dim_sizes": torch.from_numpy(self.time_dim_sizes),
            "user_phase": torch.from_numpy(self.user_phase),
        }
        self._staging = {k: (torch.empty_like(v).pin_memory() if pin else torch.empty_like(v)) for k, v in self._host.items()}
        self.device_tensors = {k: torch.empty_like(v, device=self._device) for k, v in self._host.items()}
        self._copied = torch.cuda.Event() if pin else None
        self._copy_pending = False

    def upload(self, tables_only_if_dirty: bool = True) -> dict:
        """Copies the host state to the device tensors (asynchronously, on torch's current
        stream).  The block tables go only when they changed."""
        if self._device is None:
            raise RuntimeError("bind_device() first")
        if self._copy_pending:
            self._copied.synchronize()      # the staging buffers are still being read
            self._copy_pending = False
        for name in ("cache_offsets", "time_dim_sizes", "user_phase", "block_tables"):
            if name == "block_tables" and tables_only_if_dirty and not self.tables_dirty:
                continue
            self._staging[name].copy_(self._host[name])
            self.device_tensors[name].copy_(self._staging[name], non_blocking=True)
        self.tables_dirty = False
        if self._copied is not None:
            self._copied.record()
            self._copy_pending = True
        return self.device_tensors
