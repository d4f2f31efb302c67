"""Page and slot management shared by the serving loops, the paged cache of attention decoders and the state slots of recurrent mixers.

`PageAllocator` is the free list both serving loops draw from (ContinuousBatcher: whole requests at admission; StepScheduler:
page by page as a request grows). `PagedLatentCache` stores, per layer, one row per token - the latent followed by the rotated
key part - in pages of `page_size` tokens addressed through an int32 block table [slots, max_pages]; layers may differ in row
width, so every layer has its own pool tensor over the same page ids; a layer of width 0 caches nothing and has no pool.
`PagedStateCache` adds what mixers with a fixed-size memory need: named fp32 state tensors per layer with one entry per slot
(recurrent matrices, the last inputs of short convolutions). Slots are handed out by the same scheduler that hands out pages.
"""
from __future__ import annotations

from typing import List, Sequence

import torch


class PageAllocator:
    """LIFO free list over page ids [first, first + count): freed pages are handed out again first, so block tables become
    non-contiguous as soon as requests of different lengths come and go."""

    def __init__(self, count: int, first: int = 0):
        self.count = count
        self._free: List[int] = list(range(first + count - 1, first - 1, -1))

    def available(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise RuntimeError(f"page pool exhausted: {n} pages wanted, {len(self._free)} free")
        return [self._free.pop() for _ in range(n)]

    def give(self, pages: Sequence[int]):
        self._free.extend(reversed(list(pages)))


class PagedLatentCache:
    """pools[layer]: [pages, page_size, width[layer]] of `dtype`; block_table int32 [slots, max_pages] on the device with a
    host mirror. Rows of the table that hold no page point at page `scratch` (never read: a row only reads positions it or an
    earlier step of its request has written)."""

    def __init__(self, widths: Sequence[int], n_pages: int, n_slots: int, page_size: int, dtype: torch.dtype, device,
                 max_pages_per_slot: int = 0):
        self.page_size, self.n_slots, self.n_pages = page_size, n_slots, n_pages
        self.max_pages = max_pages_per_slot or n_pages
        self.capacity = self.max_pages * page_size  # longest sequence one slot can hold
        self.pools = [torch.zeros(n_pages, page_size, w, device=device, dtype=dtype) if w > 0 else None for w in widths]
        self.scratch = 0
        self.table_host = torch.zeros(n_slots, self.max_pages, dtype=torch.int32)
        self.block_table = self.table_host.to(device)
        self.host_lens = [0] * n_slots
        self._dirty = False

    def set_pages(self, slot: int, first: int, pages: Sequence[int]):
        """Table entries first.. of `slot` <- pages (host mirror; `sync` uploads)."""
        if pages:
            self.table_host[slot, first:first + len(pages)] = torch.tensor(list(pages), dtype=torch.int32)
            self._dirty = True

    def clear_slot(self, slot: int):
        self.table_host[slot].fill_(self.scratch)
        self.host_lens[slot] = 0
        self._dirty = True

    def sync(self):
        if self._dirty:
            self.block_table.copy_(self.table_host, non_blocking=False)
            self._dirty = False

    def gather(self, layer: int, slot: int) -> torch.Tensor:
        """Contiguous rows [len, width] of one slot - for tests and debugging."""
        n = self.host_lens[slot]
        pages = self.table_host[slot, : (n + self.page_size - 1) // self.page_size].long().to(self.pools[layer].device)
        return self.pools[layer][pages].reshape(-1, self.pools[layer].shape[-1])[:n]


class PagedStateCache(PagedLatentCache):
    """PagedLatentCache + states[layer][name]: fp32 [slots, *shape] for every entry of state_shapes[layer] ({} for a layer without
    state). A request's state lives in its slot from admission to release. The kernels that carry a state start from zero when a
    portion begins at position 0, so a slot needs no clearing when it changes hands; `poison_slot` overwrites a slot's states
    with NaN, which makes any read of a previous owner's state visible (tests, debugging)."""

    def __init__(self, widths: Sequence[int], state_shapes: Sequence[dict], n_pages: int, n_slots: int, page_size: int,
                 dtype: torch.dtype, device, max_pages_per_slot: int = 0):
        super().__init__(widths, n_pages, n_slots, page_size, dtype, device, max_pages_per_slot)
        self.states = [{name: torch.zeros(n_slots, *shape, device=device, dtype=torch.float32) for name, shape in shapes.items()}
                       for shapes in state_shapes]

    def poison_slot(self, slot: int):
        for layer in self.states:
            for t in layer.values():
                t[slot].fill_(float("nan"))

    def state_bytes_per_slot(self) -> int:
        return sum(t[0].numel() * 4 for layer in self.states for t in layer.values())
