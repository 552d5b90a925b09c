"""The cache manager: device pools for every group of layers with the same
need, and (through the native runtime) the pages and the state slot each live
request holds.

Paged groups: keys and values of all order items with the same
(kv heads, head size, window, value size), pool [items, pages, kv heads, page size, head
size] each for K and V (V with rows of the value size where that differs) (K alone for a group whose rows are keys and values at once); one page id of a group means that page in every item
of the group. The reference sizes one pool for all layers, convolution layers
included (tools/infer/src/main.rs:386-392); here only items that keep keys
have pages. State groups: [items, slots, *shape] for order items with
fixed-size state; a request's slot is zeroed when it is admitted.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np
import torch

from ..parts.base import CacheBinding, FixedState, PagedKV
from .native import CacheError, checked, int_array, last_error, lib


class OutOfPages(CacheError):
    pass


class CacheManager:
    def __init__(self, needs: Sequence, cache_of: Sequence[Optional[int]], page_size: int, total_blocks,
                 num_slots: int, dtype: torch.dtype, device):
        """needs[i]: PagedKV | FixedState | None for order item i (None: no cache of
        its own), or a tuple of these for an item that keeps several things; needs beyond the run order belong to
        parts outside the layers (the embedding); cache_of[i]: the item whose cache item i reads, or None.
        total_blocks: pages of every paged group (an int) or one count per group."""
        self.page_size, self.num_slots, self.dtype, self.device = int(page_size), int(num_slots), dtype, torch.device(device)
        self.paged_keys: list[PagedKV] = []
        self.state_keys: list[FixedState] = []
        # per item: (family, group, index in group), a list of these for an item with several needs, or None
        self._item_group: list = []
        members: dict[tuple[str, int], int] = {}

        def place(need):
            if need is None:
                return None
            if isinstance(need, PagedKV):
                fam, keys = "paged", self.paged_keys
            elif isinstance(need, FixedState):
                fam, keys = "state", self.state_keys
            else:
                raise CacheError(f"unknown cache need {need!r}")
            if need not in keys:
                keys.append(need)
            g = keys.index(need)
            idx = members.get((fam, g), 0)
            members[(fam, g)] = idx + 1
            return (fam, g, idx)
        for need in needs:
            self._item_group.append([place(n) for n in need] if isinstance(need, (tuple, list)) else place(need))
        cache_of = list(cache_of) + [None] * (len(needs) - len(cache_of))
        for i, src in enumerate(cache_of):
            if src is not None:
                self._item_group[i] = self._item_group[src]
        self._borrowed = [c is not None for c in cache_of]
        n_paged = len(self.paged_keys)
        if isinstance(total_blocks, int):
            total_blocks = [total_blocks] * n_paged
        if len(total_blocks) != n_paged:
            raise CacheError(f"{len(total_blocks)} page counts for {n_paged} paged groups")
        self.group_pages = [int(p) for p in total_blocks]
        self.k_pools, self.v_pools, self.states = [], [], []
        for g, need in enumerate(self.paged_keys):
            shape = (members[("paged", g)], self.group_pages[g], need.num_kv_heads, self.page_size, need.head_dim)
            self.k_pools.append(torch.zeros(shape, dtype=dtype, device=self.device))
            v_shape = shape[:4] + (need.value_dim or need.head_dim,)
            self.v_pools.append(torch.zeros(v_shape, dtype=dtype, device=self.device) if need.values else None)
        for g, need in enumerate(self.state_keys):
            self.states.append(torch.zeros((members[("state", g)], self.num_slots) + tuple(need.shape),
                                           dtype=need.dtype, device=self.device))
        # A model without paged items (no attention at all) has no page group: its requests hold a slot only.
        windows = [k.window for k in self.paged_keys]
        keeps = [k.keep_first if k.window else 0 for k in self.paged_keys]
        self._h = lib().cellm_cache_create(self.page_size, n_paged, int_array(self.group_pages), int_array(windows),
                                           int_array(keeps), self.num_slots)
        if not self._h:
            raise CacheError(last_error())

    def __del__(self):
        if getattr(self, "_h", None):
            lib().cellm_cache_destroy(self._h)
            self._h = None

    # ------------------------------------------------------------ requests
    @property
    def handle(self):
        return self._h

    def add(self, request_id: int) -> int:
        """Takes a state slot for a new request and zeroes its state; returns the slot."""
        slot = lib().cellm_cache_add(self._h, int(request_id))
        if slot == -2:
            raise OutOfPages("no free state slot")
        checked(slot)
        self.zero_slot(slot)
        return slot

    def zero_slot(self, slot: int) -> None:
        for s in self.states:
            s[:, slot].zero_()

    def has(self, request_id: int) -> bool:
        return bool(lib().cellm_cache_has(self._h, int(request_id)))

    def reserve(self, request_id: int, new_total: int) -> bool:
        return bool(checked(lib().cellm_cache_reserve(self._h, int(request_id), int(new_total))))

    def commit(self, request_id: int, new_total: int) -> None:
        checked(lib().cellm_cache_commit(self._h, int(request_id), int(new_total)))

    def release(self, request_id: int) -> None:
        checked(lib().cellm_cache_release(self._h, int(request_id)))

    def tokens(self, request_id: int) -> int:
        return checked(lib().cellm_cache_tokens(self._h, int(request_id)))

    def slot(self, request_id: int) -> int:
        return checked(lib().cellm_cache_slot(self._h, int(request_id)))

    def block_table(self, request_id: int, group: int, out: Optional[np.ndarray] = None) -> np.ndarray:
        """The request's pages of a paged group, in order; -1 where a page was given back."""
        if out is None:
            out = np.full((self.max_blocks(group),), -1, dtype=np.int32)
        n = checked(lib().cellm_cache_block_table(self._h, int(request_id), int(group),
                                                  out.ctypes.data_as(ctypes.c_void_p), out.shape[0]))
        return out[:n]

    def free_pages(self, group: int = 0) -> int:
        return checked(lib().cellm_cache_free_pages(self._h, group))

    @property
    def free_slots(self) -> int:
        return lib().cellm_cache_free_slots(self._h)

    @property
    def live(self) -> int:
        return lib().cellm_cache_live(self._h)

    def max_blocks(self, group: int) -> int:
        return self.group_pages[group]

    def pages_for(self, group: int, tokens: int, portion: int) -> int:
        return checked(lib().cellm_cache_pages_for(self._h, group, tokens, portion))

    # ------------------------------------------------------------ bindings
    def bindings(self, block_tables: Sequence[torch.Tensor]) -> list[CacheBinding]:
        """One CacheBinding per order item for a step whose block tables
        (one [B, blocks] int32 tensor per paged group) are given."""
        def one(ig, writes: bool) -> CacheBinding:
            if ig is None:
                return CacheBinding()
            fam, g, idx = ig
            if fam == "paged":
                return CacheBinding(need=self.paged_keys[g], writes=writes,
                                    k=self.k_pools[g][idx], v=self.v_pools[g][idx] if self.v_pools[g] is not None else None,
                                    block_table=block_tables[g], page_size=self.page_size, num_pages=self.group_pages[g])
            return CacheBinding(need=self.state_keys[g], writes=writes, state=self.states[g][idx], num_slots=self.num_slots)
        out = []
        for i, ig in enumerate(self._item_group):
            writes = not self._borrowed[i]
            if isinstance(ig, list):
                parts = tuple(one(x, writes) for x in ig)
                out.append(CacheBinding(need=tuple(p.need for p in parts), writes=writes, parts=parts))
            else:
                out.append(one(ig, writes))
        return out

    def bytes_per_token(self) -> int:
        """Bytes of keys and values one token occupies over all paged groups."""
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(p.shape[0] * p.shape[2] * (p.shape[4] + (v.shape[4] if v is not None else 0)) * el
                   for p, v in zip(self.k_pools, self.v_pools))
