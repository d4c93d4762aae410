"""Block pool: reference-counted KV pages with an LRU of evictable cached pages.

A page is in exactly one of three states:

* **in use** - ``ref > 0``; owned by one or more requests (shared when a prefix was reused)
* **cached-free** - ``ref == 0`` but still registered under its content hash; it sits in
  the LRU free queue and can be revived by a prefix hit or evicted by an allocation
* **free** - no hash, at the cold end of the queue

Behavioural counterpart: max/python/max/pipelines/kv_cache/paged_kv_cache/block_pool.py:37
and the doubly-linked free queue in block_utils.py:324.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Optional


class InsufficientBlocksError(RuntimeError):
    """Raised when an allocation needs more pages than are free or evictable."""


@dataclass
class KVCacheBlock:
    block_id: int
    ref: int = 0
    block_hash: Optional[int] = None
    parent_hash: Optional[int] = None


class BlockPool:
    def __init__(self, num_blocks: int, enable_prefix_caching: bool = True, reserve_null: bool = True):
        if num_blocks < 2:
            raise ValueError("need at least two blocks")
        self.num_blocks = num_blocks
        self.enable_prefix_caching = enable_prefix_caching
        self.blocks = [KVCacheBlock(i) for i in range(num_blocks)]
        first = 1 if reserve_null else 0  # block 0 backs padded / dummy sequences
        self.null_block = 0 if reserve_null else -1
        # free queue: oldest first; popitem(last=False) evicts LRU
        self._free: "OrderedDict[int, None]" = OrderedDict((i, None) for i in range(first, num_blocks))
        self._by_hash: dict[int, int] = {}
        self.evictions = 0
        # called as on_evict(block_id, block_hash, parent_hash) just before a cached page's content is
        # given up (the lower cache tiers copy the page out here)
        self.on_evict = None

    # ---- introspection
    @property
    def usable_blocks(self) -> int:
        return self.num_blocks - (1 if self.null_block == 0 else 0)

    @property
    def free_blocks(self) -> int:
        return len(self._free)

    @property
    def used_blocks(self) -> int:
        return self.usable_blocks - len(self._free)

    @property
    def cached_blocks(self) -> int:
        return len(self._by_hash)

    # ---- allocation
    def allocate(self, n: int) -> list[int]:
        if n > len(self._free):
            raise InsufficientBlocksError(f"need {n} blocks, {len(self._free)} free")
        out = []
        for _ in range(n):
            bid, _ = self._free.popitem(last=False)
            blk = self.blocks[bid]
            if blk.block_hash is not None:
                # evict the cached content
                if self._by_hash.get(blk.block_hash) == bid:
                    del self._by_hash[blk.block_hash]
                    if self.on_evict is not None:
                        self.on_evict(bid, blk.block_hash, blk.parent_hash)
                blk.block_hash = None
                blk.parent_hash = None
                self.evictions += 1
            blk.ref = 1
            out.append(bid)
        return out

    def lookup(self, block_hash: int) -> Optional[int]:
        if not self.enable_prefix_caching:
            return None
        return self._by_hash.get(block_hash)

    def acquire_cached(self, bid: int) -> None:
        """Take a reference on a page found through ``lookup`` (revives it if it was free)."""
        blk = self.blocks[bid]
        if blk.ref == 0:
            self._free.pop(bid, None)
        blk.ref += 1

    def commit(self, bid: int, block_hash: int, parent_hash: Optional[int]) -> int:
        """Register a full page under its hash. Returns the canonical page id for that hash
        (an older identical page wins; the caller may then swap to it)."""
        if not self.enable_prefix_caching:
            return bid
        existing = self._by_hash.get(block_hash)
        if existing is not None and existing != bid:
            return existing
        blk = self.blocks[bid]
        blk.block_hash = block_hash
        blk.parent_hash = parent_hash
        self._by_hash[block_hash] = bid
        return bid

    def release(self, bid: int) -> None:
        blk = self.blocks[bid]
        if blk.ref <= 0:
            raise RuntimeError(f"double free of block {bid}")
        blk.ref -= 1
        if blk.ref == 0:
            self._free[bid] = None
            if blk.block_hash is None:
                self._free.move_to_end(bid, last=False)  # content-less pages are reused first

    def reset_prefix_cache(self) -> bool:
        """Drop every cached hash. Pages still referenced keep their data but lose the hash."""
        for blk in self.blocks:
            blk.block_hash = None
            blk.parent_hash = None
        self._by_hash.clear()
        return True
