"""Host and disk tiers behind the device prefix cache.

When the device pool evicts a cached page (a full page registered under its chained content hash) the
page's bytes move to a pinned host buffer instead of being lost; when the host buffer is full its
least-recently-used page moves on to a memory-mapped file. A later request whose prompt hashes to a
page that lives in a lower tier gets it copied back into a freshly allocated device page, so the
prefill of that page is skipped exactly as on a device hit.

The device-to-host copy is enqueued on the current stream *before* any kernel that could overwrite the
evicted page (allocation happens on the host ahead of the step's launches), so no extra
synchronisation is needed; the host-to-device copy of an onload is likewise ordered before the step
that reads the page. Demotion host -> disk waits for the device-to-host copy event of that slot. Pages
are several megabytes (16 MiB for Llama-3.1-8B with 128-token pages), so the host <-> file copies run on the
native thread pool (``ThreadPool.parallel_memcpy``: chunks on several threads, no GIL held) when the native
library is loaded, and through numpy otherwise.

Reference counterparts: the host/disk tiers of max/python/max/pipelines/kv_cache/paged_kv_cache/
block_manager.py:262 (offload queue, ``reuse_blocks_from_prefix_cache`` :457) and the tiered connector
wrapper kv_cache/connectors/rust_tier_connector.py (the library behind it is not in the tree).
"""

from __future__ import annotations

import os
from collections import OrderedDict
from typing import Optional

import numpy as np
import torch

__all__ = ["TieredKVStore"]

_POOL = None


def _copy_pool():
    """Process-wide native thread pool for page copies (None when the native library is unavailable)."""
    global _POOL
    if _POOL is None:
        try:
            from .._native import lib
            _POOL = lib().ThreadPool(min(8, max(2, (os.cpu_count() or 4) // 2)))
        except Exception:  # noqa: BLE001
            _POOL = False
    return _POOL or None


def _memcpy(dst: np.ndarray, src: np.ndarray) -> None:
    """dst[:] = src for contiguous uint8 arrays of equal size, in parallel when the pool exists."""
    pool = _copy_pool()
    if pool is not None and dst.flags.c_contiguous and src.flags.c_contiguous and dst.nbytes >= (1 << 20):
        pool.parallel_memcpy(dst.ctypes.data, src.ctypes.data, dst.nbytes)
    else:
        dst[:] = src


class TieredKVStore:
    """LRU stores of evicted pages keyed by content hash: pinned host memory, then a file."""

    def __init__(self, page_shape: tuple, dtype: torch.dtype, host_pages: int, disk_pages: int = 0,
                 disk_dir: Optional[str] = None, pin: bool = True):
        self.page_shape = tuple(page_shape)
        self.dtype = dtype
        self.host_pages = int(host_pages)
        self.disk_pages = int(disk_pages) if disk_dir else 0
        pin = pin and torch.cuda.is_available()
        self.host = torch.empty((max(self.host_pages, 1),) + self.page_shape, dtype=dtype, pin_memory=pin)
        self._host_lru: "OrderedDict[int, int]" = OrderedDict()      # hash -> host slot (oldest first)
        self._host_free = list(range(self.host_pages))
        self._host_parent: dict[int, Optional[int]] = {}
        self._host_event: dict[int, "torch.cuda.Event"] = {}         # slot -> D2H completion
        self._disk = None
        self._disk_lru: "OrderedDict[int, int]" = OrderedDict()
        self._disk_free = list(range(self.disk_pages))
        self._disk_parent: dict[int, Optional[int]] = {}
        if self.disk_pages:
            os.makedirs(disk_dir, exist_ok=True)
            self._page_bytes = int(np.prod(self.page_shape)) * torch.empty(0, dtype=dtype).element_size()
            self._disk_path = os.path.join(disk_dir, f"kv_tier_{os.getpid()}_{id(self):x}.bin")
            self._disk = np.memmap(self._disk_path, dtype=np.uint8, mode="w+",
                                   shape=(self.disk_pages, self._page_bytes))
        # counters
        self.offloaded = 0
        self.host_hits = 0
        self.disk_hits = 0
        self.demoted = 0
        self.dropped = 0

    def _stage(self) -> torch.Tensor:
        """One pinned page used to bring a disk page up (the copy to the device is synchronous from pinned
        memory only once the page has been read, so one buffer is enough)."""
        if getattr(self, "_stage_buf", None) is None:
            self._stage_buf = torch.empty(self.page_shape, dtype=self.dtype, pin_memory=self.host.is_pinned())
        elif self._stage_buf.is_pinned() and torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()      # the previous onload from this buffer has left it
        return self._stage_buf

    @property
    def host_used_pct(self) -> float:
        return len(self._host_lru) / self.host_pages if self.host_pages else 0.0

    @property
    def disk_used_pct(self) -> float:
        return len(self._disk_lru) / self.disk_pages if self.disk_pages else 0.0

    # ------------------------------------------------------------------ queries
    def __contains__(self, block_hash: int) -> bool:
        return block_hash in self._host_lru or block_hash in self._disk_lru

    @property
    def host_used(self) -> int:
        return len(self._host_lru)

    @property
    def disk_used(self) -> int:
        return len(self._disk_lru)

    # ------------------------------------------------------------------ offload (device -> host)
    def _host_slot(self) -> Optional[int]:
        if self._host_free:
            return self._host_free.pop()
        if not self._host_lru:
            return None
        old_hash, slot = self._host_lru.popitem(last=False)
        parent = self._host_parent.pop(old_hash, None)
        self._demote(old_hash, parent, slot)
        return slot

    def _demote(self, block_hash: int, parent: Optional[int], slot: int) -> None:
        """Host LRU victim: to the file if there is one, else dropped."""
        ev = self._host_event.pop(slot, None)
        if self._disk is None:
            self.dropped += 1
            return
        if ev is not None:
            ev.synchronize()
        if self._disk_free:
            dslot = self._disk_free.pop()
        else:
            old, dslot = self._disk_lru.popitem(last=False)
            self._disk_parent.pop(old, None)
            self.dropped += 1
        _memcpy(self._disk[dslot], self.host[slot].view(torch.uint8).reshape(-1).numpy())
        self._disk_lru[block_hash] = dslot
        self._disk_parent[block_hash] = parent
        self.demoted += 1

    def offload(self, page: torch.Tensor, block_hash: int, parent_hash: Optional[int]) -> bool:
        """Keep a copy of an evicted device page. Returns False when there is no host tier."""
        if self.host_pages <= 0:
            return False
        if block_hash in self._host_lru:
            self._host_lru.move_to_end(block_hash)
            return True
        if block_hash in self._disk_lru:
            return True
        slot = self._host_slot()
        if slot is None:
            return False
        self.host[slot].copy_(page, non_blocking=True)
        if page.is_cuda:
            ev = torch.cuda.Event()
            ev.record()
            self._host_event[slot] = ev
        self._host_lru[block_hash] = slot
        self._host_parent[block_hash] = parent_hash
        self.offloaded += 1
        return True

    # ------------------------------------------------------------------ onload (host/disk -> device)
    def onload(self, block_hash: int, dst: torch.Tensor) -> Optional[Optional[int]]:
        """Copy the page stored under ``block_hash`` into ``dst`` (a device page). Returns a one-element
        tuple with the page's parent hash on a hit, None on a miss."""
        slot = self._host_lru.get(block_hash)
        if slot is not None:
            ev = self._host_event.get(slot)
            if ev is not None:
                ev.synchronize()      # the page may still be on its way down
            dst.copy_(self.host[slot], non_blocking=True)
            self._host_lru.move_to_end(block_hash)
            self.host_hits += 1
            return (self._host_parent.get(block_hash),)
        dslot = self._disk_lru.get(block_hash)
        if dslot is not None:
            stage = self._stage()
            _memcpy(stage.view(torch.uint8).reshape(-1).numpy(), self._disk[dslot])
            dst.copy_(stage)
            self._disk_lru.move_to_end(block_hash)
            self.disk_hits += 1
            return (self._disk_parent.get(block_hash),)
        return None

    def clear(self) -> None:
        self._host_lru.clear()
        self._host_parent.clear()
        self._host_event.clear()
        self._host_free = list(range(self.host_pages))
        self._disk_lru.clear()
        self._disk_parent.clear()
        self._disk_free = list(range(self.disk_pages))

    def close(self) -> None:
        if self._disk is not None:
            path = self._disk_path
            del self._disk
            self._disk = None
            try:
                os.remove(path)
            except OSError:
                pass
