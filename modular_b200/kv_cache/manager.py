"""Paged KV cache manager with prefix caching.

API follows the reference's ``PagedKVCacheManager``
(max/python/max/pipelines/kv_cache/paged_kv_cache/cache_manager.py:220):

    claim(ctx)         register a request
    alloc(ctx)         reuse cached prefix pages, then allocate pages for the active window
    runtime_inputs(…)  block table + lengths for a batch (numpy; the pipeline packs and uploads)
    step(ctx)          after a forward pass: commit pages that became full to the prefix cache
    release(ctx)       drop the request's references (cached pages stay evictable)

Device layout of the cache tensor (one allocation):

    [num_pages, 2 (K,V), num_layers, n_kv_heads, page_size, head_dim]   (MHA/GQA)
    [num_pages, 1,       num_layers, 1,          page_size, kv_lora + rope]  (MLA latent)

so a (page, plane, layer, head) slice is one contiguous ``page_size x head_dim`` tile that a
bulk copy or a TMA box can fetch in one piece, and a whole page (all layers) is contiguous
for offload and transfer.

Block hashes are chained: ``h_i = H(h_{i-1} || tokens of page i)`` with the request's salt
folded into the seed; the final token of a prompt is never hashed, so a full-prompt hit
still leaves one token to run (reference: block_manager.py:62, :91-98).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, Optional, Sequence

import numpy as np
import torch

from .._native import lib as _lib
from ..pipelines.context import FUTURE_TOKEN, TextContext
from .block_pool import BlockPool, InsufficientBlocksError

__all__ = ["KVCacheParams", "PagedKVCacheManager", "InsufficientBlocksError", "hash_token_blocks"]


def _py_hash_blocks(tokens: np.ndarray, block: int, parent: int, seed: int) -> list[int]:
    import hashlib

    out, h = [], parent
    for b in range(0, len(tokens) - block + 1, block):
        d = hashlib.blake2b(tokens[b : b + block].tobytes(), digest_size=8,
                            key=int(h ^ seed).to_bytes(8, "little", signed=False)).digest()
        h = int.from_bytes(d, "little")
        out.append(h)
    return out


def hash_token_blocks(tokens: np.ndarray, block: int, parent: int = 0, seed: int = 0) -> list[int]:
    """Chained 64-bit hashes of consecutive full pages of ``tokens`` (native when available)."""
    tokens = np.ascontiguousarray(tokens, dtype=np.int64)
    native = _lib(required=False)
    if native is not None:
        return list(native.hash_token_blocks(tokens, block, parent & (2**64 - 1), seed & (2**64 - 1)))
    return _py_hash_blocks(tokens, block, parent & (2**64 - 1), seed & (2**64 - 1))


@dataclass
class KVCacheParams:
    """Shape of the cache. ``is_mla`` stores one latent "head" per token and no V plane."""

    n_layers: int
    n_kv_heads: int
    head_dim: int
    page_size: int = 128
    dtype: torch.dtype = torch.bfloat16
    is_mla: bool = False
    enable_prefix_caching: bool = True

    @property
    def kv_dim(self) -> int:
        return 1 if self.is_mla else 2

    @property
    def bytes_per_page(self) -> int:
        el = torch.empty(0, dtype=self.dtype).element_size()
        return self.kv_dim * self.n_layers * self.n_kv_heads * self.page_size * self.head_dim * el

    def shape(self, num_pages: int) -> tuple:
        return (num_pages, self.kv_dim, self.n_layers, self.n_kv_heads, self.page_size, self.head_dim)

    def compute_num_device_blocks(self, available_bytes: int, max_batch: int = 0,
                                  max_len: int = 0) -> int:
        n = int(available_bytes // self.bytes_per_page)
        if max_batch and max_len:
            cap = max_batch * ((max_len + self.page_size - 1) // self.page_size) + 1
            n = min(n, cap)
        return max(n, 2)


@dataclass
class _ReqState:
    blocks: list[int] = field(default_factory=list)
    hashes: list[int] = field(default_factory=list)   # hashes of committed (full, hashed) pages
    n_committed: int = 0
    salt: int = 0
    prefix_hit_tokens: int = 0
    prefix_checked: bool = False


class PagedKVCacheManager:
    def __init__(self, params: KVCacheParams, num_pages: int, device="cpu", max_seq_len: int = 0,
                 allocate: bool = True, host_pages: int = 0, disk_pages: int = 0,
                 disk_dir: Optional[str] = None):
        self.params = params
        self.page_size = params.page_size
        self.num_pages = num_pages
        self.device = torch.device(device)
        self.pool = BlockPool(num_pages, params.enable_prefix_caching)
        self.max_pages_per_seq = ((max_seq_len + self.page_size - 1) // self.page_size
                                  if max_seq_len else num_pages)
        self.kv = (torch.zeros(params.shape(num_pages), dtype=params.dtype, device=self.device)
                   if allocate else None)
        self._req: dict[str, _ReqState] = {}
        # lower tiers for evicted prefix pages (pinned host memory, then a file); see tiers.py
        self.tiers = None
        if allocate and params.enable_prefix_caching and host_pages > 0:
            from .tiers import TieredKVStore
            self.tiers = TieredKVStore(params.shape(1)[1:], params.dtype, host_pages, disk_pages, disk_dir)
            self.pool.on_evict = self._offload_page
        # metrics
        self.prefix_query_tokens = 0
        self.prefix_hit_tokens = 0
        self.tier_hit_tokens = 0       # part of prefix_hit_tokens that came back from host memory or disk
        self.preemptions = 0

    # ------------------------------------------------------------ bookkeeping
    def claim(self, ctx: TextContext, salt: int = 0) -> None:
        if ctx.request_id in self._req:
            raise ValueError(f"request {ctx.request_id} already claimed")
        self._req[ctx.request_id] = _ReqState(salt=salt)

    def contains(self, request_id: str) -> bool:
        return request_id in self._req

    def release(self, request_id: str) -> None:
        st = self._req.pop(request_id, None)
        if st is None:
            return
        # release in reverse so that leaf pages are evicted before their parents
        for bid in reversed(st.blocks):
            self.pool.release(bid)

    def reset_prefix_cache(self) -> bool:
        if self.tiers is not None:
            self.tiers.clear()
        return self.pool.reset_prefix_cache()

    def _offload_page(self, bid: int, block_hash: int, parent_hash) -> None:
        self.tiers.offload(self.kv[bid], block_hash, parent_hash)

    def _onload_page(self, block_hash: int, parent_hash) -> Optional[int]:
        """Bring a page of a lower tier back into a fresh device page; None if it cannot be placed."""
        try:
            bid = self.pool.allocate(1)[0]
        except InsufficientBlocksError:
            return None
        if self.tiers.onload(block_hash, self.kv[bid]) is None:   # evicted from the tier by that allocation
            self.pool.release(bid)
            return None
        self.pool.commit(bid, block_hash, parent_hash)
        return bid

    @property
    def free_blocks(self) -> int:
        return self.pool.free_blocks

    @property
    def used_blocks_pct(self) -> float:
        return self.pool.used_blocks / max(1, self.pool.usable_blocks)

    @property
    def cache_hit_rate(self) -> float:
        return self.prefix_hit_tokens / max(1, self.prefix_query_tokens)

    def blocks_of(self, request_id: str) -> list[int]:
        return self._req[request_id].blocks

    # ------------------------------------------------------------ allocation
    def _reuse_prefix(self, ctx: TextContext, st: _ReqState) -> None:
        toks = ctx.tokens.all
        hashable = len(toks) - 1  # never hash the final token
        n_full = hashable // self.page_size
        self.prefix_query_tokens += len(toks)
        if n_full == 0 or not self.params.enable_prefix_caching:
            return
        known = toks[: n_full * self.page_size]
        if (known == FUTURE_TOKEN).any():
            return
        hashes = hash_token_blocks(known, self.page_size, 0, st.salt)
        parent = None
        for h in hashes:
            bid = self.pool.lookup(h)
            if bid is None:
                if self.tiers is None or h not in self.tiers:
                    break
                bid = self._onload_page(h, parent)
                if bid is None:
                    break
                self.tier_hit_tokens += self.page_size
            else:
                self.pool.acquire_cached(bid)
            st.blocks.append(bid)
            st.hashes.append(h)
            parent = h
        st.n_committed = len(st.blocks)
        hit = st.n_committed * self.page_size
        if hit:
            # the active window starts after the cached prefix; at least one token remains
            ctx.tokens.skip_processing(min(hit, ctx.tokens.active_length - 1))
            st.prefix_hit_tokens = hit
            self.prefix_hit_tokens += hit

    def lookup_prefix(self, ctx: TextContext) -> int:
        """Once per (re)claimed request: attach cached pages matching the prompt prefix and move
        the active window past them. Returns the number of tokens served from the cache."""
        st = self._req[ctx.request_id]
        if st.prefix_checked:
            return st.prefix_hit_tokens
        st.prefix_checked = True
        if not st.blocks and ctx.tokens.processed == 0:
            self._reuse_prefix(ctx, st)
        return st.prefix_hit_tokens

    def alloc(self, ctx: TextContext, extra_tokens: int = 0) -> None:
        """Make sure pages exist for every token up to the end of the active window
        (+ ``extra_tokens`` look-ahead). Raises InsufficientBlocksError without side effects
        on the request's existing pages."""
        st = self._req[ctx.request_id]
        self.lookup_prefix(ctx)
        need_tokens = ctx.tokens.active_end + extra_tokens
        need = (need_tokens + self.page_size - 1) // self.page_size - len(st.blocks)
        if need > 0:
            if len(st.blocks) + need > self.max_pages_per_seq:
                raise InsufficientBlocksError(
                    f"request {ctx.request_id} needs {len(st.blocks) + need} pages; the per-sequence "
                    f"limit is {self.max_pages_per_seq}")
            st.blocks.extend(self.pool.allocate(need))

    def can_alloc(self, ctx: TextContext, extra_tokens: int = 0) -> bool:
        st = self._req.get(ctx.request_id)
        have = len(st.blocks) if st else 0
        need = (ctx.tokens.active_end + extra_tokens + self.page_size - 1) // self.page_size - have
        return need <= self.pool.free_blocks

    # ------------------------------------------------------------ after a forward pass
    def step(self, ctx: TextContext) -> None:
        """Commit pages that are now full and whose tokens are all known."""
        if not self.params.enable_prefix_caching:
            return
        st = self._req.get(ctx.request_id)
        if st is None:
            return
        toks = ctx.tokens.all
        known_len = len(toks) - ctx.pending_future
        n_full = min(ctx.tokens.processed, known_len) // self.page_size
        if n_full <= st.n_committed:
            return
        parent = st.hashes[-1] if st.hashes else 0
        seg = toks[st.n_committed * self.page_size : n_full * self.page_size]
        new_hashes = hash_token_blocks(seg, self.page_size, parent, st.salt)
        for i, h in enumerate(new_hashes):
            idx = st.n_committed + i
            self.pool.commit(st.blocks[idx], h, parent)
            st.hashes.append(h)
            parent = h
        st.n_committed = n_full

    # ------------------------------------------------------------ batch inputs
    def runtime_inputs(self, ctxs: Sequence[TextContext], bt_stride: int = 0):
        """Returns (block_table int32 [B, bt_stride], kv_len int32 [B]) for a batch; kv_len
        counts every token that will be in the cache after this pass."""
        B = len(ctxs)
        if bt_stride <= 0:
            bt_stride = max((len(self._req[c.request_id].blocks) for c in ctxs), default=1)
        table = np.zeros((B, bt_stride), dtype=np.int32)
        kv_len = np.empty(B, dtype=np.int32)
        for i, c in enumerate(ctxs):
            blocks = self._req[c.request_id].blocks
            n = min(len(blocks), bt_stride)
            table[i, :n] = blocks[:n]
            kv_len[i] = c.tokens.active_end
        return table, kv_len

    def slot_mapping(self, ctx: TextContext) -> np.ndarray:
        """Flat cache slot (page * page_size + offset) of every active token."""
        st = self._req[ctx.request_id]
        pos = np.arange(ctx.tokens.processed, ctx.tokens.active_end, dtype=np.int64)
        blocks = np.asarray(st.blocks, dtype=np.int64)
        return blocks[pos // self.page_size] * self.page_size + pos % self.page_size

    def layer_views(self, layer: int):
        """(k_cache, v_cache) views [pages, n_kv, page_size, head_dim] of one layer."""
        if self.params.is_mla:
            return self.kv[:, 0, layer], None
        return self.kv[:, 0, layer], self.kv[:, 1, layer]
