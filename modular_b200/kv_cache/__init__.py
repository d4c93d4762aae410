"""Paged KV cache: block pool, prefix caching, per-batch runtime inputs."""

from .block_pool import BlockPool, InsufficientBlocksError, KVCacheBlock
from .manager import KVCacheParams, PagedKVCacheManager, hash_token_blocks

__all__ = ["BlockPool", "InsufficientBlocksError", "KVCacheBlock", "KVCacheParams",
           "PagedKVCacheManager", "hash_token_blocks"]
