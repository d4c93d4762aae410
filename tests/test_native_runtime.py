"""Native host runtime (csrc/runtime): thread pool + futures, MPSC ring, blob cache, and their users."""

import threading
import time

import numpy as np
import pytest
import torch

from modular_b200._native import lib


def test_thread_pool_futures_and_parallel_memcpy():
    L = lib()
    pool = L.ThreadPool(4)
    assert pool.size() == 4
    hits, lock = [], threading.Lock()

    def job(i):
        def run():
            with lock:
                hits.append(i)
        return run

    futs = [pool.submit(job(i)) for i in range(64)]
    assert all(f.wait(5.0) and f.ok() for f in futs) and sorted(hits) == list(range(64))

    def boom():
        raise RuntimeError("task failed")

    f = pool.submit(boom)
    assert f.wait(5.0) and not f.ok() and "task failed" in f.error()
    src = np.random.default_rng(0).integers(0, 255, size=(37 << 20) + 123, dtype=np.uint8)
    dst = np.zeros_like(src)
    pool.parallel_memcpy(dst.ctypes.data, src.ctypes.data, src.nbytes)
    assert np.array_equal(dst, src)
    rev = src[::-1].copy()        # must stay alive until the asynchronous copy has run
    g = pool.submit_memcpy(dst.ctypes.data, rev.ctypes.data, 1024)
    assert g.wait(5.0) and g.ok() and np.array_equal(dst[:1024], rev[:1024])


def test_mpsc_ring_many_producers_one_consumer():
    L = lib()
    ring = L.MpscRing(256)
    assert ring.capacity() == 256 and ring.pop() is None
    n_prod, per = 4, 2000
    got = []

    def producer(p):
        for i in range(per):
            v = (p << 32) | i
            while not ring.push(v):
                time.sleep(0)

    ts = [threading.Thread(target=producer, args=(p,)) for p in range(n_prod)]
    for t in ts:
        t.start()
    deadline = time.time() + 30
    while len(got) < n_prod * per and time.time() < deadline:
        v = ring.pop()
        if v is None:
            time.sleep(0)
        else:
            got.append(v)
    for t in ts:
        t.join()
    assert len(got) == n_prod * per
    for p in range(n_prod):       # per-producer order is preserved
        seq = [v & 0xFFFFFFFF for v in got if v >> 32 == p]
        assert seq == list(range(per))
    for i in range(256):
        assert ring.push(i)
    assert not ring.push(999)     # full: refused, not overwritten


def test_blob_cache_memory_then_disk(tmp_path):
    L = lib()
    c = L.BlobCache(str(tmp_path / "blobs"), 1 << 16)
    blob = bytes(range(256)) * 64
    key = L.BlobCache.content_key(blob)
    assert len(key) >= 16 and key == L.BlobCache.content_key(blob) and key != L.BlobCache.content_key(blob + b"x")
    assert c.get(key) is None
    c.put(key, blob)
    assert c.get(key) == blob
    for i in range(16):           # push the first blob out of the memory tier
        c.put(f"k{i}", bytes([i]) * (1 << 13))
    assert c.get(key) == blob     # served from the directory
    c2 = L.BlobCache(str(tmp_path / "blobs"), 1 << 16)
    assert c2.get(key) == blob and c2.get("missing") is None


def test_kv_tier_page_copies_run_on_the_native_pool(tmp_path):
    """Pages of several megabytes go host -> file -> host through ThreadPool.parallel_memcpy."""
    from modular_b200.kv_cache import tiers

    store = tiers.TieredKVStore((2, 4, 8, 64, 128), torch.bfloat16, host_pages=1, disk_pages=2,
                                disk_dir=str(tmp_path), pin=False)
    assert tiers._copy_pool() is not None
    pages = [torch.randn(2, 4, 8, 64, 128).to(torch.bfloat16) for _ in range(3)]
    for i, p in enumerate(pages):
        assert store.offload(p, 100 + i, None)
    assert store.demoted == 2 and store.host_used == 1 and store.disk_used == 2
    for i, p in enumerate(pages):
        out = torch.empty_like(p)
        assert store.onload(100 + i, out) is not None and torch.equal(out, p)
    assert store.disk_hits == 2 and store.host_hits == 1
    store.close()
