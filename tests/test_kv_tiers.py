"""Host and disk tiers of the prefix cache: pages evicted from the device pool come back on a later hit."""

import numpy as np
import torch

from modular_b200.entrypoints.llm import LLM
from modular_b200.kv_cache.manager import KVCacheParams, PagedKVCacheManager
from modular_b200.kv_cache.tiers import TieredKVStore
from modular_b200.models.llama3 import Llama3Config
from modular_b200.pipelines.context import SamplingParams, TextContext


def test_tiered_store_lru_and_demotion(tmp_path):
    st = TieredKVStore((2, 3, 4), torch.float32, host_pages=2, disk_pages=2, disk_dir=str(tmp_path))
    pages = [torch.full((2, 3, 4), float(i)) for i in range(5)]
    for i, p in enumerate(pages):
        assert st.offload(p, 100 + i, 99 + i if i else None)
    # 2 on the host (the newest), 2 in the file, the oldest dropped
    assert st.host_used == 2 and st.disk_used == 2 and st.dropped == 1
    assert 100 not in st and 101 in st and 104 in st
    dst = torch.empty(2, 3, 4)
    assert st.onload(104, dst) == (103,) and torch.equal(dst, pages[4])      # host hit
    assert st.onload(101, dst) == (100,) and torch.equal(dst, pages[1])      # disk hit
    assert st.onload(100, dst) is None
    assert st.host_hits == 1 and st.disk_hits == 1
    st.close()


def _ctx(rid, toks, max_len=4096):
    return TextContext.from_prompt(np.asarray(toks, dtype=np.int64), max_len, rid, SamplingParams(), ())


def test_manager_reloads_evicted_prefix_from_host():
    kvp = KVCacheParams(n_layers=2, n_kv_heads=2, head_dim=8, page_size=16, dtype=torch.float32)
    mgr = PagedKVCacheManager(kvp, num_pages=6, device="cpu", host_pages=8)     # 5 usable device pages
    rng = np.random.default_rng(0)
    a = rng.integers(0, 1000, 16 * 3 + 1)
    ca = _ctx("a", a)
    mgr.claim(ca)
    mgr.alloc(ca)
    blocks_a = list(mgr.blocks_of("a"))
    for i, b in enumerate(blocks_a[:3]):
        mgr.kv[b].fill_(float(i + 1))                   # stand-in for the prefill's KV
    ca.tokens.advance_processed()
    mgr.step(ca)
    mgr.release("a")
    assert mgr.pool.cached_blocks == 3
    # a second request needs every device page: a's cached pages are evicted -> host tier
    cb = _ctx("b", rng.integers(1000, 2000, 16 * 5))
    mgr.claim(cb)
    mgr.alloc(cb)
    assert mgr.tiers.offloaded == 3 and mgr.pool.cached_blocks == 0
    mgr.kv.zero_()
    mgr.release("b")
    # the first prompt again: all three pages come back from the host
    ca2 = _ctx("a2", a)
    mgr.claim(ca2)
    mgr.alloc(ca2)
    assert mgr.tier_hit_tokens == 48 and mgr.prefix_hit_tokens == 48
    assert ca2.tokens.active_length == 1
    for i, b in enumerate(mgr.blocks_of("a2")[:3]):
        assert torch.all(mgr.kv[b] == float(i + 1))


def test_generation_is_unchanged_by_a_round_trip_through_the_host_tier():
    cfg = Llama3Config.tiny()
    prompt = list(np.random.default_rng(3).integers(5, 200, 40))
    other = [list(np.random.default_rng(10 + i).integers(5, 200, 60)) for i in range(3)]
    sp = SamplingParams(max_new_tokens=6, temperature=0.0, ignore_eos=True)

    def run(host_gb):
        llm = LLM(cfg, device="cpu", max_length=128, max_batch_size=2, page_size=16, num_kv_pages=9,
                  host_kvcache_swap_space_gb=host_gb, seed=1)
        first = llm.generate([prompt], sp)[0].tokens
        for o in other:                                  # push the first prompt's pages out of the device pool
            llm.generate([o], sp)
        again = llm.generate([prompt], sp)[0].tokens
        return first, again, llm.kv

    f0, a0, kv0 = run(0.0)
    f1, a1, kv1 = run(0.001)
    assert f0 == a0 == f1 == a1
    assert kv0.tiers is None
    assert kv1.tiers.offloaded > 0 and kv1.tier_hit_tokens >= 32
