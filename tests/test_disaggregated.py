"""Disaggregated prefill/decode on CPU: two engines with separate KV caches joined by a transfer."""

import queue
import time

import numpy as np
import pytest
import torch

from modular_b200.entrypoints.llm import LLM
from modular_b200.models.llama3 import Llama3Config, Llama3Weights
from modular_b200.pipelines.context import SamplingParams
from modular_b200.serve.scheduler.disaggregated import DecodeNode, LocalTransfer, PrefillNode


def _engine(w, cfg, **kw):
    return LLM(cfg, w, device="cpu", dtype=torch.float32, max_length=256, max_batch_size=4, max_batch_input_tokens=48,
               page_size=16, num_kv_pages=64, enable_prefix_caching=False, **kw)


def test_prefill_node_feeds_decode_node():
    cfg = Llama3Config.tiny()
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=0, std=0.05)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (40, 9, 75)]     # 75 is chunked on prefill
    sp = SamplingParams(temperature=0.0, max_new_tokens=7, ignore_eos=True)
    want = [r.tokens for r in _engine(w, cfg).generate(prompts, sp)]
    to_p, from_p = queue.SimpleQueue(), queue.SimpleQueue()
    prefill = PrefillNode(_engine(w, cfg), to_p, from_p, LocalTransfer())
    decode = DecodeNode(_engine(w, cfg), to_p, from_p, LocalTransfer())
    rids = [decode.add_request(p, sp) for p in prompts]
    done = {}
    for _ in range(200):
        prefill.run_iteration()
        for rec in decode.step():
            done[rec.request_id] = rec.tokens
        if not decode.has_unfinished():
            break
    assert [done[r] for r in rids] == want
    assert prefill.completed == 3 and decode.llm.kv.free_blocks == prefill.llm.kv.free_blocks   # everything released
    one = SamplingParams(temperature=0.0, max_new_tokens=1, ignore_eos=True)
    rid = decode.add_request(prompts[1], one)
    prefill.run_iteration()
    recs = decode.step()
    assert [r.request_id for r in recs] == [rid] and recs[0].tokens == want[1][:1]           # ends at the prefill token


def test_decode_node_ttl_and_stall_watchdog():
    cfg = Llama3Config.tiny()
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=0, std=0.05)
    to_p, from_p = queue.SimpleQueue(), queue.SimpleQueue()
    decode = DecodeNode(_engine(w, cfg), to_p, from_p, request_ttl_s=0.05, decode_stall_timeout_s=1000)
    free0 = decode.llm.kv.free_blocks
    rid = decode.add_request([1, 2, 3, 4], SamplingParams(max_new_tokens=2))
    assert decode.llm.kv.free_blocks < free0
    time.sleep(0.1)
    assert decode.step() == [] and decode.expired == [rid] and decode.llm.kv.free_blocks == free0
    stalled = DecodeNode(_engine(w, cfg), to_p, from_p, request_ttl_s=1000, decode_stall_timeout_s=0.05)
    stalled.add_request([1, 2, 3], SamplingParams(max_new_tokens=2))
    stalled.step()
    time.sleep(0.1)
    with pytest.raises(SystemExit):
        stalled.step()
