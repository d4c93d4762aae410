"""DP batch padding and the one-shot scheduler (CPU)."""

import numpy as np
import torch

from modular_b200.kv_cache import KVCacheParams, PagedKVCacheManager
from modular_b200.pipelines.context import GenerationStatus, TextContext, TextGenerationOutput
from modular_b200.serve.scheduler import (DPBatchPadder, OneShotScheduler, SchedulerProgress,
                                          TokenGenerationSchedulerConfig, load_scheduler)


def _decoding(rid, n=5):
    c = TextContext.from_prompt(np.arange(1, n + 1), 64, rid)
    c.tokens.processed = n - 1
    return c


def test_pad_batches_equalises_decode_replicas_and_releases_dummies():
    kvp = KVCacheParams(2, 2, 16, 16, torch.float32, False, False)
    kv = PagedKVCacheManager(kvp, 32, torch.device("cpu"), max_seq_len=64)
    padder = DPBatchPadder(kv, 64, "m")
    batches = [[_decoding("a"), _decoding("b"), _decoding("c")], [_decoding("d")], []]
    used0 = kv.pool.used_blocks
    padded, info = padder.pad_batches(batches)
    assert [len(b) for b in padded] == [3, 3, 3] and len(info.dummies) == 5
    assert all(padder.is_decode_batch(b) for b in padded) and kv.pool.used_blocks > used0
    outs = {c.request_id: TextGenerationOutput(c.request_id, [1]) for b in padded for c in b}
    assert sorted(info.strip(outs)) == ["a", "b", "c", "d"]
    info.release()
    assert kv.pool.used_blocks == used0
    info.release()      # idempotent
    # nothing to do: equal sizes, or a step that contains prefill work
    assert padder.pad_batches([[_decoding("x")], [_decoding("y")]])[1] is None
    prefill = TextContext.from_prompt(np.arange(1, 9), 64, "p")
    assert padder.pad_batches([[prefill], []])[1] is None


def test_pad_local_builds_a_dummy_only_step_and_buckets():
    padder = DPBatchPadder(None, 64)
    batch, info = padder.pad_local([], 4)
    assert len(batch) == 4 and len(info.dummies) == 4 and padder.is_decode_batch(batch)
    same, none = padder.pad_local([_decoding("a"), _decoding("b")], 2)
    assert none is None and len(same) == 2
    assert DPBatchPadder.bucket(5, [1, 2, 4, 8, 16]) == 8 and DPBatchPadder.bucket(40, [8, 16]) == 40


class _Classifier:
    one_shot = True

    def __init__(self):
        self.batches = []

    def execute(self, batch):
        self.batches.append([c.request_id for c in batch])
        return {c.request_id: TextGenerationOutput(c.request_id, [int(c.tokens.prompt.sum()) % 7],
                                                   GenerationStatus.END_OF_SEQUENCE) for c in batch}


def test_one_shot_scheduler_batches_cancels_and_is_selected_by_the_loader():
    pipe = _Classifier()
    sched = load_scheduler(pipe, TokenGenerationSchedulerConfig(max_batch_size=2, target_tokens_per_batch_ce=100))
    assert isinstance(sched, OneShotScheduler)
    assert sched.run_iteration() is SchedulerProgress.NO_PROGRESS
    for i in range(5):
        sched.add_request(TextContext.from_prompt(np.arange(1, 4 + i), 64, f"r{i}"))
    sched.cancel_queue.put_nowait("r3")
    n = 0
    while sched.run_iteration() is SchedulerProgress.MADE_PROGRESS:
        n += 1
    assert n == 2 and pipe.batches == [["r0", "r1"], ["r2", "r4"]]
    got = {}
    while not sched.response_queue.empty():
        got.update(sched.response_queue.get_nowait())
    assert got["r3"].final_status is GenerationStatus.CANCELLED and got["r0"].is_done and len(got) == 5
