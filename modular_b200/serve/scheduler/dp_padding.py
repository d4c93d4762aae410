"""Data-parallel batch padding: every replica of a decode step runs with the same number of sequences.

CUDA graphs are captured per batch size, and with expert parallelism every rank has to enter the same
dispatch / combine collectives in every step. When replicas (ranks that each decode their own requests) hold
different numbers of sequences, the short ones are padded with dummy one-token requests up to the largest, and a
replica without work still executes a step of dummies. Dummies are fresh contexts that claim KV pages like a real
request; they are released, and their outputs dropped, right after the step.

Reference: max/python/max/serve/scheduler/dp_padding.py:45 (``DPBatchPadder``) and the empty-batch execution of
max/python/max/pipelines/lib/pipeline_variants/overlap_text_generation.py:4009-4014.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from ...pipelines.context import SamplingParams, TextContext

_dummy_ids = itertools.count()


@dataclass
class DPPaddingInfo:
    dummies: list = field(default_factory=list)
    _release: Optional[callable] = None

    def release(self) -> None:
        """Free the dummies' KV pages and pipeline state; call once the step's device work has been synchronised."""
        if self._release is not None:
            self._release(self.dummies)
            self._release = None

    def strip(self, outputs: dict) -> dict:
        """The step's outputs without the dummies' entries."""
        drop = {d.request_id for d in self.dummies}
        return {rid: o for rid, o in outputs.items() if rid not in drop}


class DPBatchPadder:
    def __init__(self, kv=None, max_length: int = 1 << 20, model_name: str = "", pipeline=None, dummy_token: int = 0):
        self.kv, self.max_length, self.model_name, self.pipeline = kv, max_length, model_name, pipeline
        self.dummy_token = dummy_token

    # ------------------------------------------------------------ helpers
    def _new_dummy(self) -> TextContext:
        c = TextContext.from_prompt(np.asarray([self.dummy_token, self.dummy_token]), self.max_length,
                                    f"dp-pad-{next(_dummy_ids)}",
                                    SamplingParams(temperature=0.0, max_new_tokens=1, ignore_eos=True),
                                    model_name=self.model_name)
        c.tokens.processed = 1          # looks like a decoding request: one token of context, one active token
        if self.kv is not None:
            self.kv.claim(c)
            self.kv.alloc(c)
        return c

    def _release(self, dummies: Sequence[TextContext]) -> None:
        for d in dummies:
            if self.kv is not None:
                self.kv.release(d.request_id)
            if self.pipeline is not None and hasattr(self.pipeline, "release"):
                self.pipeline.release(d.request_id)

    @staticmethod
    def is_decode_batch(batch: Sequence[TextContext]) -> bool:
        # one new token per sequence: the shape that decode CUDA graphs are captured for
        return all(c.tokens.active_length == 1 for c in batch)

    # ------------------------------------------------------------ one process, several replicas
    def pad_batches(self, batches: Sequence[Sequence[TextContext]]):
        """``batches[r]`` = sequences of replica r in this step. Returns (padded batches, info or None). Only pure
        decode steps are padded (prefill steps are not graph-replayed)."""
        sizes = [len(b) for b in batches]
        target = max(sizes, default=0)
        if target == 0 or all(s == target for s in sizes) or not all(self.is_decode_batch(b) for b in batches):
            return [list(b) for b in batches], None
        info = DPPaddingInfo(_release=self._release)
        padded = []
        for b in batches:
            extra = [self._new_dummy() for _ in range(target - len(b))]
            info.dummies.extend(extra)
            padded.append(list(b) + extra)
        return padded, info

    # ------------------------------------------------------------ one process per replica
    def pad_local(self, batch: Sequence[TextContext], target: int):
        """Pad this replica's decode batch to ``target`` sequences (the largest size over all replicas, exchanged
        by the caller). ``target`` > 0 with an empty ``batch`` yields a step made of dummies only."""
        if target <= len(batch) or not self.is_decode_batch(batch):
            return list(batch), None
        info = DPPaddingInfo(_release=self._release)
        info.dummies = [self._new_dummy() for _ in range(target - len(batch))]
        return list(batch) + info.dummies, info

    @staticmethod
    def bucket(size: int, graph_batch_sizes: Sequence[int]) -> int:
        """Smallest captured batch size that holds ``size`` sequences (``size`` itself when none does)."""
        fits = [b for b in sorted(graph_batch_sizes) if b >= size]
        return fits[0] if fits else size
