"""Device memory planning: weights + activations + KV cache -> pages, batch size, max length.

Reference: max/python/max/pipelines/lib/memory_estimation.py:222 (``MemoryEstimator.plan``,
``plan_from_sizes`` :468, ``MemoryPlan`` :87) and kv_cache/memory_planner.py:223.
The plan starts from free device memory times ``device_memory_utilization``, subtracts weights,
activation workspace and communication buffers, and turns what is left into KV pages; when the
rest cannot hold even one full-length sequence it fails with concrete suggestions.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


class InsufficientMemoryError(RuntimeError):
    pass


@dataclass
class MemoryPlan:
    total_bytes: int
    usable_bytes: int
    weight_bytes: int
    activation_bytes: int
    comm_bytes: int
    available_cache_memory: int
    num_kv_pages: int
    max_batch_size: int
    max_length: int
    max_batch_total_tokens: int

    def describe(self) -> str:
        gib = lambda b: f"{b / 2**30:.2f} GiB"
        return (f"usable {gib(self.usable_bytes)} = weights {gib(self.weight_bytes)} + activations "
                f"{gib(self.activation_bytes)} + comm {gib(self.comm_bytes)} + KV {gib(self.available_cache_memory)} "
                f"({self.num_kv_pages} pages); max_batch_size={self.max_batch_size}, max_length={self.max_length}")


class MemoryEstimator:
    @staticmethod
    def activation_bytes(hidden: int, q_dim: int, kv_dim: int, inter: int, vocab: int,
                         max_batch_input_tokens: int, max_batch_size: int, dtype_bytes: int = 2) -> int:
        per_tok = (3 * hidden + q_dim + 2 * kv_dim + q_dim + 3 * inter) * dtype_bytes
        return max_batch_input_tokens * per_tok + max_batch_size * vocab * 4 + (128 << 20)

    @staticmethod
    def plan_from_sizes(free_bytes: int, total_bytes: int, weight_bytes: int, activation_bytes: int,
                        bytes_per_page: int, page_size: int, device_memory_utilization: float = 0.9,
                        comm_bytes: int = 0, max_batch_size: Optional[int] = None,
                        max_length: Optional[int] = None, model_max_length: int = 131072,
                        weights_loaded: bool = False) -> MemoryPlan:
        usable = int(free_bytes - (1.0 - device_memory_utilization) * total_bytes)
        need = activation_bytes + comm_bytes + (0 if weights_loaded else weight_bytes)
        cache = usable - need
        want_len = max_length or model_max_length
        pages_per_seq = (want_len + page_size - 1) // page_size
        if cache < bytes_per_page * (pages_per_seq + 1):
            # can a shorter max_length fit?
            fit_pages = max(0, cache // bytes_per_page - 1)
            hint = []
            if fit_pages > 0:
                hint.append(f"lower --max-length to <= {fit_pages * page_size}")
            hint.append("raise --device-memory-utilization")
            hint.append("use more GPUs (--devices gpu:0,1,...) or a quantized encoding")
            raise InsufficientMemoryError(
                f"not enough device memory for one sequence of {want_len} tokens: "
                f"{cache / 2**30:.2f} GiB left for the KV cache after weights "
                f"({weight_bytes / 2**30:.2f} GiB) and activations ({activation_bytes / 2**30:.2f} GiB); "
                f"a sequence needs {bytes_per_page * pages_per_seq / 2**30:.2f} GiB. Try: " + "; ".join(hint))
        pages = int(cache // bytes_per_page)
        if max_batch_size is None:
            # enough sequences to fill the cache at a typical quarter of the max length, capped
            max_batch_size = int(max(1, min(512, pages // max(1, pages_per_seq // 4))))
        total_tokens = (pages - 1) * page_size
        return MemoryPlan(total_bytes, usable, weight_bytes, activation_bytes, comm_bytes, cache, pages,
                          max_batch_size, want_len, total_tokens)
