"""Offline inference entry point.

``LLM`` builds model + KV cache + pipeline + scheduler in-process and exposes

* ``generate(prompts, sampling_params, max_concurrency=...)`` - run a set of requests to
  completion with closed-loop admission (at most ``max_concurrency`` in flight) and return
  per-request token ids and latency records;
* ``add_request`` / ``step`` / ``has_unfinished`` - the engine loop for callers that drive
  it themselves.

Reference: the offline ``LLM`` class (max/python/max/_entrypoints/llm.py:74) and
``GenerateMixin.generate`` (max/python/max/pipelines/lib/interfaces/generate.py:44).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional, Sequence, Union

import numpy as np
import torch

from ..kv_cache import KVCacheParams, PagedKVCacheManager
from ..pipelines.context import SamplingParams, TextContext
from ..pipelines.text_generation import TextGenerationPipeline
from ..serve.scheduler import TokenGenerationScheduler, TokenGenerationSchedulerConfig


@dataclass
class RequestRecord:
    request_id: str
    prompt_len: int
    tokens: list = field(default_factory=list)
    arrival: float = 0.0
    first_token: Optional[float] = None
    last_token: Optional[float] = None
    finished: bool = False

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token is None else self.first_token - self.arrival

    @property
    def tpot(self) -> Optional[float]:
        n = len(self.tokens)
        if n < 2 or self.first_token is None:
            return None
        return (self.last_token - self.first_token) / (n - 1)


def merge_expert_load(parts: Sequence, slots_per_rank: Optional[int] = None) -> Optional[dict]:
    """Per-rank load slices [layers, experts per rank] -> the statistics the balancer works on."""
    from ..pipelines.eplb import rebalance

    if not parts or any(p is None for p in parts):
        return None
    load = np.concatenate([np.asarray(p) for p in parts], axis=1)            # [layers, experts]
    world, e_local = len(parts), np.asarray(parts[0]).shape[1]
    per_rank = load.reshape(load.shape[0], world, e_local).sum(-1).astype(np.float64)
    imb = per_rank.max(-1) / np.maximum(per_rank.mean(-1), 1e-9)
    worst = int(np.argmax(imb))
    plan = rebalance(load[worst], world, slots_per_rank or e_local + 1)
    return {"load": load.tolist(), "imbalance": imb.tolist(), "worst_layer": worst,
            "plan": {"phy2log": plan.phy2log.tolist(), "replica_count": plan.replica_count.tolist(),
                     "imbalance_after": float(plan.imbalance)}}


class LLM:
    def _draft_proposer(self, max_tokens: int, max_batch_size: int):
        if self.draft is None:
            return None
        from ..pipelines.speculative import BatchedDraftProposer

        d_model, d_kv = self.draft
        return BatchedDraftProposer(d_model, d_kv, max_tokens, max_batch_size, target_kv=self.kv)

    def __init__(self, model_config, weights=None, *, device: Optional[str] = None,
                 dtype: Optional[torch.dtype] = None, max_length: int = 4096, max_batch_size: int = 256,
                 max_batch_input_tokens: int = 8192, page_size: int = 128,
                 device_memory_utilization: float = 0.9, num_kv_pages: Optional[int] = None,
                 enable_prefix_caching: bool = True, enable_chunked_prefill: bool = True,
                 enable_in_flight_batching: bool = False, enable_overlap_scheduler: Optional[bool] = None,
                 device_graph_capture: bool = True, graph_batch_sizes: Optional[Sequence[int]] = None,
                 eos_token_ids: Sequence[int] = (), seed: int = 0, tp_size: int = 1,
                 tp_rank: int = 0, host_kvcache_swap_space_gb: float = 0.0,
                 disk_kvcache_dir: Optional[str] = None, disk_kvcache_space_gb: float = 0.0,
                 step_token_alignment: Optional[int] = None, weights_are_sharded: bool = False,
                 ep_size: int = 1, ep_rank: int = 0, ep_fp8_dispatch: bool = False, speculative=None,
                 draft_model_config=None, draft_weights=None):
        """``speculative``: a :class:`pipelines.speculative.SpeculativeConfig`; decode steps of greedy requests
        then verify proposals (several tokens per step, same output as plain greedy decoding): n-gram look-ups in
        the request's own history, or with ``method="draft_model"`` the greedy continuation of a smaller model of
        the same vocabulary (``draft_model_config`` / ``draft_weights``; random weights when none are given),
        which gets its own paged cache and drafts for all requests of a step at once."""
        from ..models import family_for

        fam = family_for(model_config)
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        on_gpu = self.device.type == "cuda"
        if dtype is None:
            dtype = torch.bfloat16 if on_gpu else torch.float32
        self.cfg = model_config
        self.tp = None
        if tp_size > 1:
            # one process per GPU; every rank runs the same scheduler on the same requests
            from ..parallel.tp import TPContext, shard_llama_config, shard_llama_weights

            if not on_gpu:
                raise ValueError("tensor parallelism needs CUDA devices")
            if not fam.supports_tp:
                raise ValueError(f"tensor parallelism is not implemented for the {fam.name} family")
            self.tp = TPContext(device=self.device)
            if self.tp.world != tp_size or self.tp.rank != tp_rank:
                raise ValueError("tp_size / tp_rank do not match the initialised process group")
            full_cfg = model_config
            if weights is None:
                weights = fam.weights_class.random_init(full_cfg, self.device, dtype, seed=seed)
            if not weights_are_sharded:      # ``weights`` may already be this rank's shard (random_init_shard)
                weights = shard_llama_weights(full_cfg, weights, tp_rank, tp_size)
            model_config = shard_llama_config(full_cfg, tp_size)
            torch.cuda.empty_cache()
        elif ep_size > 1:
            # expert parallelism with data-parallel attention: one process per GPU, the routed experts are sharded,
            # every rank serves its own requests and the ranks meet in the dispatch / combine kernels of every MoE
            # layer, so all ranks must run the same sequence of steps (same batch shapes)
            from ..parallel.tp import TPContext

            if not on_gpu or not fam.supports_ep:
                raise ValueError(f"expert parallelism needs CUDA devices and a MoE family (got {fam.name})")
            self.tp = TPContext(device=self.device)
            if self.tp.world != ep_size or self.tp.rank != ep_rank:
                raise ValueError("ep_size / ep_rank do not match the initialised process group")
            if weights is None:
                weights = fam.weights_class.random_init_ep(model_config, ep_rank, ep_size, self.device, dtype, seed=seed)
        elif weights is None:
            weights = fam.weights_class.random_init(model_config, self.device, dtype, seed=seed)
        if speculative is not None and fam.name in ("mamba", "lfm2"):
            # verifying a draft runs the rejected tokens through the recurrence too, and a state cannot be rolled back
            raise ValueError("speculative decoding is not implemented for state-space models")
        self.weights = weights
        self.max_length = max_length
        # the draft model of speculative decoding comes first, so that the cache sizing below sees what it took
        self.draft = None
        if speculative is not None and speculative.method == "draft_model":
            if draft_model_config is None:
                raise ValueError("speculative method draft_model needs draft_model_config")
            if tp_size > 1 or ep_size > 1:
                raise ValueError("draft-model speculation runs on one device")
            if draft_model_config.vocab_size != model_config.vocab_size:
                raise ValueError("the draft model must share the target's vocabulary")
            dfam = family_for(draft_model_config)
            if draft_weights is None:
                draft_weights = dfam.weights_class.random_init(draft_model_config, self.device, dtype, seed=seed + 1)
            dkvp = dfam.kv_params(draft_model_config, page_size, dtype, False)   # no prefix cache: drafts get rewritten
            if on_gpu:
                free, total = torch.cuda.mem_get_info(self.device)
                d_budget = int(0.1 * (free - (1.0 - device_memory_utilization) * total))
                d_pages = dkvp.compute_num_device_blocks(d_budget, max_batch_size * 4, max_length)
            else:
                d_pages = dkvp.compute_num_device_blocks(1 << 62, max_batch_size, max_length)
            d_kv = PagedKVCacheManager(dkvp, d_pages, self.device, max_seq_len=max_length)
            d_extra = {"tp": None} if dfam.supports_tp else {}
            d_model = dfam.model_class(draft_model_config, draft_weights, d_kv.kv, max_tokens=max_batch_input_tokens,
                                       max_seqs=max_batch_size, max_position=max_length, **d_extra)
            self.draft = (d_model, d_kv)
        kvp = fam.kv_params(model_config, page_size, dtype, enable_prefix_caching)
        if num_kv_pages is None:
            if on_gpu:
                free, total = torch.cuda.mem_get_info(self.device)
                act = fam.activation_bytes(model_config, max_batch_input_tokens, max_batch_size)
                budget = int(free - (1.0 - device_memory_utilization) * total - act)
                num_kv_pages = kvp.compute_num_device_blocks(budget, max_batch_size * 4, max_length)
            else:
                num_kv_pages = kvp.compute_num_device_blocks(1 << 62, max_batch_size, max_length)
        # evicted prefix pages fall back to pinned host memory and then to a file (kv_cache/tiers.py)
        host_pages = int(host_kvcache_swap_space_gb * (1 << 30) // kvp.bytes_per_page)
        disk_pages = int(disk_kvcache_space_gb * (1 << 30) // kvp.bytes_per_page) if disk_kvcache_dir else 0
        self.kv = PagedKVCacheManager(kvp, num_kv_pages, self.device, max_seq_len=max_length,
                                      host_pages=host_pages, disk_pages=disk_pages, disk_dir=disk_kvcache_dir)
        extra = {"tp": self.tp} if fam.supports_tp else {}
        if ep_size > 1:
            from ..parallel.ep import EPContext

            c = model_config
            import datetime

            import torch.distributed as dist

            # the ranks agree on the token bound of every step over a host-side group (they serve different
            # requests, so their batches differ)
            extra["ep"] = EPContext(self.tp, c.hidden_size, c.n_routed_experts, c.num_experts_per_tok,
                                    max_tokens=max_batch_input_tokens, fp8_dispatch=ep_fp8_dispatch, collect_load=True,
                                    host_group=dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=300)))
        # verification asks for the logits of every draft position: size the model's logit rows for it
        spec_rows = (speculative.num_speculative_tokens + 1) if speculative is not None else 1
        self._ep = extra.get("ep")
        self.model = fam.model_class(model_config, weights, self.kv.kv, max_tokens=max_batch_input_tokens,
                                     max_seqs=max_batch_size * spec_rows, max_position=max_length, **extra)
        overlap = on_gpu if enable_overlap_scheduler is None else enable_overlap_scheduler
        overlap = overlap and bool(getattr(self.model, "use_executor", False)) and speculative is None
        if graph_batch_sizes is None:
            graph_batch_sizes = [b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256) if b <= max_batch_size]
        self.pipeline = TextGenerationPipeline(
            self.model, self.kv, max_batch_input_tokens, max_batch_size, overlap=overlap,
            graph_batch_sizes=graph_batch_sizes if (device_graph_capture and on_gpu) else (),
            eos_token_ids=eos_token_ids, speculative=speculative, draft=self._draft_proposer(max_batch_input_tokens,
                                                                                             max_batch_size))
        if device_graph_capture and on_gpu:
            self.pipeline.warmup_graph_capture()
            if hasattr(self.model, "capture_decode_graphs"):
                # models whose step is driven op by op capture their decode steps themselves
                self.model.capture_decode_graphs(graph_batch_sizes)
        self.sched_config = TokenGenerationSchedulerConfig(
            max_batch_size=max_batch_size, target_tokens_per_batch_ce=max_batch_input_tokens,
            max_seq_len=max_length, enable_chunked_prefill=enable_chunked_prefill,
            enable_in_flight_batching=enable_in_flight_batching,
            kv_lookahead_tokens=1 if overlap else 0,
            # on the GPU, steps that would overshoot a multiple of 1024 tokens by a few are trimmed to it (whole
            # waves of GEMM tiles, see ActiveTokenBudget)
            step_token_alignment=(1024 if on_gpu else 0) if step_token_alignment is None else step_token_alignment)
        self.scheduler = TokenGenerationScheduler(self.sched_config, self.pipeline, self.kv)
        self.eos_token_ids = tuple(eos_token_ids)
        self._records: dict[str, RequestRecord] = {}
        self._n = 0

    # ------------------------------------------------------------ engine loop
    # ------------------------------------------------------------ LoRA
    def load_lora(self, name: str, state_dict: dict, alpha: Optional[float] = None, max_loras: int = 8) -> None:
        """Make a PEFT-layout adapter available to requests (``add_request(..., lora_name=name)``)."""
        from ..pipelines.lora import LoRAAdapter, LoRAManager
        if self.pipeline.lora_manager is None:
            self.pipeline.lora_manager = LoRAManager(max_loras)
        dtype = self.weights.embed.dtype
        self.pipeline.lora_manager.load(LoRAAdapter.from_state_dict(name, state_dict, alpha=alpha,
                                                                    device=self.device, dtype=dtype))

    def unload_lora(self, name: str) -> bool:
        return self.pipeline.lora_manager is not None and self.pipeline.lora_manager.unload(name)

    def add_request(self, prompt_ids, sampling_params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, lora_name: Optional[str] = None) -> str:
        if getattr(self.model, "generates", True) is False:
            raise NotImplementedError(f"{type(self.model).__name__} serves embeddings (encode), not generation")
        self._n += 1
        rid = request_id or f"llm-{self._n}"
        ctx = TextContext.from_prompt(prompt_ids, self.max_length, rid, sampling_params,
                                      self.eos_token_ids)
        if lora_name:
            if self.pipeline.lora_manager is None:
                raise KeyError(f"LoRA adapter {lora_name!r} is not loaded")
            self.pipeline.lora_manager.slot_of(lora_name)      # raises when unknown
            ctx.lora_name = lora_name
        self._records[rid] = RequestRecord(rid, ctx.tokens.prompt_len, arrival=ctx.arrival_time)
        self.scheduler.add_request(ctx)
        return rid

    def step(self) -> list[RequestRecord]:
        """One scheduler iteration; returns the records of requests that finished in it. Expert-parallel ranks
        keep in step: a rank whose scheduler launched nothing runs an idle step, because every MoE layer of every
        step is an exchange that all ranks take part in."""
        fw0 = getattr(self.model, "forward_calls", 0)
        self.scheduler.run_iteration()
        if self._ep and getattr(self.model, "forward_calls", 0) == fw0:
            self.model.idle_step()
        finished = []
        q = self.scheduler.response_queue
        while not q.empty():
            for rid, out in q.get_nowait().items():
                rec = self._records.get(rid)
                if rec is None:
                    continue
                if out.tokens:
                    now = time.perf_counter()
                    if rec.first_token is None:
                        rec.first_token = now
                    rec.last_token = now
                    rec.tokens.extend(out.tokens)
                if out.is_done:
                    rec.finished = True
                    finished.append(rec)
        return finished

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work() or not self.scheduler.request_queue.empty()

    def encode(self, prompts: Sequence[Sequence[int]], pooling: str = "default") -> torch.Tensor:
        """Pooled, L2-normalised embeddings of token-id prompts: fp32 [n, hidden]. ``default`` is the model's own
        pooling (the last token for decoders, the mean for encoders)."""
        if not hasattr(self.model, "encode"):
            raise NotImplementedError(f"{type(self.model).__name__} does not produce embeddings")
        if pooling in (None, "default"):
            pooling = getattr(self.model, "default_pooling", "last")
        return self.model.encode([list(p) for p in prompts], pooling)

    # ------------------------------------------------------------ batch API
    def generate(self, prompts: Sequence[Union[Sequence[int], np.ndarray]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 max_concurrency: Optional[int] = None) -> list[RequestRecord]:
        """Run every prompt (token ids) to completion. With ``max_concurrency`` a new request is
        admitted only when one finishes (closed loop), as a serving benchmark client would."""
        n = len(prompts)
        if isinstance(sampling_params, SamplingParams) or sampling_params is None:
            sps = [sampling_params] * n
        else:
            sps = list(sampling_params)
        conc = n if not max_concurrency else min(max_concurrency, n)
        order, nxt, inflight = [], 0, 0
        while nxt < conc:
            order.append(self.add_request(prompts[nxt], sps[nxt]))
            nxt += 1
            inflight += 1
        while self._any_rank_busy(inflight > 0):
            for _ in self.step():
                inflight -= 1
                if nxt < n:
                    order.append(self.add_request(prompts[nxt], sps[nxt]))
                    nxt += 1
                    inflight += 1
        recs = [self._records.pop(rid) for rid in order]
        return recs

    def eplb_stats(self, slots_per_rank: Optional[int] = None) -> Optional[dict]:
        """Expert load of all ranks (collective: every rank calls it): tokens per (MoE layer, logical expert), the
        per-layer imbalance max / mean over ranks, and for the most imbalanced layer the balancer's placement with
        ``slots_per_rank`` physical slots per rank (default: experts per rank + 1)."""
        if not self._ep:
            return None
        import torch.distributed as dist

        mine = self.model.expert_load()
        parts = [None] * self._ep.world
        dist.all_gather_object(parts, mine, group=self._ep.host_group)
        return merge_expert_load(parts, slots_per_rank)

    def _any_rank_busy(self, busy: bool) -> bool:
        """``busy`` on one GPU; under expert parallelism whether ANY rank still has requests (the others keep
        taking idle steps until all are done)."""
        if not self._ep:
            return busy
        import torch.distributed as dist

        t = torch.tensor([1 if busy else 0], dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self._ep.host_group)
        return bool(int(t))
