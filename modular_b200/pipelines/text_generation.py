"""Text-generation pipelines: one forward + sample per ``execute`` call.

``TextGenerationPipeline.execute(batch)`` runs a ragged batch of contexts (each contributes
its active window), samples one token for every context whose window reaches its last
token, updates the contexts and the KV manager, and returns ``{request_id:
TextGenerationOutput}``. (Reference: max/python/max/pipelines/lib/pipeline_variants/
text_generation.py:135, ``execute`` :498.)

With ``overlap=True`` the pipeline behaves like the reference's
``OverlapTextGenerationPipeline`` (overlap_text_generation.py:14-60, :3899): ``execute``
enqueues step N and returns the outputs of step N-1, so the host prepares the next batch
while the GPU runs the current one. Token ids sampled by step N stay on the device; step
N+1 picks them up there (``FUTURE_TOKEN`` placeholders in the context until the readback
lands). Decode-only steps of a captured batch size replay as CUDA graphs.
"""

from __future__ import annotations

import gc

import time
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..kv_cache import PagedKVCacheManager
from .batch import BatchPacker, StepBatch, meta_layout
from .context import FUTURE_TOKEN, GenerationStatus, TextContext, TextGenerationOutput


@dataclass
class _InFlight:
    batch: StepBatch
    event: Optional[torch.cuda.Event]
    host_tokens: Optional[torch.Tensor]   # pinned int64 [n_logits] (GPU) or plain tensor (CPU)
    launched_at: float = 0.0
    logprobs: Optional[tuple] = None      # (chosen [n], top values [n, k], top ids [n, k]) when a request asked


@dataclass
class PipelineStats:
    steps: int = 0
    graph_replays: int = 0
    tokens_in: int = 0
    tokens_out: int = 0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    gpu_launches_at_start: int = 0


class TextGenerationPipeline:
    def __init__(self, model, kv_manager: PagedKVCacheManager, max_batch_tokens: int = 8192,
                 max_batch_size: int = 256, overlap: bool = False, graph_batch_sizes: Sequence[int] = (),
                 eos_token_ids: Sequence[int] = (), speculative=None, draft=None):
        """``speculative``: a :class:`speculative.SpeculativeConfig` turns decode steps of greedy requests into
        propose-and-verify steps (the step runs synchronously: the proposals need the previous token values).
        ``draft``: the :class:`speculative.BatchedDraftProposer` of the ``draft_model`` method."""
        self.model = model
        self.kv = kv_manager
        self.device = model.device
        self.on_gpu = self.device.type == "cuda"
        # overlap scheduling needs the native step (future tokens are realised on the device)
        self.overlap = overlap and self.on_gpu and bool(getattr(model, "use_executor", False)) and speculative is None
        self.eos_token_ids = frozenset(eos_token_ids)
        cfg = model.cfg
        self.spec = speculative
        self.spec_stats = None
        self.proposer = None
        self.draft = None
        rows = max_batch_size
        if speculative is not None:
            from .speculative import NgramProposer, SpecStats

            if speculative.method == "draft_model":
                if draft is None:
                    raise ValueError("the draft_model method needs a BatchedDraftProposer (LLM(draft_model_config=...))")
            elif speculative.method != "ngram":
                raise ValueError(f"unknown speculative method {speculative.method!r} (ngram | draft_model)")
            self.draft = draft if speculative.method == "draft_model" else None
            self.proposer = NgramProposer(speculative)
            self.spec_stats = SpecStats()
            rows = min(max_batch_size * (speculative.num_speculative_tokens + 1), getattr(model, "max_seqs", 1 << 30))
        self.packer = BatchPacker(cfg.num_attention_heads, cfg.num_key_value_heads, kv_manager.page_size,
                                  max_batch_tokens, max_batch_size, kv_manager.max_pages_per_seq,
                                  device=self.device, max_logit_rows=rows)
        self.stats = PipelineStats()
        self._pending: Optional[_InFlight] = None
        self._step = 0
        self._graphs: dict[int, tuple] = {}
        self._d2h = [torch.empty(rows, dtype=torch.long, pin_memory=self.on_gpu) for _ in range(4)]
        self._d2h_i = 0
        self.graph_batch_sizes = tuple(sorted(set(int(b) for b in graph_batch_sizes)))
        self._cpu_gen = torch.Generator().manual_seed(0)
        self._gpu_events: list = []
        self._graph_launches: dict[int, int] = {}
        self._replayed_launches = 0
        self.record_gpu_time = self.on_gpu
        self.structured = None      # StructuredOutputBackend, see enable_structured_output
        self.lora_manager = None    # pipelines.lora.LoRAManager when adapters are enabled

    # ------------------------------------------------------------ grammar-constrained decoding
    def enable_structured_output(self, tokenizer) -> None:
        from .structured_output import StructuredOutputBackend
        self.structured = StructuredOutputBackend(tokenizer, self.model.cfg.vocab_size)

    def _prepare_grammars(self, batch: Sequence[TextContext]) -> bool:
        """Compile grammars of new requests; True when any request of the batch is constrained."""
        any_grammar = False
        for c in batch:
            spec = c.sampling_params.response_format
            if spec is None:
                continue
            if self.structured is None:
                raise RuntimeError("a request asked for structured output but the pipeline was built without it")
            if c.grammar_state is None:
                c.grammar_state = self.structured.compile(spec)
                # tokens generated before a preemption are replayed into the fresh matcher
                for t in c.tokens.generated:
                    if t >= 0:
                        c.grammar_state.accept(int(t))
            any_grammar = True
        return any_grammar

    def _grammar_bitmask(self, sb: StepBatch):
        states = [c.grammar_state for c in sb.logit_ctx]
        return self.structured.bitmask_for(states) if any(s is not None for s in states) else None

    # ------------------------------------------------------------ CUDA graphs
    def warmup_graph_capture(self) -> None:
        """Capture one decode graph per configured batch size (layout pinned per size)."""
        if not (self.on_gpu and self.model.use_executor):
            return
        for B in self.graph_batch_sizes:
            if B in self._graphs or B > self.packer.max_seqs:
                continue
            fixed = (B, B, self.kv.max_pages_per_seq, 1)
            off, words = meta_layout(*fixed)
            meta = self.packer.meta_dev
            # a harmless all-dummy batch for the capture run
            host = np.zeros(words, dtype=np.int32)
            host[off["q_len"] : off["q_len"] + B] = 1
            host[off["kv_len"] : off["kv_len"] + B] = 1
            host[off["q_start"] : off["q_start"] + B] = np.arange(B)
            host[off["decode_seq"] : off["decode_seq"] + B] = np.arange(B)
            host[off["logit_rows"] : off["logit_rows"] + B] = np.arange(B)
            host[off["future_src"] : off["future_src"] + B] = -1
            host.view(np.int64)[off["slots"] // 2 : off["slots"] // 2 + B] = -1
            host.view(np.float32)[off["top_p"] : off["top_p"] + B] = 1.0
            meta[:words].copy_(torch.from_numpy(host))
            args = (meta, off, B, B, fixed[2], 0, B, B, True, True, 0)
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):
                    self.model.forward_packed(*args)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            n0 = self.model.executor.launches()
            # dead cycles (an engine that is no longer referenced, with its CUDA graphs) go now, not while the
            # stream captures: destroying a graph during a capture invalidates it
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(g):
                    self.model.forward_packed(*args)
            finally:
                if gc_was_on:
                    gc.enable()
            self._graph_launches[B] = self.model.executor.launches() - n0
            self._graphs[B] = (g, fixed, off, words)
        torch.cuda.synchronize()

    def _graph_bucket(self, batch: Sequence[TextContext]) -> int:
        if not self._graphs:
            return 0
        n = len(batch)
        for B in self.graph_batch_sizes:
            if B >= n and B in self._graphs:
                # the captured graph samples inside the step: anything the replay cannot apply per request
                # (penalties, grammar masks, log-probabilities, adapters) keeps the batch on the eager path
                if all(c.tokens.active_length == 1 and c.sampling_params.is_greedy
                       and c.sampling_params.response_format is None and not c.sampling_params.logprobs
                       and not c.sampling_params.needs_penalties and not c.lora_name
                       for c in batch):
                    return B
                return 0
        return 0

    # ------------------------------------------------------------ one step
    def _launch(self, batch: Sequence[TextContext]) -> _InFlight:
        self._step += 1
        self.stats.steps += 1
        model = self.model
        uses_lora = self.lora_manager is not None and any(c.lora_name for c in batch)
        if self.on_gpu and model.use_executor and not uses_lora:
            # device time of a step = from after the metadata upload to after the sampled-token copy is queued
            ev0 = torch.cuda.Event(enable_timing=True) if self.record_gpu_time else None
            step_logprobs = None
            B_graph = self._graph_bucket(batch)
            if B_graph:
                g, fixed, off, words = self._graphs[B_graph]
                sb = self.packer.pack(batch, self.kv, fixed=fixed, pad_to=B_graph)
                self.packer.upload(sb)
                if ev0 is not None:
                    ev0.record()
                g.replay()
                self.stats.graph_replays += 1
                self._replayed_launches += self._graph_launches[B_graph]
            else:
                sb = self.packer.pack(batch, self.kv)
                meta = self.packer.upload(sb)
                if ev0 is not None:
                    ev0.record()
                needs_pen = any(c.sampling_params.needs_penalties for c in sb.logit_ctx)
                mask = self._grammar_bitmask(sb) if self.structured is not None else None
                wants_lp = any(c.sampling_params.logprobs for c in sb.logit_ctx)
                host_sample = needs_pen or mask is not None or wants_lp
                model.forward_packed(meta, sb.offsets, sb.T, sb.B, sb.bt_stride, sb.n_tiles,
                                     sb.n_decode, sb.n_logits, sb.has_future, not host_sample, self._step)
                if mask is not None:
                    ops.apply_token_bitmask(model.logits_buf[: sb.n_logits], mask)
                if host_sample:
                    self._penalties_and_sample(sb, meta)
                if wants_lp:
                    step_logprobs = self._logprobs_of(sb, model.logits_buf, model.sampled)
            self.stats.h2d_bytes += sb.words * 4
            host = self._d2h[self._d2h_i]
            self._d2h_i = (self._d2h_i + 1) % len(self._d2h)
            host[: sb.n_logits].copy_(model.sampled[: sb.n_logits], non_blocking=True)
            ev = torch.cuda.Event(enable_timing=self.record_gpu_time)
            ev.record()
            if self.record_gpu_time:
                self._gpu_events.append((ev0, ev))
            self.stats.d2h_bytes += sb.n_logits * 8
            inflight = _InFlight(sb, ev, host, time.perf_counter(), step_logprobs)
        else:
            sb = self.packer.pack(batch, self.kv)
            t = BatchPacker.tensors(sb, self.device)
            toks = t["tokens"]
            if sb.has_future:
                raise RuntimeError("future tokens require the overlap (GPU) pipeline")
            extra = {}
            if uses_lora:
                # steps that touch an adapter run op by op: base GEMMs plus grouped shrink/expand GEMMs
                from .lora import LoRABatch, token_slots_for
                extra["lora"] = LoRABatch(self.lora_manager, token_slots_for(
                    self.lora_manager, [c.tokens.active_length for c in sb.ctxs], [c.lora_name for c in sb.ctxs],
                    self.device))
            logits = model.forward_tensors(toks, t["positions"], t["slots"], t["block_table"],
                                           t["q_start"], t["q_len"], t["kv_len"], t["logit_rows"], **extra)
            mask = self._grammar_bitmask(sb) if self.structured is not None else None
            if mask is not None:
                ops.apply_token_bitmask(logits, mask)
            sampled = self._sample_host(sb, t, logits)
            inflight = _InFlight(sb, None, sampled.cpu(), time.perf_counter(), self._logprobs_of(sb, logits, sampled))
            self.last_logits = logits
        self.stats.tokens_in += sb.T
        # bookkeeping that does not need the token values
        for i, c in enumerate(sb.logit_ctx):
            c.sample_slot = i
        for c in sb.ctxs:
            c.tokens.advance_processed()
        for c in sb.logit_ctx:
            c.update_with_future_token()
        return inflight

    def _penalties_and_sample(self, sb: StepBatch, meta: torch.Tensor) -> None:
        n, off = sb.n_logits, sb.offsets
        logits = self.model.logits_buf[:n]
        tok, cnt, offs = [], [], [0]
        freq = np.zeros(n, np.float32)
        pres = np.zeros(n, np.float32)
        rep = np.ones(n, np.float32)
        for i, c in enumerate(sb.logit_ctx):
            sp = c.sampling_params
            if sp.needs_penalties:
                allt = c.tokens.all
                allt = allt[allt >= 0]
                gen_start = c.tokens.prompt_len
                u, _ = np.unique(allt, return_counts=True)
                gen = c.tokens.all[gen_start:]
                gen = gen[gen >= 0]
                gu, gc = np.unique(gen, return_counts=True)
                counts = dict(zip(gu.tolist(), gc.tolist()))
                tok.extend(u.tolist())
                cnt.extend(counts.get(int(x), 0) for x in u.tolist())
                freq[i], pres[i], rep[i] = sp.frequency_penalty, sp.presence_penalty, sp.repetition_penalty
            offs.append(len(tok))
        dev = self.device
        mk = lambda a, dt: torch.tensor(a, dtype=dt, device=dev)
        ops.apply_penalties(logits, mk(tok or [0], torch.int32), mk(cnt or [0], torch.int32),
                            mk(offs, torch.int32), mk(freq, torch.float32), mk(pres, torch.float32),
                            mk(rep, torch.float32))
        self._add_logit_bias(sb, logits)
        f32 = lambda name: meta[off[name] : off[name] + n].view(torch.float32)
        ops.sample(logits, f32("temperature"), meta[off["top_k"] : off["top_k"] + n], f32("top_p"),
                   f32("min_p"), meta[off["seeds"] : off["seeds"] + 2 * n].view(torch.int64),
                   self._step, out=self.model.sampled[:n])

    @staticmethod
    def _logprobs_of(sb: StepBatch, logits: torch.Tensor, sampled: torch.Tensor) -> Optional[tuple]:
        """Log-probabilities of the sampled tokens and the top-k alternatives (k = the largest request)."""
        k = max(((c.sampling_params.logprobs or 0) for c in sb.logit_ctx), default=0)
        if k <= 0:
            return None
        lp = torch.log_softmax(logits[: sb.n_logits].float(), dim=-1)
        chosen = lp.gather(1, sampled[: sb.n_logits].view(-1, 1).long()).squeeze(1)
        top_v, top_i = lp.topk(min(int(k), lp.shape[1]), dim=-1)
        return chosen.cpu(), top_v.cpu(), top_i.cpu()

    def _sample_host(self, sb: StepBatch, t: dict, logits: torch.Tensor) -> torch.Tensor:
        if any(c.sampling_params.needs_penalties for c in sb.logit_ctx):
            tok, cnt, offs = [], [], [0]
            for c in sb.logit_ctx:
                if c.sampling_params.needs_penalties:
                    u = np.unique(c.tokens.all)
                    gu, gc = np.unique(c.tokens.generated, return_counts=True)
                    counts = dict(zip(gu.tolist(), gc.tolist()))
                    tok.extend(u.tolist())
                    cnt.extend(counts.get(int(x), 0) for x in u.tolist())
                offs.append(len(tok))
            sp = [c.sampling_params for c in sb.logit_ctx]
            ops.apply_penalties(logits, torch.tensor(tok or [0], dtype=torch.int32),
                                torch.tensor(cnt or [0], dtype=torch.int32), torch.tensor(offs, dtype=torch.int32),
                                torch.tensor([s.frequency_penalty for s in sp]),
                                torch.tensor([s.presence_penalty for s in sp]),
                                torch.tensor([s.repetition_penalty for s in sp]))
        self._add_logit_bias(sb, logits)
        if sb.all_greedy:
            return ops.argmax(logits)
        return ops.sample(logits, t["temperature"], t["top_k"], t["top_p"], t["min_p"],
                          generator=self._cpu_gen)

    @staticmethod
    def _add_logit_bias(sb: StepBatch, logits: torch.Tensor) -> None:
        """Per-request additive biases (``SamplingParams.logit_bias``) on the rows that sample this step; ids
        outside the vocabulary are ignored."""
        rows, toks, vals = [], [], []
        V = logits.shape[1]
        for i, c in enumerate(sb.logit_ctx):
            lb = c.sampling_params.logit_bias
            if lb:
                for t_, v in lb.items():
                    if t_ < V:
                        rows.append(i), toks.append(t_), vals.append(v)
        if rows:
            dev = logits.device
            logits.index_put_((torch.tensor(rows, device=dev), torch.tensor(toks, device=dev)),
                              torch.tensor(vals, dtype=logits.dtype, device=dev), accumulate=True)

    def _collect(self, inflight: Optional[_InFlight]) -> dict:
        """Wait for a launched step's tokens, fold them into the contexts, build outputs."""
        out: dict[str, TextGenerationOutput] = {}
        if inflight is None:
            return out
        if inflight.event is not None:
            inflight.event.synchronize()
        sb = inflight.batch
        vals = inflight.host_tokens[: sb.n_logits].numpy()
        for i, c in enumerate(sb.logit_ctx):
            c.realize_future_token(int(vals[i]))
            if c.grammar_state is not None:
                c.grammar_state.accept(int(vals[i]))
            if inflight.logprobs is not None and c.sampling_params.logprobs:
                chosen, top_v, top_i = inflight.logprobs
                k = int(c.sampling_params.logprobs)
                c.logprob_entries.append({"token": int(vals[i]), "logprob": float(chosen[i]),
                                          "top": [(int(a), float(b)) for a, b in zip(top_i[i, :k], top_v[i, :k])]})
            self.stats.tokens_out += 1
        for c in sb.ctxs:
            if self.kv.contains(c.request_id):
                self.kv.step(c)
        for c in sb.logit_ctx:
            out[c.request_id] = c.to_generation_output()
        return out

    # ------------------------------------------------------------ speculative decoding
    def _spec_eligible(self, batch: Sequence[TextContext]) -> bool:
        """Propose-and-verify applies to decode-only steps whose requests are greedy and need nothing per token
        that the verification pass does not provide (masks, penalties, log-probabilities, adapters)."""
        for c in batch:
            sp = c.sampling_params
            if (c.tokens.active_length != 1 or c.needs_ce or c.pending_future or not sp.is_greedy
                    or sp.response_format is not None or sp.logprobs or sp.needs_penalties or c.lora_name):
                return False
        return True

    def _speculative_step(self, batch: Sequence[TextContext]) -> dict:
        """One propose-and-verify step (reference: pipelines/lib/pipeline_variants/overlap_text_generation.py:306,
        nn/sampling/rejection_sampler.py:121 greedy acceptance). Every request brings its last token plus up to k
        draft tokens; the target model scores all of them in one ragged pass; the longest prefix of drafts that
        equals the target's own greedy choice is accepted together with one more token. The output is exactly
        that of plain greedy decoding."""
        k = self.spec.num_speculative_tokens
        budget = self.packer.max_tokens - len(batch)          # rows left for drafts in this step
        rows_left = self.packer.max_logit_rows - len(batch)
        rooms = []
        for c in batch:
            tb = c.tokens
            room = max(0, min(k, c.max_new_tokens_effective - tb.generated_length - 1, c.max_length - len(tb) - 1,
                              budget, rows_left))
            rooms.append(room)
            budget -= room
            rows_left -= room
        if self.draft is not None:
            proposals = self.draft.propose_batch(batch, rooms)     # k batched steps of the draft model
        else:
            proposals = [self.proposer.propose(c.tokens.all, r)[0] if r > 0 else [] for c, r in zip(batch, rooms)]
        base_len, drafts = [], []
        for c, d, room in zip(batch, proposals, rooms):
            tb = c.tokens
            d = list(d[:room])
            while d and not self.kv.can_alloc(c, len(d)):
                d = d[:-1]
            base_len.append(len(tb))
            drafts.append(d)
            for t in d:                                        # tentative: rolled back below
                tb.advance_with_token(int(t))
            tb.active_end = len(tb)
            self.kv.alloc(c)
        self._step += 1
        self.stats.steps += 1
        sb = self.packer.pack(batch, self.kv, all_logits=True)
        if self.on_gpu and self.model.use_executor:
            meta = self.packer.upload(sb)
            self.model.forward_packed(meta, sb.offsets, sb.T, sb.B, sb.bt_stride, sb.n_tiles, sb.n_decode, sb.n_logits,
                                      False, True, self._step)
            self.stats.h2d_bytes += sb.words * 4
            self.stats.d2h_bytes += sb.n_logits * 8
            vals = self.model.sampled[: sb.n_logits].cpu().numpy()
        else:
            t = BatchPacker.tensors(sb, self.device)
            logits = self.model.forward_tensors(t["tokens"], t["positions"], t["slots"], t["block_table"], t["q_start"],
                                                t["q_len"], t["kv_len"], t["logit_rows"])
            vals = ops.argmax(logits).cpu().numpy()
        self.stats.tokens_in += sb.T
        out: dict[str, TextGenerationOutput] = {}
        row = 0
        st = self.spec_stats
        for c, d, L in zip(batch, drafts, base_len):
            n = len(d) + 1
            target = vals[row: row + n]
            row += n
            acc = 0
            while acc < len(d) and int(d[acc]) == int(target[acc]):
                acc += 1
            tb = c.tokens
            tb.truncate(L)                                     # drop the drafts ...
            for j in range(acc + 1):                           # ... and append what the target chose
                c.update(int(target[j]))
                self.stats.tokens_out += 1
                st.emitted += 1
                if c.is_done:
                    break
            # the cache holds the last token and the accepted drafts; the newest token is the next window
            tb.processed = len(tb) - 1
            tb.active_end = len(tb)
            st.steps += 1
            st.proposed += len(d)
            st.accepted += acc
            if self.kv.contains(c.request_id):
                self.kv.step(c)
            out[c.request_id] = c.to_generation_output()
        return out

    def execute(self, batch: Sequence[TextContext]) -> dict:
        """Run one step. Synchronous mode returns this step's outputs; overlap mode returns the
        previous step's (call with an empty batch to drain)."""
        if batch and self.spec is not None and self._spec_eligible(batch):
            return self._speculative_step(batch)
        constrained = self._prepare_grammars(batch) if batch else False
        if batch and self.lora_manager is not None and any(c.lora_name for c in batch):
            constrained = True      # adapter steps run synchronously on real token values
        if not self.overlap:
            return self._collect(self._launch(batch)) if batch else {}
        if constrained and self._pending is not None:
            # the mask of a constrained request depends on its previous token: read that back first
            out = self._collect(self._pending)
            self._pending = self._launch(batch)
            return out
        new = self._launch(batch) if batch else None
        out = self._collect(self._pending)
        self._pending = new
        return out

    # ------------------------------------------------------------ accounting
    def gpu_launches(self) -> int:
        """Kernels of this library launched so far (direct launches + launches inside replayed
        graphs)."""
        ex = getattr(self.model, "executor", None)
        direct = ex.launches() if ex is not None else 0
        return direct - sum(self._graph_launches.values()) + self._replayed_launches

    def reset_gpu_time(self) -> None:
        self._gpu_events.clear()

    def gpu_time_s(self) -> float:
        """Device time between the first and last operation of every recorded step, summed."""
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in self._gpu_events) * 1e-3

    def has_pending(self) -> bool:
        return self._pending is not None

    def abort_pending(self) -> None:
        """Forget a launched step whose results nobody will collect (its requests were failed by the caller)."""
        self._pending = None

    def release(self, request_id: str) -> None:
        self.kv.release(request_id)
        if self.draft is not None:
            self.draft.release(request_id)
