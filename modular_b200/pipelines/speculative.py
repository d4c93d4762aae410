"""Speculative decoding: propose several tokens cheaply, verify them with one target-model step.

Three proposers:
* ``NgramProposer`` (prompt lookup): continue the longest recent n-gram match in the request's own
  history; no second model.
* ``DraftModelProposer``: a smaller model with its own paged cache decodes ``k`` tokens greedily
  (or by sampling, returning its probabilities for rejection sampling), one sequence at a time.
* ``BatchedDraftProposer``: the same for the serving loop - the draft model has its own paged cache manager
  and batches the requests of a step: ``k`` draft steps over all of them, then one verification step of the
  target (the reference's ``standalone`` draft-model method).

``SpeculativeDecoder.generate`` runs one sequence: each iteration feeds ``[last, d1..dk]`` to the
target as a k+1-token ragged step (logits on every row), accepts the longest valid prefix and one
bonus token, and rewinds the cache length past rejected drafts (their slots are simply overwritten by
the next step). Acceptance rules: exact match for greedy requests (output is identical to plain
greedy decoding) and the residual-distribution rejection sampler otherwise, which preserves the
target distribution.

Reference: max/python/max/pipelines/speculative/ (config, ragged token merger), the rejection
samplers in max/python/max/pipelines/sampling/sampling.py:433-1018 (greedy / residual acceptance).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from .. import ops


@dataclass
class SpeculativeConfig:
    method: str = "ngram"            # "ngram" | "draft_model"
    num_speculative_tokens: int = 4
    ngram_max: int = 4               # longest n-gram to match
    ngram_min: int = 1


@dataclass
class SpecStats:
    steps: int = 0
    proposed: int = 0
    accepted: int = 0
    emitted: int = 0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0

    @property
    def tokens_per_step(self) -> float:
        return self.emitted / self.steps if self.steps else 0.0


class NgramProposer:
    def __init__(self, cfg: SpeculativeConfig):
        self.cfg = cfg

    def propose(self, history: Sequence[int], k: int):
        """Draft tokens (possibly fewer than k, possibly none) and None for their probabilities."""
        import numpy as np

        h = np.asarray(history, dtype=np.int64).reshape(-1)
        if k <= 0:
            return [], None
        for n in range(min(self.cfg.ngram_max, len(h) - 1), self.cfg.ngram_min - 1, -1):
            # the most recent earlier occurrence of the last n tokens (vectorised: the serving loop calls this
            # for every request of every decode step)
            win = np.lib.stride_tricks.sliding_window_view(h[:-1], n)
            hits = np.flatnonzero((win == h[-n:]).all(axis=1))
            if hits.size:
                start = int(hits[-1])
                cont = h[start + n:start + n + k]
                if cont.size:
                    return [int(t) for t in cont], None
        return [], None

    def observe(self, accepted_len: int) -> None:       # nothing to roll back
        pass


class _SeqCache:
    """One sequence's pages in a private cache tensor + the tensors of a ragged single-sequence step."""

    def __init__(self, model, max_len: int):
        c, page = model.cfg, model.page_size
        n_pages = (max_len + page - 1) // page
        self.model, self.page, self.len = model, page, 0
        self.capacity = n_pages * page          # token slots of the private cache
        shape = list(model.kv.shape)
        shape[0] = n_pages + 1
        self.kv = torch.zeros(shape, dtype=model.kv.dtype, device=model.device)
        self.bt = torch.arange(1, n_pages + 1, dtype=torch.int32, device=model.device).unsqueeze(0)

    def step(self, tokens: Sequence[int], all_logits: bool) -> torch.Tensor:
        """Append ``tokens`` at the current length; fp32 logits of every row (or the last)."""
        dev, n = self.model.device, len(tokens)
        if n < 1 or self.len + n > self.capacity:
            # slots past the private cache would be written by the KV-store kernel and read through the block table
            raise ValueError(f"sequence of {self.len} + {n} tokens exceeds the cache capacity of {self.capacity}")
        pos = torch.arange(self.len, self.len + n, dtype=torch.int32, device=dev)
        i32 = lambda v: torch.tensor([v], dtype=torch.int32, device=dev)
        rows = torch.arange(n, dtype=torch.int32, device=dev) if all_logits else i32(n - 1)
        old_kv, self.model.kv = self.model.kv, self.kv
        try:
            logits = self.model.forward_tensors(torch.tensor(list(tokens), dtype=torch.long, device=dev), pos,
                                                (pos.long() + self.page), self.bt, i32(0), i32(n), i32(self.len + n), rows)
        finally:
            self.model.kv = old_kv
        self.len += n
        return logits

    def rewind(self, new_len: int) -> None:
        self.len = new_len


class DraftModelProposer:
    def __init__(self, draft_model, max_len: int, temperature: float = 0.0, generator=None):
        self.cache = _SeqCache(draft_model, max_len)
        self.temperature, self.gen = temperature, generator
        self._fed = 0          # how many tokens of the history the draft cache has consumed

    def propose(self, history: Sequence[int], k: int):
        self.cache.rewind(min(self._fed, len(history) - 1))
        pending = list(history[self.cache.len:])
        drafts, probs = [], []
        # every draft step appends to the draft cache: stop where it would run out
        k = max(0, min(k, self.cache.capacity - self.cache.len - len(pending) + 1))
        for _ in range(k):
            logits = self.cache.step(pending, all_logits=False)[0]
            if self.temperature == 0.0:
                t = int(torch.argmax(logits))
                probs.append(None)
            else:
                p = torch.softmax(logits / self.temperature, -1)
                t = int(torch.multinomial(p.cpu(), 1, generator=self.gen))
                probs.append(p.cpu())
            drafts.append(t)
            pending = [t]
        self._fed = len(history)       # the drafts after it are speculative
        return drafts, (probs if self.temperature > 0.0 else None)

    def observe(self, accepted_len: int) -> None:
        pass


class BatchedDraftProposer:
    """Draft-model proposals for all requests of a serving step (reference: the ``standalone`` method of
    max/python/max/pipelines/speculative/, where a second pipeline model with its own KV cache drafts).

    Every request has a mirror context in the draft model's own paged cache. Before drafting, a mirror is brought
    in line with the request's accepted tokens (its rejected drafts are cut off at the first difference; cache
    rows behind that point are simply written again), then the mirrors step together: prompts catch up in chunks,
    and every further step appends one greedy draft token per request that still has room."""

    def __init__(self, draft_model, kv_manager, max_batch_tokens: int, max_batch_size: int, target_kv=None):
        from .batch import BatchPacker

        self.model, self.kv = draft_model, kv_manager
        self.target_kv = target_kv      # requests that left the target's cache lose their mirror at the next step
        cfg = draft_model.cfg
        self.device = draft_model.device
        self.packer = BatchPacker(cfg.num_attention_heads, cfg.num_key_value_heads, kv_manager.page_size,
                                  max_batch_tokens, max_batch_size, kv_manager.max_pages_per_seq, device=self.device)
        self.mirror: dict = {}
        self.draft_steps = 0
        self._step = 0

    def release(self, request_id: str) -> None:
        m = self.mirror.pop(request_id, None)
        if m is not None and self.kv.contains(m.request_id):
            self.kv.release(m.request_id)

    def _sync(self, ctx):
        import numpy as np

        from .context import TextContext

        hist = ctx.tokens.all
        m = self.mirror.get(ctx.request_id)
        if m is None:
            from .context import SamplingParams

            # greedy drafts: the device-side sampler reads the mirror's parameters
            m = TextContext.from_prompt(hist, ctx.max_length, request_id="draft:" + ctx.request_id,
                                        sampling_params=SamplingParams(temperature=0.0))
            self.kv.claim(m)
            self.mirror[ctx.request_id] = m
            return m
        mt = m.tokens
        n = min(len(mt), len(hist))
        diff = np.flatnonzero(mt.all[:n] != hist[:n])
        keep = max(int(diff[0]) if diff.size else n, mt.prompt_len)
        mt.truncate(keep)
        for t in hist[keep:]:
            mt.advance_with_token(int(t))
        mt.processed = min(mt.processed, len(mt) - 1)      # at least the newest token is fed again
        mt.active_end = len(mt)
        return m

    def _forward(self, sel) -> list:
        """One draft step over ``sel`` (their active windows); the greedy token after each window."""
        from .batch import BatchPacker

        self._step += 1
        self.draft_steps += 1
        sb = self.packer.pack(sel, self.kv)
        if self.device.type == "cuda" and getattr(self.model, "use_executor", False):
            meta = self.packer.upload(sb)
            self.model.forward_packed(meta, sb.offsets, sb.T, sb.B, sb.bt_stride, sb.n_tiles, sb.n_decode, sb.n_logits,
                                      False, True, self._step)
            return [int(v) for v in self.model.sampled[: sb.n_logits].cpu().numpy()]
        t = BatchPacker.tensors(sb, self.device)
        logits = self.model.forward_tensors(t["tokens"], t["positions"], t["slots"], t["block_table"], t["q_start"],
                                            t["q_len"], t["kv_len"], t["logit_rows"])
        return [int(v) for v in ops.argmax(logits).cpu().numpy()]

    def propose_batch(self, batch, rooms: Sequence[int]) -> list:
        """Up to ``rooms[i]`` greedy draft tokens for ``batch[i]`` (fewer when the draft cache is full)."""
        if self.target_kv is not None:
            for rid in [r for r in self.mirror if not self.target_kv.contains(r)]:
                self.release(rid)
        mirrors = [self._sync(c) for c in batch]
        want = [max(0, int(r)) for r in rooms]
        drafts = [[] for _ in batch]
        while True:
            budget = self.packer.max_tokens
            sel = []
            for i, m in enumerate(mirrors):
                if len(drafts[i]) >= want[i] or budget <= 0 or len(sel) >= self.packer.max_seqs:
                    continue
                mt = m.tokens
                mt.active_end = len(mt)
                mt.chunk(budget)
                if not self.kv.can_alloc(m) or len(mt) >= m.max_length:
                    want[i] = len(drafts[i])               # no pages left for this request: stop drafting for it
                    continue
                self.kv.alloc(m)
                budget -= mt.active_length
                sel.append(i)
            if not sel:
                break
            toks = iter(self._forward([mirrors[i] for i in sel]))
            for i in sel:
                mt = mirrors[i].tokens
                whole = mt.active_end == len(mt)           # a chunk of a prompt has no logit row: no next token yet
                mt.advance_processed()
                if whole:
                    t = next(toks)
                    drafts[i].append(t)
                    mt.advance_with_token(t)
        return drafts


class SpeculativeDecoder:
    def __init__(self, target_model, cfg: SpeculativeConfig = SpeculativeConfig(), draft_model=None,
                 max_len: int = 2048):
        self.target, self.cfg, self.draft, self.max_len = target_model, cfg, draft_model, max_len
        self.stats = SpecStats()
        if cfg.method == "draft_model" and draft_model is None:
            raise ValueError("method draft_model needs a draft model")

    def generate(self, prompt: Sequence[int], max_new_tokens: int, temperature: float = 0.0,
                 eos_token_ids: Sequence[int] = (), seed: int = 0) -> list:
        if len(prompt) < 1 or len(prompt) >= self.max_len:
            raise ValueError(f"prompt of {len(prompt)} tokens does not fit max_len {self.max_len} with room to generate")
        gen = torch.Generator().manual_seed(seed)
        k = self.cfg.num_speculative_tokens
        proposer = (DraftModelProposer(self.draft, self.max_len, temperature, gen) if self.cfg.method == "draft_model"
                    else NgramProposer(self.cfg))
        cache = _SeqCache(self.target, self.max_len)
        history = list(prompt)
        out: list = []
        # prefill everything but the last prompt token; each iteration then feeds [last] + drafts
        if len(history) > 1:
            cache.step(history[:-1], all_logits=False)
        while len(out) < max_new_tokens:
            if len(history) >= self.max_len:
                return out          # length finish: the next step would not fit the cache
            budget = min(k, max_new_tokens - len(out) - 1, self.max_len - len(history) - 1)
            drafts, q = proposer.propose(history, budget) if budget > 0 else ([], None)
            base = cache.len
            logits = cache.step([history[-1]] + list(drafts), all_logits=True)      # [len(drafts) + 1, V]
            accepted, bonus = self._verify(logits, drafts, q, temperature, gen)
            self.stats.steps += 1
            self.stats.proposed += len(drafts)
            self.stats.accepted += accepted
            new = list(drafts[:accepted]) + [bonus]
            cache.rewind(base + 1 + accepted)        # rows of rejected drafts are overwritten next step
            for t in new:
                out.append(t)
                history.append(t)
                self.stats.emitted += 1
                if t in eos_token_ids or len(out) >= max_new_tokens:
                    return out
        return out

    @staticmethod
    def _verify(logits, drafts, q, temperature, gen):
        """Returns (number of accepted drafts, the token that follows them)."""
        if temperature == 0.0:
            top = ops.argmax(logits).tolist()
            a = 0
            while a < len(drafts) and top[a] == drafts[a]:
                a += 1
            return a, int(top[a])
        p = torch.softmax(logits.float().cpu() / temperature, -1)
        for i, d in enumerate(drafts):
            qi = q[i][d] if q is not None else 1.0        # n-gram drafts are a point mass
            if torch.rand((), generator=gen) < torch.clamp(p[i, d] / qi, max=1.0):
                continue
            resid = p[i].clone()
            if q is not None:
                resid = torch.clamp(resid - q[i], min=0.0)
            else:
                resid[d] = 0.0
            resid = resid / resid.sum().clamp_min(1e-20)
            return i, int(torch.multinomial(resid, 1, generator=gen))
        return len(drafts), int(torch.multinomial(p[len(drafts)], 1, generator=gen))
