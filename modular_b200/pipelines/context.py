"""Request state: token buffer, sampling parameters, generation status, outputs.

Same vocabulary as the reference (max/python/max/pipelines/context/tokens.py:165
``TokenBuffer``; context.py:454 ``TextContext``; sampling_params.py:208 ``SamplingParams``)
so schedulers and pipelines written against one read naturally against the other.

A ``TokenBuffer`` holds every token of a request (prompt then generated) and three
cursors:

    [0, processed)            tokens whose KV entries are already in the cache
    [processed, active_end)   the *active window* the next forward pass consumes
    [active_end, len)         prompt tokens deferred to later chunks (chunked prefill)
"""

from __future__ import annotations

import enum
import itertools
import time
from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

import numpy as np

FUTURE_TOKEN = -999  # placeholder for a token sampled on the device but not yet read back


class GenerationStatus(str, enum.Enum):
    ACTIVE = "active"
    END_OF_SEQUENCE = "end_of_sequence"
    MAXIMUM_LENGTH = "maximum_length"
    CANCELLED = "cancelled"
    ERROR = "error"              # the request could not be served (e.g. its grammar does not compile)

    @property
    def is_done(self) -> bool:
        return self is not GenerationStatus.ACTIVE


@dataclass
class SamplingParams:
    top_k: int = -1
    top_p: float = 1.0
    min_p: float = 0.0
    temperature: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    max_new_tokens: Optional[int] = None
    min_new_tokens: int = 0
    ignore_eos: bool = False
    stop: Optional[list[str]] = None
    stop_token_ids: Optional[list[int]] = None
    detokenize: bool = True
    seed: int = 0
    logprobs: int = 0
    # grammar spec for constrained decoding: {"type": "json_object" | "json_schema" | "regex" | "ebnf", ...}
    response_format: Optional[dict] = None
    # additive bias on the logits of given token ids before sampling (OpenAI ``logit_bias``; -100 bans a token)
    logit_bias: Optional[dict] = None

    def __post_init__(self):
        # any integer is a seed; 40 bits of it are kept (it is multiplied by a 20-bit constant into an int64 stream id)
        self.seed = int(self.seed or 0) & 0xFFFFFFFFFF
        if self.max_new_tokens is not None and self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must not be negative")
        if self.logit_bias:
            try:
                self.logit_bias = {int(k): float(v) for k, v in self.logit_bias.items()}
            except (TypeError, ValueError) as e:
                raise ValueError("logit_bias must map token ids to numbers") from e
            if any(k < 0 for k in self.logit_bias) or any(not -100.0 <= v <= 100.0 for v in self.logit_bias.values()):
                raise ValueError("logit_bias: token ids must be >= 0 and values in [-100, 100]")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")
        if self.top_k == 0 or self.top_k < -1:
            raise ValueError("top_k must be -1 (off) or >= 1")

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1

    @property
    def needs_penalties(self) -> bool:
        return (self.frequency_penalty != 0.0 or self.presence_penalty != 0.0
                or self.repetition_penalty != 1.0 or bool(self.logit_bias))


class TokenBuffer:
    """Growable int64 token array with prompt/generated/active/processed windows."""

    __slots__ = ("_arr", "_len", "prompt_len", "processed", "active_end")

    def __init__(self, prompt: Sequence[int] | np.ndarray):
        p = np.asarray(prompt, dtype=np.int64).reshape(-1)
        if p.size == 0:
            raise ValueError("prompt must contain at least one token")
        cap = max(64, int(p.size * 1.5))
        self._arr = np.empty(cap, dtype=np.int64)
        self._arr[: p.size] = p
        self._len = int(p.size)
        self.prompt_len = int(p.size)
        self.processed = 0
        self.active_end = self._len

    # ---- views
    def __len__(self) -> int:
        return self._len

    @property
    def all(self) -> np.ndarray:
        return self._arr[: self._len]

    @property
    def prompt(self) -> np.ndarray:
        return self._arr[: self.prompt_len]

    @property
    def generated(self) -> np.ndarray:
        return self._arr[self.prompt_len : self._len]

    @property
    def active(self) -> np.ndarray:
        return self._arr[self.processed : self.active_end]

    @property
    def active_length(self) -> int:
        return self.active_end - self.processed

    @property
    def generated_length(self) -> int:
        return self._len - self.prompt_len

    # ---- mutation
    def chunk(self, max_tokens: int) -> None:
        """Shrink the active window to at most ``max_tokens`` (chunked prefill)."""
        if max_tokens < 1:
            raise ValueError("chunk size must be >= 1")
        self.active_end = min(self._len, self.processed + max_tokens)

    def skip_processing(self, n: int) -> None:
        """Mark ``n`` leading active tokens as already cached (prefix-cache hit)."""
        if n < 0 or n >= self.active_length:
            raise ValueError("must leave at least one active token")
        self.processed += n

    def advance_processed(self) -> None:
        """The active window was consumed by a forward pass; open the next window."""
        self.processed = self.active_end
        self.active_end = self._len

    def advance_with_token(self, token: int) -> None:
        """Append a generated token; it becomes the next active window."""
        if self._len == self._arr.size:
            arr = np.empty(self._arr.size * 2, dtype=np.int64)
            arr[: self._len] = self._arr[: self._len]
            self._arr = arr
        self._arr[self._len] = token
        self._len += 1
        self.active_end = self._len

    def set_token(self, index: int, token: int) -> None:
        self._arr[index] = token

    def truncate(self, length: int) -> None:
        """Drop tokens past ``length`` (tentative draft tokens that were not accepted)."""
        if length < self.prompt_len or length > self._len:
            raise ValueError("truncate: length out of range")
        self._len = length
        self.active_end = min(self.active_end, length)
        self.processed = min(self.processed, length)

    def reset(self) -> None:
        """Forget cache state (after preemption): everything becomes one prompt again."""
        self.processed = 0
        self.active_end = self._len


@dataclass
class TextGenerationOutput:
    request_id: str
    tokens: list[int]
    final_status: GenerationStatus = GenerationStatus.ACTIVE
    log_probabilities: Optional[list[Any]] = None
    error: Optional[str] = None          # with final_status ERROR: what to tell the client

    @property
    def is_done(self) -> bool:
        return self.final_status.is_done


@dataclass
class EmbeddingsOutput:
    """Final (and only) answer to an embeddings request."""
    request_id: str
    embedding: list
    prompt_tokens: int = 0
    final_status: GenerationStatus = GenerationStatus.END_OF_SEQUENCE
    tokens: tuple = ()

    @property
    def is_done(self) -> bool:
        return True


_req_counter = itertools.count()


@dataclass
class TextContext:
    """Everything the scheduler and pipeline know about one request."""

    request_id: str
    tokens: TokenBuffer
    max_length: int
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    eos_token_ids: frozenset = frozenset()
    model_name: str = ""
    status: GenerationStatus = GenerationStatus.ACTIVE
    arrival_time: float = field(default_factory=time.perf_counter)
    task: str = "generate"          # "generate" | "embed" (answered by the embeddings scheduler)
    pooling: str = "last"
    grammar_state: Any = None       # matcher of a grammar-constrained request (built inside the worker)
    lora_name: Optional[str] = None  # adapter applied to this request (None = base model)
    # one entry per generated token when sampling_params.logprobs > 0:
    # {"token": id, "logprob": float, "top": [(id, logprob), ...]}
    logprob_entries: list = field(default_factory=list)
    logprobs_emitted: int = 0
    first_token_time: Optional[float] = None
    last_token_time: Optional[float] = None
    # bookkeeping owned by the engine
    pending_future: int = 0          # tokens sampled on device whose values are still in flight
    emitted: int = 0                 # generated tokens already handed to the caller
    sample_slot: int = -1            # row of this request in the previous step's sampled-token buffer
    dp_replica: int = 0
    # salt of this request's prefix-cache hashes: the caller's own salt (requests with different salts never
    # share pages); the scheduler folds the adapter identity in before the first claim
    cache_salt: int = 0
    json_schema: Optional[str] = None
    matcher: Any = None
    seq: int = field(default_factory=lambda: next(_req_counter))

    @classmethod
    def from_prompt(cls, prompt_ids, max_length: int, request_id: Optional[str] = None,
                    sampling_params: Optional[SamplingParams] = None, eos_token_ids=(), **kw):
        rid = request_id or f"req-{next(_req_counter)}"
        return cls(request_id=rid, tokens=TokenBuffer(prompt_ids), max_length=max_length,
                   sampling_params=sampling_params or SamplingParams(),
                   eos_token_ids=frozenset(eos_token_ids), **kw)

    # ---- derived
    @property
    def is_done(self) -> bool:
        return self.status.is_done

    @property
    def current_length(self) -> int:
        return len(self.tokens)

    @property
    def max_new_tokens_effective(self) -> int:
        room = self.max_length - self.tokens.prompt_len
        m = self.sampling_params.max_new_tokens
        return max(0, room if m is None else min(m, room))

    @property
    def needs_ce(self) -> bool:
        """True when the next pass is context encoding (prompt, chunk or re-encode after
        preemption) rather than a single-token decode step."""
        t = self.tokens
        return t.active_length > 1 or t.active_end < len(t) or t.generated_length == 0

    # ---- updates
    def _check_done(self, token: int) -> None:
        sp = self.sampling_params
        n_gen = self.tokens.generated_length
        if n_gen >= self.max_new_tokens_effective or len(self.tokens) >= self.max_length:
            self.status = GenerationStatus.MAXIMUM_LENGTH
            return
        if n_gen < sp.min_new_tokens or token == FUTURE_TOKEN:
            return
        if not sp.ignore_eos and token in self.eos_token_ids:
            self.status = GenerationStatus.END_OF_SEQUENCE
        elif sp.stop_token_ids and token in sp.stop_token_ids:
            self.status = GenerationStatus.END_OF_SEQUENCE

    def update(self, token: int) -> None:
        """Record a sampled token whose value is known."""
        now = time.perf_counter()
        if self.first_token_time is None:
            self.first_token_time = now
        self.last_token_time = now
        self.tokens.advance_with_token(int(token))
        self._check_done(int(token))

    def update_with_future_token(self) -> None:
        """Record that a token was sampled on the device; its value arrives later."""
        self.tokens.advance_with_token(FUTURE_TOKEN)
        self.pending_future += 1
        self._check_done(FUTURE_TOKEN)

    def realize_future_token(self, token: int) -> None:
        """Fill in the oldest outstanding placeholder with the value read back."""
        if self.pending_future <= 0:
            raise RuntimeError("no future token outstanding")
        idx = len(self.tokens) - self.pending_future
        self.tokens.set_token(idx, int(token))
        self.pending_future -= 1
        now = time.perf_counter()
        if self.first_token_time is None:
            self.first_token_time = now
        self.last_token_time = now
        if self.status is GenerationStatus.ACTIVE or self.status is GenerationStatus.MAXIMUM_LENGTH:
            sp = self.sampling_params
            n_gen = idx - self.tokens.prompt_len + 1
            if n_gen >= sp.min_new_tokens and (
                (not sp.ignore_eos and int(token) in self.eos_token_ids)
                or (sp.stop_token_ids and int(token) in sp.stop_token_ids)
            ):
                self.status = GenerationStatus.END_OF_SEQUENCE

    def reset(self) -> None:
        """Return to the pre-prefill state keeping generated tokens (used on preemption)."""
        self.tokens.reset()

    def to_generation_output(self) -> TextGenerationOutput:
        """Tokens generated since the last call (only those whose values are known)."""
        known_end = len(self.tokens) - self.pending_future
        start = self.tokens.prompt_len + self.emitted
        toks = [int(t) for t in self.tokens.all[start:known_end]]
        if self.status is GenerationStatus.END_OF_SEQUENCE and toks:
            # tokens speculatively produced after the stop token are dropped
            for i, t in enumerate(toks):
                sp = self.sampling_params
                if (not sp.ignore_eos and t in self.eos_token_ids) or (
                    sp.stop_token_ids and t in sp.stop_token_ids
                ):
                    toks = toks[: i + 1]
                    break
        lps = None
        if self.sampling_params.logprobs and toks:
            lps = self.logprob_entries[self.logprobs_emitted:self.logprobs_emitted + len(toks)]
            self.logprobs_emitted += len(toks)
        self.emitted += len(toks)
        done = self.is_done and self.pending_future == 0
        if lps is not None:
            return TextGenerationOutput(self.request_id, toks,
                                        self.status if done else GenerationStatus.ACTIVE, lps)
        return TextGenerationOutput(self.request_id, toks,
                                    self.status if done else GenerationStatus.ACTIVE)
