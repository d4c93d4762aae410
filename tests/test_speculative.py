"""Speculative decoding on CPU: greedy verification reproduces plain greedy decoding exactly."""

import torch

from modular_b200.models.llama3 import Llama3Config, Llama3Model, Llama3Weights
from modular_b200.pipelines.speculative import NgramProposer, SpeculativeConfig, SpeculativeDecoder


def _model(seed, layers=2):
    cfg = Llama3Config.tiny(num_hidden_layers=layers, vocab_size=64)
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=seed, std=0.08)
    kv = torch.zeros(2, 2, cfg.num_hidden_layers, cfg.num_key_value_heads, 16, cfg.head_dim)
    return Llama3Model(cfg, w, kv)


def _plain_greedy(model, prompt, n):
    dec = SpeculativeDecoder(model, SpeculativeConfig(num_speculative_tokens=0), max_len=256)
    return dec.generate(prompt, n)


def test_ngram_proposer_continues_most_recent_match():
    p = NgramProposer(SpeculativeConfig(ngram_max=3))
    assert p.propose([1, 2, 3, 9, 1, 2, 3], 2)[0] == [9, 1]
    assert p.propose([5, 6, 7], 3)[0] == []


def test_greedy_speculation_is_exact_with_ngram_and_draft_model():
    target = _model(0)
    prompt = [3, 4, 5, 3, 4, 5, 3, 4]
    want = _plain_greedy(target, prompt, 24)
    ng = SpeculativeDecoder(target, SpeculativeConfig("ngram", 4), max_len=256)
    assert ng.generate(prompt, 24) == want
    assert ng.stats.emitted == 24 and ng.stats.steps <= 24
    same = SpeculativeDecoder(target, SpeculativeConfig("draft_model", 3), draft_model=_model(0), max_len=256)
    assert same.generate(prompt, 24) == want
    assert same.stats.acceptance_rate == 1.0 and same.stats.steps <= 7      # k + 1 tokens per step
    other = SpeculativeDecoder(target, SpeculativeConfig("draft_model", 3), draft_model=_model(1, layers=1), max_len=256)
    assert other.generate(prompt, 24) == want                               # wrong drafts cost speed, not accuracy


def test_rejection_sampling_runs_and_respects_eos():
    target = _model(0)
    dec = SpeculativeDecoder(target, SpeculativeConfig("draft_model", 3), draft_model=_model(2, layers=1), max_len=256)
    out = dec.generate([1, 2, 3], 30, temperature=0.8, seed=3)
    assert 1 <= len(out) <= 30 and all(0 <= t < 64 for t in out)
    greedy = _plain_greedy(target, [3, 4, 5, 3, 4], 20)
    eos = greedy[6]
    cut = SpeculativeDecoder(target, SpeculativeConfig("ngram", 3), max_len=256).generate(
        [3, 4, 5, 3, 4], 20, eos_token_ids=(eos,))
    assert cut == greedy[: greedy.index(eos) + 1]


def test_generation_stops_at_the_cache_capacity():
    """The private caches hold ceil(max_len / page) pages: prompts that do not fit are refused, generation ends
    with a length finish before a step would write past them, and the draft cache is bounded the same way."""
    import pytest

    target = _model(0)
    with pytest.raises(ValueError):
        SpeculativeDecoder(target, SpeculativeConfig("ngram", 4), max_len=32).generate(list(range(32)), 4)
    prompt = [3, 4, 5, 3, 4, 5, 3, 4]
    want = _plain_greedy(target, prompt, 24)
    for method, draft in (("ngram", None), ("draft_model", _model(0))):
        dec = SpeculativeDecoder(target, SpeculativeConfig(method, 4), draft_model=draft, max_len=20)
        out = dec.generate(prompt, 64)
        assert len(prompt) + len(out) <= 20 and out == want[: len(out)] and len(out) >= 11
    from modular_b200.pipelines.speculative import _SeqCache
    cache = _SeqCache(target, 16)
    cache.step(list(range(16)), all_logits=False)
    with pytest.raises(ValueError):
        cache.step([1], all_logits=False)
