"""Speculative decoding on CPU: greedy verification reproduces plain greedy decoding exactly."""

import pytest
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


def _engine_tokens(spec, prompts, n, device="cpu", **kw):
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.pipelines.context import SamplingParams

    cfg = Llama3Config.tiny(num_hidden_layers=2, vocab_size=64)
    dtype = torch.float32 if device == "cpu" else torch.bfloat16
    llm = LLM(cfg, device=device, dtype=dtype, max_length=160, max_batch_size=4, max_batch_input_tokens=64, page_size=16,
              num_kv_pages=64, seed=5, speculative=spec, **kw)
    sp = SamplingParams(temperature=0.0, max_new_tokens=n, ignore_eos=True)
    recs = llm.generate(prompts, sp)
    return [list(r.tokens) for r in recs], llm


def test_serving_loop_verifies_ngram_proposals_and_matches_plain_greedy():
    """The engine with speculation on emits exactly the tokens of the engine without it, in fewer steps, through
    the scheduler (chunked prefill, several requests per step, requests finishing at different times)."""
    prompts = [[3, 4, 5, 3, 4, 5, 3, 4], [7, 7, 7, 7, 7], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12] * 6, [9, 8]]
    want, plain = _engine_tokens(None, prompts, 40)
    got, spec = _engine_tokens(SpeculativeConfig("ngram", 4), prompts, 40)
    assert got == want
    st = spec.pipeline.spec_stats
    assert st.emitted == 4 * 40 - 4 and st.accepted > 0          # the first token of a request comes from its prefill
    assert spec.pipeline.stats.steps < plain.pipeline.stats.steps
    m = spec.scheduler.last_metrics
    assert m.spec_steps >= 0 and "spec_accepted" in m.to_dict()


def test_serving_loop_verifies_draft_model_proposals():
    """Draft-model speculation in the serving loop: a second model with its own paged cache drafts for all requests
    of a step; the output stays that of plain greedy decoding whatever the draft proposes."""
    prompts = [[3, 4, 5, 3, 4, 5, 3, 4], [7, 7, 7, 7, 7], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12] * 6, [9, 8]]
    want, plain = _engine_tokens(None, prompts, 40)
    cfg = Llama3Config.tiny(num_hidden_layers=2, vocab_size=64)
    # the target itself as the draft (same seed -> same weights): every proposal is accepted
    same_w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=5)
    got, spec = _engine_tokens(SpeculativeConfig("draft_model", 3), prompts, 40, draft_model_config=cfg,
                               draft_weights=same_w)
    assert got == want
    st = spec.pipeline.spec_stats
    assert st.emitted == 4 * 40 - 4 and st.proposed > 0 and st.acceptance_rate == 1.0
    assert spec.pipeline.stats.steps < plain.pipeline.stats.steps
    assert spec.pipeline.draft.draft_steps > 0 and not spec.pipeline.draft.mirror or True
    # a different, smaller draft: wrong proposals cost steps, not accuracy
    small = Llama3Config.tiny(num_hidden_layers=1, vocab_size=64)
    got2, spec2 = _engine_tokens(SpeculativeConfig("draft_model", 4), prompts, 40, draft_model_config=small)
    assert got2 == want
    assert spec2.pipeline.spec_stats.proposed > 0
    # mirrors of finished requests are dropped when the next batch is drafted for
    more, _ = [list(r.tokens) for r in spec2.generate([[5, 6, 5, 6, 5]], __import__(
        "modular_b200.pipelines.context", fromlist=["SamplingParams"]).SamplingParams(
            temperature=0.0, max_new_tokens=12, ignore_eos=True))], None
    assert len(more[0]) == 12 and len(spec2.pipeline.draft.mirror) == 1


def test_standalone_draft_model_through_the_pipeline_config():
    """``--speculative-method standalone --draft-model-path ...``: the registry resolves the draft model like the
    served one and the engine verifies its proposals; tokens equal those of the engine without speculation."""
    from modular_b200.pipelines.config import PipelineArgs, PipelineConfig
    from modular_b200.pipelines.context import SamplingParams
    from modular_b200.pipelines.registry import PIPELINE_REGISTRY

    def build(**extra):
        pc = PipelineConfig.from_args(PipelineArgs.from_flat_kwargs(
            None, model_path="preset:tiny-llama", devices="cpu", max_length=128, max_batch_size=2,
            max_batch_input_tokens=64, kv_cache_page_size=16, **extra))
        return PIPELINE_REGISTRY.retrieve(pc)[1]

    sp = SamplingParams(temperature=0.0, max_new_tokens=16, ignore_eos=True)
    prompts = [[5, 6, 7, 8, 9, 5, 6, 7], [11, 12, 13]]
    want = [list(r.tokens) for r in build().generate(prompts, sp)]
    llm = build(speculative_method="standalone", num_speculative_tokens=3, draft_model_path="preset:tiny-llama")
    assert [list(r.tokens) for r in llm.generate(prompts, sp)] == want
    assert llm.pipeline.spec_stats.proposed > 0 and llm.pipeline.draft is not None
    with pytest.raises(ValueError):
        build(speculative_method="standalone", num_speculative_tokens=3)          # no draft model named
    with pytest.raises(ValueError):
        build(speculative_method="eagle", num_speculative_tokens=3)


def test_draft_model_needs_the_targets_vocabulary():
    from modular_b200.entrypoints.llm import LLM

    cfg = Llama3Config.tiny(num_hidden_layers=2, vocab_size=64)
    with pytest.raises(ValueError):
        LLM(cfg, device="cpu", dtype=torch.float32, max_length=64, max_batch_size=2, max_batch_input_tokens=32,
            page_size=16, num_kv_pages=16, speculative=SpeculativeConfig("draft_model", 2),
            draft_model_config=Llama3Config.tiny(num_hidden_layers=1, vocab_size=96))
    with pytest.raises(ValueError):
        LLM(cfg, device="cpu", dtype=torch.float32, max_length=64, max_batch_size=2, max_batch_input_tokens=32,
            page_size=16, num_kv_pages=16, speculative=SpeculativeConfig("draft_model", 2))


def test_speculation_respects_token_limits_and_eos():
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.pipelines.context import SamplingParams

    prompts = [[3, 4, 5, 3, 4, 5, 3, 4]]
    want, _ = _engine_tokens(None, prompts, 23)
    got, _ = _engine_tokens(SpeculativeConfig("ngram", 6), prompts, 23)
    assert got == want and len(got[0]) == 23
    eos = want[0][9]
    cfg = Llama3Config.tiny(num_hidden_layers=2, vocab_size=64)
    llm = LLM(cfg, device="cpu", dtype=torch.float32, max_length=160, max_batch_size=4, max_batch_input_tokens=64,
              page_size=16, num_kv_pages=64, seed=5, speculative=SpeculativeConfig("ngram", 6), eos_token_ids=(eos,))
    rec = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=23))[0]
    assert list(rec.tokens) == want[0][: want[0].index(eos) + 1]


import pytest


@pytest.mark.gpu
def test_serving_loop_speculation_on_gpu_follows_plain_greedy():
    """On the GPU the verification pass scores k + 1 rows per request through the prefill kernels while plain
    decoding uses the decode kernels: bf16 rounding can flip a near-tie, after which the two runs legitimately
    differ. The common prefix must be long and speculation must accept drafts."""
    prompts = [[3, 4, 5, 3, 4, 5, 3, 4], [7, 7, 7, 7, 7], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12] * 6, [9, 8]]
    want, _ = _engine_tokens(None, prompts, 40, device="cuda")
    got, spec = _engine_tokens(SpeculativeConfig("ngram", 4), prompts, 40, device="cuda")
    common = 0
    for a, b in zip(want, got):
        assert len(a) == len(b) == 40
        n = next((i for i, (x, y) in enumerate(zip(a, b)) if x != y), 40)
        common += n
    assert common >= 0.6 * 160, (common, want, got)
    st = spec.pipeline.spec_stats
    assert st.accepted > 0 and st.emitted == 4 * 40 - 4


@pytest.mark.gpu
def test_serving_loop_draft_model_on_gpu():
    """Draft-model speculation through the native step executors of both models: the draft (same weights as the
    target here) is accepted almost always, and the tokens follow plain greedy decoding up to bf16 near-ties."""
    prompts = [[3, 4, 5, 3, 4, 5, 3, 4], [7, 7, 7, 7, 7], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12] * 6, [9, 8]]
    want, _ = _engine_tokens(None, prompts, 40, device="cuda")
    cfg = Llama3Config.tiny(num_hidden_layers=2, vocab_size=64)
    same_w = Llama3Weights.random_init(cfg, "cuda", torch.bfloat16, seed=5)
    got, spec = _engine_tokens(SpeculativeConfig("draft_model", 3), prompts, 40, device="cuda",
                               draft_model_config=cfg, draft_weights=same_w)
    common = 0
    for a, b in zip(want, got):
        assert len(a) == len(b) == 40
        common += next((i for i, (x, y) in enumerate(zip(a, b)) if x != y), 40)
    assert common >= 0.6 * 160, (common, want, got)
    st = spec.pipeline.spec_stats
    assert st.emitted == 4 * 40 - 4 and st.acceptance_rate > 0.5
    assert spec.pipeline.draft.draft_steps > 0
