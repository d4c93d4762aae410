"""End-to-end engine tests on CPU: tiny Llama-3 in fp32 through LLM.generate against an
eager reference (full-sequence attention, no cache, no batching)."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from modular_b200.entrypoints.llm import LLM
from modular_b200.models.llama3 import Llama3Config, Llama3Weights
from modular_b200.nn.rotary_embedding import RopeScaling, cos_sin_table
from modular_b200.pipelines.context import SamplingParams


def eager_logits(cfg, w, ids):
    """Plain fp32 forward over a whole sequence; returns logits for every position."""
    T = len(ids)
    hd, nq, nkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    cs = cos_sin_table(hd, T, cfg.rope_theta, RopeScaling.from_hf(cfg.rope_scaling))
    cos, sin = cs[:, : hd // 2], cs[:, hd // 2 :]

    def rope(x):
        a, b = x[..., : hd // 2], x[..., hd // 2 :]
        c, s = cos[:, None], sin[:, None]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    def norm(x, g):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * g

    h = w.embed[torch.as_tensor(ids)].float()
    for l in w.layers:
        x = norm(h, l.attn_norm.float())
        qkv = x @ l.wqkv.float().t()
        q, k, v = torch.split(qkv, [cfg.q_dim, cfg.kv_dim, cfg.kv_dim], -1)
        q, k, v = rope(q.view(T, nq, hd)), rope(k.view(T, nkv, hd)), v.view(T, nkv, hd)
        k, v = k.repeat_interleave(nq // nkv, 1), v.repeat_interleave(nq // nkv, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / hd**0.5
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        a = torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(T, -1)
        h = h + a @ l.wo.float().t()
        x = norm(h, l.mlp_norm.float())
        gu = x @ l.wgu.float().t()
        g, u = gu[:, : cfg.intermediate_size], gu[:, cfg.intermediate_size :]
        h = h + (F.silu(g) * u) @ l.wd.float().t()
    return norm(h, w.final_norm.float()) @ w.lm_head.float().t()


def eager_greedy(cfg, w, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(eager_logits(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.fixture(scope="module")
def tiny():
    cfg = Llama3Config.tiny()
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=0)
    return cfg, w


def _llm(cfg, w, **kw):
    args = dict(device="cpu", dtype=torch.float32, max_length=512, max_batch_size=8,
                max_batch_input_tokens=256, page_size=16, num_kv_pages=200)
    args.update(kw)
    return LLM(cfg, w, **args)


def test_greedy_matches_eager(tiny):
    cfg, w = tiny
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (128, 128, 37, 5)]
    llm = _llm(cfg, w)
    recs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True))
    for p, r in zip(prompts, recs):
        assert r.finished and len(r.tokens) == 8
        assert r.tokens == eager_greedy(cfg, w, p, 8)


def test_logits_match_eager(tiny):
    cfg, w = tiny
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, cfg.vocab_size, size=128).tolist()
    llm = _llm(cfg, w)
    llm.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=1, ignore_eos=True))
    ref = eager_logits(cfg, w, prompt)[-1]
    got = llm.pipeline.last_logits[0]
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-4)


@pytest.mark.parametrize("budget,inflight", [(32, False), (48, True), (1000, True)])
def test_chunked_prefill_and_inflight_batching(tiny, budget, inflight):
    cfg, w = tiny
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (100, 61, 17, 90, 33)]
    llm = _llm(cfg, w, max_batch_input_tokens=budget, enable_in_flight_batching=inflight)
    recs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True),
                        max_concurrency=3)
    for p, r in zip(prompts, recs):
        assert r.tokens == eager_greedy(cfg, w, p, 6)
    assert llm.kv.pool.used_blocks == 0  # everything released


def test_prefix_cache_reuse(tiny):
    cfg, w = tiny
    rng = np.random.default_rng(3)
    shared = rng.integers(0, cfg.vocab_size, size=80).tolist()
    p1 = shared + rng.integers(0, cfg.vocab_size, size=10).tolist()
    p2 = shared + rng.integers(0, cfg.vocab_size, size=12).tolist()
    llm = _llm(cfg, w)
    sp = SamplingParams(temperature=0.0, max_new_tokens=4, ignore_eos=True)
    r1 = llm.generate([p1], sp)[0]
    assert llm.kv.prefix_hit_tokens == 0
    r2 = llm.generate([p2], sp)[0]
    assert llm.kv.prefix_hit_tokens == 80  # five 16-token pages shared
    assert r1.tokens == eager_greedy(cfg, w, p1, 4)
    assert r2.tokens == eager_greedy(cfg, w, p2, 4)


def test_preemption_when_cache_is_small(tiny):
    cfg, w = tiny
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg.vocab_size, size=40).tolist() for _ in range(4)]
    # 12 usable pages of 16 tokens: four 40-token prompts (3 pages each) fill it; decoding
    # past 48 tokens per request forces preemption
    llm = _llm(cfg, w, num_kv_pages=13, enable_prefix_caching=False)
    recs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True))
    assert llm.scheduler.batch_constructor.total_preemptions > 0
    for p, r in zip(prompts, recs):
        assert r.tokens == eager_greedy(cfg, w, p, 12)


def test_eos_and_sampling(tiny):
    cfg, w = tiny
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, cfg.vocab_size, size=20).tolist()
    ref = eager_greedy(cfg, w, prompt, 6)
    eos = ref[2]
    llm = _llm(cfg, w, eos_token_ids=[eos])
    r = llm.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=6))[0]
    assert r.tokens == ref[: ref.index(eos) + 1]
    r = llm.generate([prompt], SamplingParams(temperature=0.9, top_k=50, top_p=0.9, max_new_tokens=5,
                                              ignore_eos=True))[0]
    assert len(r.tokens) == 5 and all(0 <= t < cfg.vocab_size for t in r.tokens)


def test_logprobs_follow_the_sampled_tokens():
    import math

    from modular_b200.entrypoints.llm import LLM
    from modular_b200.models.llama3 import Llama3Config
    from modular_b200.pipelines.context import SamplingParams, TextContext

    cfg = Llama3Config.tiny()
    llm = LLM(cfg, device="cpu", dtype=torch.float32, max_length=128, max_batch_size=4, max_batch_input_tokens=64,
              page_size=16, num_kv_pages=32)
    sp = SamplingParams(temperature=0.0, max_new_tokens=5, ignore_eos=True, logprobs=4)
    ctx = TextContext.from_prompt([5, 6, 7, 8, 9], 128, "lp", sp, ())
    llm.scheduler.add_request(ctx)
    plain = llm.add_request([5, 6, 7, 8, 9], SamplingParams(temperature=0.0, max_new_tokens=5, ignore_eos=True))
    while llm.has_unfinished():
        llm.step()
    ents = ctx.logprob_entries
    assert [e["token"] for e in ents] == [int(t) for t in ctx.tokens.generated]
    for e in ents:      # greedy: the sampled token is the most likely one; the alternatives are sorted
        assert e["top"][0][0] == e["token"] and abs(e["top"][0][1] - e["logprob"]) < 1e-6
        assert len(e["top"]) == 4 and all(a[1] >= b[1] for a, b in zip(e["top"], e["top"][1:]))
        assert e["logprob"] <= 0 and math.isfinite(e["logprob"])


def test_mistral_checkpoint_is_served_by_the_llama_family(tmp_path):
    """``MistralForCausalLM`` directories (same layers and tensor names as Llama) load through the registry and give
    the tokens of the same weights served as a Llama model; a sliding window caps the served context."""
    import json

    import pytest
    from safetensors.torch import save_file

    from modular_b200.models.llama3 import Llama3Config, Llama3Weights, MistralConfig
    from modular_b200.pipelines.config import PipelineArgs, PipelineConfig
    from modular_b200.pipelines.context import SamplingParams
    from modular_b200.pipelines.registry import PIPELINE_REGISTRY

    cfg = MistralConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, vocab_size=300, max_position_embeddings=512)
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=3, std=0.08)
    save_file({k: v.contiguous() for k, v in w.to_hf_state_dict(cfg).items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_hf()))

    def build(path):
        pc = PipelineConfig.from_args(PipelineArgs.from_flat_kwargs(
            None, model_path=str(path), devices="cpu", max_length=128, max_batch_size=2, max_batch_input_tokens=64,
            kv_cache_page_size=16, quantization_encoding="float32"))
        return PIPELINE_REGISTRY.retrieve(pc)[1]

    sp = SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True)
    llm = build(tmp_path)
    assert type(llm.cfg).__name__ == "MistralConfig"
    got = [list(r.tokens) for r in llm.generate([[5, 6, 7, 8], [9, 10]], sp)]
    from modular_b200.entrypoints.llm import LLM

    as_llama = Llama3Config(**{k: getattr(cfg, k) for k in Llama3Config.__dataclass_fields__ if k != "architectures"})
    ref = LLM(as_llama, w, device="cpu", dtype=torch.float32, max_length=128, max_batch_size=2,
              max_batch_input_tokens=64, page_size=16)
    assert got == [list(r.tokens) for r in ref.generate([[5, 6, 7, 8], [9, 10]], sp)]
    # a sliding window caps the served context at the window length (there the two attentions are the same)
    assert MistralConfig.from_hf(dict(cfg.to_hf(), sliding_window=64)).max_position_embeddings == 64


def test_checkpoints_with_parts_this_family_lacks_are_refused():
    """Nothing is dropped silently: another activation, MLP biases or an output-projection bias raise."""
    import pytest

    from modular_b200.models.llama3 import Llama3Config, Llama3Weights

    base = Llama3Config.tiny(num_hidden_layers=1, vocab_size=64).to_hf()
    with pytest.raises(ValueError):
        Llama3Config.from_hf(dict(base, hidden_act="gelu_pytorch_tanh"))
    with pytest.raises(ValueError):
        Llama3Config.from_hf(dict(base, mlp_bias=True))
    cfg = Llama3Config.tiny(num_hidden_layers=1, vocab_size=64)
    sd = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=0).to_hf_state_dict(cfg)
    Llama3Weights.from_state_dict(cfg, dict(sd, **{"model.layers.0.self_attn.o_proj.bias": torch.zeros(cfg.hidden_size)}),
                                  "cpu", torch.float32)          # an all-zero bias changes nothing
    with pytest.raises(ValueError):
        Llama3Weights.from_state_dict(cfg, dict(sd, **{"model.layers.0.self_attn.o_proj.bias": torch.ones(cfg.hidden_size)}),
                                      "cpu", torch.float32)


def test_logit_bias_forces_and_bans_tokens():
    """OpenAI ``logit_bias``: +100 on a token makes greedy decoding emit it, -100 on the greedy choice removes it;
    other requests of the same batch are untouched, and the map survives the worker transport."""
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.models.llama3 import Llama3Config
    from modular_b200.pipelines.context import SamplingParams

    cfg = Llama3Config.tiny(num_hidden_layers=2, vocab_size=64)
    llm = LLM(cfg, device="cpu", dtype=torch.float32, max_length=96, max_batch_size=4, max_batch_input_tokens=64,
              page_size=16, num_kv_pages=32, seed=2)
    prompt = [3, 4, 5, 6]
    plain = SamplingParams(temperature=0.0, max_new_tokens=5, ignore_eos=True)
    base = list(llm.generate([prompt], plain)[0].tokens)
    forced = SamplingParams(temperature=0.0, max_new_tokens=5, ignore_eos=True, logit_bias={"17": 100})
    banned = SamplingParams(temperature=0.0, max_new_tokens=5, ignore_eos=True, logit_bias={base[0]: -100.0})
    recs = llm.generate([prompt, prompt, prompt], [forced, banned, plain])
    assert list(recs[0].tokens) == [17] * 5
    assert recs[1].tokens[0] != base[0]
    assert list(recs[2].tokens) == base
    with pytest.raises(ValueError):
        SamplingParams(logit_bias={"x": 1.0})
    with pytest.raises(ValueError):
        SamplingParams(logit_bias={3: 1000.0})
    from modular_b200.serve.worker_interface.codec import decode, encode
    from modular_b200.pipelines.context import TextContext

    ctx = TextContext.from_prompt(prompt, 64, sampling_params=forced)
    back = decode(encode(ctx))
    assert back.sampling_params.logit_bias == {17: 100.0}
