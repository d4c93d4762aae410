"""Golden check against Hugging Face transformers on CPU: a randomly initialised HF model is saved as a checkpoint
directory, served by this engine through the registry, and both must produce the same greedy tokens. Covers the Llama layer and its variants: Mistral (same tensors), Qwen2 (projection bias), Qwen3 (RMSNorm on
every query and key head), Phi-3 (projections fused
in the checkpoint), Mixtral and Qwen3-MoE (mixture-of-experts feed-forward), Granite (scalar multipliers folded into the weights), OLMo (LayerNorm without parameters, clamped projections) and OLMo 2 / 3 (norms on the block outputs and over the whole query / key projection)."""

import json

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _save(model, cfg_dict, path):
    from safetensors.torch import save_file

    sd = {k: v.detach().clone().contiguous() for k, v in model.state_dict().items()}
    if cfg_dict.get("tie_word_embeddings"):
        sd.pop("lm_head.weight", None)
    save_file(sd, str(path / "model.safetensors"))
    (path / "config.json").write_text(json.dumps(cfg_dict))


def _engine(path):
    from modular_b200.pipelines.config import PipelineArgs, PipelineConfig
    from modular_b200.pipelines.registry import PIPELINE_REGISTRY

    pc = PipelineConfig.from_args(PipelineArgs.from_flat_kwargs(
        None, model_path=str(path), devices="cpu", max_length=128, max_batch_size=2, max_batch_input_tokens=64,
        kv_cache_page_size=16, quantization_encoding="float32"))
    return PIPELINE_REGISTRY.retrieve(pc)[1]


def _assert_logits_close(llm, hf, prompt, tol=2e-3):
    """Logits of every prompt position against transformers (the engine's model on a private cache)."""
    from modular_b200.pipelines.speculative import _SeqCache

    ours = _SeqCache(llm.model, 64).step(prompt, all_logits=True).float().cpu()
    with torch.no_grad():
        want = hf(torch.tensor([prompt])).logits[0].float()
    err = (ours - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), err


CASES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", dict(rope_theta=500000.0, rms_norm_eps=1e-5)),
    "mistral": ("MistralConfig", "MistralForCausalLM", dict(rope_theta=1e6, rms_norm_eps=1e-5, sliding_window=None)),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", dict(rope_theta=1e6, rms_norm_eps=1e-6, use_sliding_window=False)),
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(rope_theta=1e6, rms_norm_eps=1e-6, use_sliding_window=False,
                                                      head_dim=32)),
    "mixtral": ("MixtralConfig", "MixtralForCausalLM", dict(rope_theta=1e6, rms_norm_eps=1e-5, sliding_window=None,
                                                            num_local_experts=4, num_experts_per_tok=2)),
    "qwen3_moe": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM", dict(rope_theta=1e6, rms_norm_eps=1e-6, head_dim=32,
                                                                num_experts=8, num_experts_per_tok=2,
                                                                moe_intermediate_size=48, norm_topk_prob=True,
                                                                mlp_only_layers=[0])),
    "granite": ("GraniteConfig", "GraniteForCausalLM", dict(rope_theta=10000.0, rms_norm_eps=1e-5,
                                                            embedding_multiplier=12.0, residual_multiplier=0.22,
                                                            attention_multiplier=0.0078125 * 16, logits_scaling=8.0)),
    "gemma3": ("Gemma3TextConfig", "Gemma3ForCausalLM", dict(rms_norm_eps=1e-6, head_dim=32, query_pre_attn_scalar=24,
                                                             sliding_window=256, num_hidden_layers=6, pad_token_id=0,
                                                             rope_parameters={
                                                                 "sliding_attention": {"rope_type": "default",
                                                                                       "rope_theta": 10000.0},
                                                                 "full_attention": {"rope_type": "linear", "factor": 4.0,
                                                                                    "rope_theta": 1000000.0}})),
    "olmo": ("OlmoConfig", "OlmoForCausalLM", dict(rope_theta=10000.0, clip_qkv=0.05, pad_token_id=0)),
    "olmo2": ("Olmo2Config", "Olmo2ForCausalLM", dict(rope_theta=500000.0, rms_norm_eps=1e-6, pad_token_id=0)),
    "olmo3": ("Olmo3Config", "Olmo3ForCausalLM", dict(rope_theta=500000.0, rms_norm_eps=1e-6, pad_token_id=0,
                                                      sliding_window=256)),
    "phi3": ("Phi3Config", "Phi3ForCausalLM", dict(rope_theta=10000.0, rms_norm_eps=1e-5, sliding_window=None,
                                                   pad_token_id=0)),
}


@pytest.mark.parametrize("family", sorted(CASES))
@pytest.mark.parametrize("tied", [False, True])
def test_greedy_tokens_match_transformers(tmp_path, family, tied):
    from modular_b200.pipelines.context import SamplingParams

    cfg_name, model_name, extra = CASES[family]
    torch.manual_seed(7)
    kw = dict(hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              vocab_size=320, max_position_embeddings=512, tie_word_embeddings=tied)
    kw.update(extra)
    hf_cfg = getattr(transformers, cfg_name)(**kw)
    hf = getattr(transformers, model_name)(hf_cfg).eval()
    with torch.no_grad():       # the default initialisation leaves biases at zero and norms at one: move them
        for n, p in hf.named_parameters():
            if n.endswith(".bias") or "layernorm" in n or n.endswith("norm.weight"):
                p.add_(torch.randn_like(p) * 0.1)
    d = hf_cfg.to_dict()
    d["architectures"] = [model_name]
    _save(hf, d, tmp_path)
    llm = _engine(tmp_path)
    assert (llm.weights.layers[0].qkv_bias is not None) == (family == "qwen2")
    assert (llm.weights.layers[-1].moe is not None) == (family in ("mixtral", "qwen3_moe"))
    prompts = [[5, 6, 7, 8, 9, 10, 11], [200, 3, 17]]
    n_new = 10
    recs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=n_new, ignore_eos=True))
    for prompt, rec in zip(prompts, recs):
        with torch.no_grad():
            want = hf.generate(torch.tensor([prompt]), max_new_tokens=n_new, do_sample=False, pad_token_id=0,
                               eos_token_id=None)[0, len(prompt):].tolist()
        assert list(rec.tokens) == want, (family, tied)
    _assert_logits_close(llm, hf, prompts[0])


@pytest.mark.parametrize("q_lora,yarn", [(96, False), (None, False), (96, True)])
def test_deepseek_v3_greedy_tokens_match_transformers(tmp_path, q_lora, yarn):
    """DeepSeek-V3 (multi-head latent attention in the absorbed form over the latent cache, interleaved rotary
    convention of the checkpoint, group-limited sigmoid routing with the correction bias, shared experts, a dense
    first layer): same greedy tokens as ``DeepseekV3ForCausalLM``. The expert weights arrive in the two-tensor layout
    transformers keeps in memory (``experts.gate_up_proj`` / ``experts.down_proj``)."""
    from modular_b200.pipelines.context import SamplingParams

    torch.manual_seed(11)
    hf_cfg = transformers.DeepseekV3Config(
        vocab_size=512, hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=3,
        num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8,
        routed_scaling_factor=2.5, kv_lora_rank=64, q_lora_rank=q_lora, qk_rope_head_dim=16, v_head_dim=32,
        qk_nope_head_dim=32, n_group=2, topk_group=1, num_experts_per_tok=2, first_k_dense_replace=1,
        norm_topk_prob=True, max_position_embeddings=512, rope_theta=10000.0,
        rope_scaling={"rope_type": "yarn", "type": "yarn", "factor": 40.0, "beta_fast": 32, "beta_slow": 1,
                      "mscale": 1.0, "mscale_all_dim": 1.0, "original_max_position_embeddings": 16} if yarn else None,
        tie_word_embeddings=False)
    hf = transformers.DeepseekV3ForCausalLM(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.add_(torch.randn_like(b) * 0.1)
    d = hf_cfg.to_dict()
    d["architectures"] = ["DeepseekV3ForCausalLM"]
    _save(hf, d, tmp_path)
    llm = _engine(tmp_path)
    prompts = [[5, 6, 7, 8, 9, 10, 11], [200, 3, 17], [41, 42, 43, 44, 45, 46, 47, 48, 49, 50, 51, 52]]
    recs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=10, ignore_eos=True))
    for prompt, rec in zip(prompts, recs):
        with torch.no_grad():
            want = hf.generate(torch.tensor([prompt]), max_new_tokens=10, do_sample=False, pad_token_id=0,
                               eos_token_id=None)[0, len(prompt):].tolist()
        assert list(rec.tokens) == want
    _assert_logits_close(llm, hf, prompts[2] * 3)      # 36 positions: past the original context of the yarn case


def test_phi3_longrope_matches_transformers(tmp_path):
    """Phi-3 128k variants: LongRoPE divides the rotary frequencies by per-frequency factors (short ones while the
    context fits the original length, long ones beyond) and scales cos / sin by an attention factor from the ratio
    of the two lengths. Both regimes against transformers, and the comparison is sensitive to the scaling."""
    from modular_b200.models.llama3 import Llama3Model
    from modular_b200.pipelines.speculative import _SeqCache

    torch.manual_seed(3)
    hd = 16
    rs = {"rope_type": "longrope", "type": "longrope", "short_factor": [1.0 + 0.05 * i for i in range(hd // 2)],
          "long_factor": [1.5 + 0.4 * i for i in range(hd // 2)]}
    hf_cfg = transformers.Phi3Config(
        hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        vocab_size=320, max_position_embeddings=96, original_max_position_embeddings=16, rope_scaling=rs,
        rope_theta=10000.0, sliding_window=None, pad_token_id=0, tie_word_embeddings=False)
    hf = transformers.Phi3ForCausalLM(hf_cfg).eval()
    d = hf_cfg.to_dict()
    d["architectures"] = ["Phi3ForCausalLM"]
    _save(hf, d, tmp_path)

    def engine(max_len):
        from modular_b200.pipelines.config import PipelineArgs, PipelineConfig
        from modular_b200.pipelines.registry import PIPELINE_REGISTRY

        pc = PipelineConfig.from_args(PipelineArgs.from_flat_kwargs(
            None, model_path=str(tmp_path), devices="cpu", max_length=max_len, max_batch_size=2,
            max_batch_input_tokens=64, kv_cache_page_size=16, quantization_encoding="float32"))
        return PIPELINE_REGISTRY.retrieve(pc)[1]

    for max_len, n in ((16, 12), (96, 40)):      # short factors / long factors
        llm = engine(max_len)
        assert llm.cfg.rope_scaling["rope_type"] == "longrope" and llm.cfg.rope_scaling["factor"] == 6.0
        prompt = [(7 * i + 3) % 320 for i in range(n)]
        ours = _SeqCache(llm.model, 64).step(prompt, all_logits=True).float()
        with torch.no_grad():
            want = hf(torch.tensor([prompt])).logits[0].float()
        assert (ours - want).abs().max().item() < 1e-5
    import copy

    plain = copy.copy(llm.cfg)
    plain.rope_scaling = None
    other = _SeqCache(Llama3Model(plain, llm.weights, llm.model.kv), 64).step(prompt, all_logits=True).float()
    assert (other - want).abs().max().item() > 1e-3


@pytest.mark.parametrize("scaling", [
    {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
     "original_max_position_embeddings": 32},
    {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 24, "beta_fast": 32, "beta_slow": 1},
    {"rope_type": "linear", "factor": 2.5},
])
def test_llama_rope_scaling_families_match_transformers(tmp_path, scaling):
    """The rotary scaling rules of Llama-3.1 (``llama3``), YaRN and linear interpolation: logits of a prompt that
    reaches past the original context, against transformers."""
    from modular_b200.pipelines.speculative import _SeqCache

    torch.manual_seed(5)
    hf_cfg = transformers.LlamaConfig(
        hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        vocab_size=320, max_position_embeddings=128, rope_theta=10000.0, rope_scaling=dict(scaling),
        tie_word_embeddings=False)
    hf = transformers.LlamaForCausalLM(hf_cfg).eval()
    d = hf_cfg.to_dict()
    d["architectures"] = ["LlamaForCausalLM"]
    _save(hf, d, tmp_path)
    llm = _engine(tmp_path)
    assert llm.cfg.rope_scaling["rope_type"] == scaling["rope_type"]
    prompt = [(11 * i + 5) % 320 for i in range(60)]
    ours = _SeqCache(llm.model, 64).step(prompt, all_logits=True).float()
    with torch.no_grad():
        want = hf(torch.tensor([prompt])).logits[0].float()
    assert (ours - want).abs().max().item() < 1e-5


@pytest.mark.parametrize("method", ["greedy", "group_limited_greedy"])
def test_deepseek_v2_matches_transformers(tmp_path, method):
    """DeepSeek-V2 shapes (``DeepseekV2ForCausalLM``): the V3 model code with a softmax router - plain top-k without
    renormalisation and no query low-rank projection (V2-Lite), or top-k inside the best groups with a scaling
    factor (V2) - and two shared experts."""
    from modular_b200.models.deepseek_v3 import DeepseekV3Config
    from modular_b200.pipelines.speculative import _SeqCache

    torch.manual_seed(13)
    hf_cfg = transformers.DeepseekV2Config(
        vocab_size=512, hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=3,
        num_attention_heads=4, num_key_value_heads=4, n_shared_experts=2, n_routed_experts=8,
        routed_scaling_factor=1.0 if method == "greedy" else 4.0, kv_lora_rank=64,
        q_lora_rank=None if method == "greedy" else 96, qk_rope_head_dim=16, v_head_dim=32,
        qk_nope_head_dim=32, topk_method=method, n_group=1 if method == "greedy" else 4,
        topk_group=1 if method == "greedy" else 2, num_experts_per_tok=3,
        first_k_dense_replace=1, norm_topk_prob=False, max_position_embeddings=512, rope_theta=10000.0,
        tie_word_embeddings=False)
    hf = transformers.DeepseekV2ForCausalLM(hf_cfg).eval()
    for mod in hf.modules():          # the group-limited branch of this transformers version reads an unset attribute
        if type(mod).__name__ == "DeepseekV2Moe" and not hasattr(mod, "num_experts"):
            mod.num_experts = hf_cfg.n_routed_experts
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
    d = hf_cfg.to_dict()
    d["architectures"] = ["DeepseekV2ForCausalLM"]
    _save(hf, d, tmp_path)
    llm = _engine(tmp_path)
    assert llm.cfg.scoring_func == "softmax" and not llm.cfg.norm_topk_prob
    assert llm.cfg.n_group == (1 if method == "greedy" else 4)
    prompt = [(7 * i + 3) % 512 for i in range(30)]
    ours = _SeqCache(llm.model, 64).step(prompt, all_logits=True).float()
    with torch.no_grad():
        want = hf(torch.tensor([prompt])).logits[0].float()
    assert (ours - want).abs().max().item() < 1e-5
    with pytest.raises(ValueError):
        DeepseekV3Config.from_hf(dict(d, topk_method="something_else"))


@pytest.mark.parametrize("pooling", ["last", "mean"])
def test_embeddings_match_transformers_hidden_states(tmp_path, pooling):
    """The embeddings path pools the final-normed hidden states: the same vectors as pooling transformers'
    ``last_hidden_state`` (prompts of different lengths in one ragged batch)."""
    torch.manual_seed(11)
    hf_cfg = transformers.Qwen2Config(
        hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        vocab_size=320, max_position_embeddings=512, rope_theta=1e6, rms_norm_eps=1e-6, use_sliding_window=False)
    hf = transformers.Qwen2ForCausalLM(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith(".bias") or n.endswith("norm.weight"):
                p.add_(torch.randn_like(p) * 0.1)
    d = hf_cfg.to_dict()
    d["architectures"] = ["Qwen2ForCausalLM"]
    _save(hf, d, tmp_path)
    llm = _engine(tmp_path)
    prompts = [[5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22], [200, 3, 17], [9]]
    ours = llm.encode(prompts, pooling=pooling).cpu()
    for i, p in enumerate(prompts):
        with torch.no_grad():
            hs = hf.model(torch.tensor([p])).last_hidden_state[0].float()
        want = hs[-1] if pooling == "last" else hs.mean(0)
        want = want / want.norm()
        assert (ours[i] - want).abs().max().item() < 2e-4, (pooling, i)


def _mamba_checkpoint(tmp_path, **kw):
    torch.manual_seed(5)
    hf_cfg = transformers.MambaConfig(hidden_size=64, state_size=16, num_hidden_layers=2, vocab_size=320, expand=2,
                                      conv_kernel=4, tie_word_embeddings=True, pad_token_id=0, bos_token_id=0,
                                      eos_token_id=0, **kw)
    hf = transformers.MambaForCausalLM(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("norm.weight") or n.endswith("norm_f.weight") or n.endswith("conv1d.bias"):
                p.add_(torch.randn_like(p) * 0.1)
    d = hf_cfg.to_dict()
    d["architectures"] = ["MambaForCausalLM"]
    _save(hf, d, tmp_path)
    return hf


def test_mamba_matches_transformers(tmp_path):
    """State-space family: greedy tokens of two requests of different lengths served together (prefill, then
    single-token steps on the recurrent state) against transformers' own recurrence."""
    from modular_b200.pipelines.context import SamplingParams

    hf = _mamba_checkpoint(tmp_path)
    llm = _engine(tmp_path)
    assert type(llm.model).__name__ == "MambaModel"
    prompts = [[5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15], [200, 3, 17]]
    n_new = 12
    recs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=n_new, ignore_eos=True))
    for prompt, rec in zip(prompts, recs):
        with torch.no_grad():
            want = hf.generate(torch.tensor([prompt]), max_new_tokens=n_new, do_sample=False)[0, len(prompt):].tolist()
        assert list(rec.tokens) == want


def test_mamba_chunked_prefill_and_slot_reuse_keep_the_state_right(tmp_path):
    """A prompt longer than the step budget is prefilled in chunks (the state carries over between steps), and with
    no more state slots than requests a slot is handed from a finished request to a new one, which must start from
    a zero state: tokens stay those of one-request runs."""
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.pipelines.context import SamplingParams
    from modular_b200.models.mamba import MambaConfig, MambaWeights

    cfg = MambaConfig.tiny(hidden_size=64, vocab_size=320)
    w = MambaWeights.random_init(cfg, "cpu", torch.float32, seed=3, std=0.05)
    import numpy as np
    rng = np.random.default_rng(0)
    prompts = [rng.integers(1, 320, size=n).tolist() for n in (70, 9, 33, 21)]
    sp = SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True)
    solo = []
    for p in prompts:
        one = LLM(cfg, w, device="cpu", dtype=torch.float32, max_length=256, max_batch_size=1,
                  max_batch_input_tokens=256)
        solo.append(list(one.generate([p], sp)[0].tokens))
    llm = LLM(cfg, w, device="cpu", dtype=torch.float32, max_length=256, max_batch_size=4, max_batch_input_tokens=32,
              num_kv_pages=3)
    got = [list(r.tokens) for r in llm.generate(prompts, sp)]
    assert got == solo
    # round trip through the checkpoint layout
    w2 = MambaWeights.from_state_dict(cfg, w.to_hf_state_dict(cfg), "cpu", torch.float32)
    again = LLM(cfg, w2, device="cpu", dtype=torch.float32, max_length=256, max_batch_size=4,
                max_batch_input_tokens=256)
    assert [list(r.tokens) for r in again.generate(prompts, sp)] == solo


@pytest.mark.parametrize("kind", ["bert", "mpnet"])
def test_encoder_embeddings_match_transformers(tmp_path, kind):
    """Encoder-only embedding models: pooled final hidden states against transformers (MPNet: relative-position
    biases over distances beyond the exact buckets, positions counted from the padding index)."""
    torch.manual_seed(3)
    common = dict(vocab_size=320, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                  max_position_embeddings=128)
    if kind == "bert":
        hf_cfg = transformers.BertConfig(**common)
        hf = transformers.BertModel(hf_cfg, add_pooling_layer=False).eval()
        arch = "BertModel"
    else:
        hf_cfg = transformers.MPNetConfig(**common)
        hf = transformers.MPNetModel(hf_cfg, add_pooling_layer=False).eval()
        arch = "MPNetForMaskedLM"
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith(".bias") or "LayerNorm" in n or "relative_attention_bias" in n:
                p.add_(torch.randn_like(p) * 0.1)
    d = hf_cfg.to_dict()
    d["architectures"] = [arch]
    _save(hf, d, tmp_path)
    llm = _engine(tmp_path)
    assert type(llm.model).__name__ == "BertModel"
    prompts = [list(range(5, 75)), [200, 3, 17], [9, 8]]
    for pooling in ("default", "cls", "last"):
        ours = llm.encode(prompts, pooling=pooling).cpu()
        for i, p in enumerate(prompts):
            with torch.no_grad():
                hs = hf(torch.tensor([p])).last_hidden_state[0].float()
            want = hs.mean(0) if pooling == "default" else hs[0] if pooling == "cls" else hs[-1]
            want = want / want.norm()
            assert (ours[i] - want).abs().max().item() < 2e-4, (kind, pooling, i)
    with pytest.raises(NotImplementedError):
        from modular_b200.pipelines.context import SamplingParams
        llm.generate([[1, 2, 3]], SamplingParams(max_new_tokens=2))


def test_gemma3_vision_language_checkpoint_serves_its_language_model(tmp_path):
    """``Gemma3ForConditionalGeneration``: settings nested under ``text_config``, tensors under a ``language_model``
    wrapper next to a vision tower; the language model is served for text and matches the text-only model."""
    from modular_b200.pipelines.context import SamplingParams

    torch.manual_seed(2)
    text = transformers.Gemma3TextConfig(hidden_size=64, intermediate_size=176, num_hidden_layers=6, num_attention_heads=4,
                                         num_key_value_heads=2, head_dim=32, vocab_size=320, sliding_window=256,
                                         query_pre_attn_scalar=24, max_position_embeddings=512, pad_token_id=0)
    hf = transformers.Gemma3ForCausalLM(text).eval()
    sd = {k.replace("model.", "model.language_model.", 1): v.detach().clone() for k, v in hf.state_dict().items()
          if k != "lm_head.weight"}
    sd["model.vision_tower.vision_model.embeddings.position_embedding.weight"] = torch.zeros(4, 8)
    sd["model.multi_modal_projector.mm_input_projection_weight"] = torch.zeros(8, 64)
    from safetensors.torch import save_file
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({
        "architectures": ["Gemma3ForConditionalGeneration"], "model_type": "gemma3", "text_config": text.to_dict(),
        "vision_config": {"model_type": "siglip_vision_model", "hidden_size": 8}}))
    llm = _engine(tmp_path)
    prompt = [5, 6, 7, 8, 9, 10, 11]
    rec = llm.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True))[0]
    with torch.no_grad():
        want = hf.generate(torch.tensor([prompt]), max_new_tokens=8, do_sample=False, pad_token_id=0,
                           eos_token_id=None)[0, len(prompt):].tolist()
    assert list(rec.tokens) == want


@pytest.mark.parametrize("layout", ["mistral3", "idefics3"])
def test_vision_language_checkpoint_around_mistral_serves_its_language_model(tmp_path, layout):
    """``Mistral3ForConditionalGeneration`` in the ``language_model.model.*`` layout with an untied head, and the
    ``model.text_model.*`` layout of ``Idefics3ForConditionalGeneration``: the vision tower and projector are dropped,
    the language model matches ``MistralForCausalLM``."""
    from modular_b200.pipelines.context import SamplingParams
    from safetensors.torch import save_file

    torch.manual_seed(4)
    text = transformers.MistralConfig(hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
                                      num_key_value_heads=2, vocab_size=320, max_position_embeddings=512,
                                      sliding_window=None, tie_word_embeddings=False)
    hf = transformers.MistralForCausalLM(text).eval()
    if layout == "mistral3":
        sd = {"language_model." + k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()}
        sd["vision_tower.transformer.layers.0.attention.q_proj.weight"] = torch.zeros(8, 8)
        sd["multi_modal_projector.linear_1.weight"] = torch.zeros(64, 8)
    else:
        sd = {k.replace("model.", "model.text_model.", 1): v.detach().clone().contiguous()
              for k, v in hf.state_dict().items()}
        sd["model.vision_model.embeddings.patch_embedding.weight"] = torch.zeros(8, 8)
        sd["model.connector.modality_projection.proj.weight"] = torch.zeros(64, 8)
    save_file(sd, str(tmp_path / "model.safetensors"))
    arch = "Mistral3ForConditionalGeneration" if layout == "mistral3" else "Idefics3ForConditionalGeneration"
    (tmp_path / "config.json").write_text(json.dumps({
        "architectures": [arch], "model_type": layout, "text_config": text.to_dict(),
        "vision_config": {"model_type": "pixtral", "hidden_size": 8}}))
    llm = _engine(tmp_path)
    prompt = [5, 6, 7, 8, 9, 10, 11]
    rec = llm.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True))[0]
    with torch.no_grad():
        want = hf.generate(torch.tensor([prompt]), max_new_tokens=8, do_sample=False, pad_token_id=0,
                           eos_token_id=None)[0, len(prompt):].tolist()
    assert list(rec.tokens) == want
    _assert_logits_close(llm, hf, prompt)


def test_lfm2_hybrid_matches_transformers(tmp_path):
    """Hybrid of gated short convolutions and attention layers: greedy tokens of two requests served together and
    the logits of every prompt position; then a long prompt prefilled in chunks with few state slots."""
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.pipelines.context import SamplingParams

    torch.manual_seed(9)
    hf_cfg = transformers.Lfm2Config(hidden_size=64, intermediate_size=176, num_hidden_layers=4, num_attention_heads=4,
                                     num_key_value_heads=2, vocab_size=320, conv_L_cache=3, block_multiple_of=16,
                                     block_auto_adjust_ff_dim=True, max_position_embeddings=512,
                                     layer_types=["conv", "conv", "full_attention", "conv"], pad_token_id=0)
    hf = transformers.Lfm2ForCausalLM(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("norm.weight"):
                p.add_(torch.randn_like(p) * 0.1)
    d = hf_cfg.to_dict()
    d["architectures"] = ["Lfm2ForCausalLM"]
    _save(hf, d, tmp_path)
    llm = _engine(tmp_path)
    assert type(llm.model).__name__ == "Lfm2Model" and llm.kv.kv.shape[2] == 1      # one KV plane: one attention layer
    prompts = [[5, 6, 7, 8, 9, 10, 11, 12, 13], [200, 3, 17]]
    sp = SamplingParams(temperature=0.0, max_new_tokens=10, ignore_eos=True)
    want = []
    for prompt in prompts:
        with torch.no_grad():
            want.append(hf.generate(torch.tensor([prompt]), max_new_tokens=10, do_sample=False, pad_token_id=0,
                                    eos_token_id=None)[0, len(prompt):].tolist())
    assert [list(r.tokens) for r in llm.generate(prompts, sp)] == want
    # chunked prefill (the convolution tail crosses step boundaries) and slot reuse
    long = [(7 * i) % 300 + 1 for i in range(50)]
    with torch.no_grad():
        want_long = hf.generate(torch.tensor([long]), max_new_tokens=6, do_sample=False, pad_token_id=0,
                                eos_token_id=None)[0, len(long):].tolist()
    small = LLM(llm.cfg, llm.weights, device="cpu", dtype=torch.float32, max_length=128, max_batch_size=2,
                max_batch_input_tokens=16, page_size=16, num_kv_pages=12)
    sp6 = SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True)
    got = small.generate([long, prompts[1], prompts[0]], sp6)
    assert list(got[0].tokens) == want_long and list(got[1].tokens) == want[1][:6] and list(got[2].tokens) == want[0][:6]


def test_qwen2_5_vl_checkpoint_serves_text_like_transformers(tmp_path):
    """A real (tiny) ``Qwen2_5_VLForConditionalGeneration``: vision tower beside the language model, multimodal
    rotary sections in the config. Text-only requests give transformers' tokens."""
    from modular_b200.pipelines.context import SamplingParams

    torch.manual_seed(0)
    cfg = transformers.Qwen2_5_VLConfig(
        text_config=dict(hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, vocab_size=320, max_position_embeddings=512, rope_theta=1e6,
                         rms_norm_eps=1e-6, use_sliding_window=False, tie_word_embeddings=False,
                         rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}),
        vision_config=dict(depth=1, hidden_size=32, intermediate_size=64, num_heads=2, out_hidden_size=64, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, fullatt_block_indexes=[0], window_size=28),
        image_token_id=300, video_token_id=301, vision_start_token_id=302, vision_end_token_id=303)
    hf = transformers.Qwen2_5_VLForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "language_model" in n and (n.endswith(".bias") or n.endswith("norm.weight")):
                p.add_(torch.randn_like(p) * 0.1)
    d = cfg.to_dict()
    d["architectures"] = ["Qwen2_5_VLForConditionalGeneration"]
    _save(hf, d, tmp_path)
    llm = _engine(tmp_path)
    assert llm.weights.layers[0].qkv_bias is not None
    for prompt in ([5, 6, 7, 8, 9, 10, 11], [200, 3, 17]):
        rec = llm.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True))[0]
        with torch.no_grad():
            want = hf.generate(torch.tensor([prompt]), max_new_tokens=8, do_sample=False, pad_token_id=0,
                               eos_token_id=None)[0, len(prompt):].tolist()
        assert list(rec.tokens) == want


def test_qwen3_vl_checkpoint_serves_text_like_transformers(tmp_path):
    """A tiny ``Qwen3VLForConditionalGeneration`` (interleaved multimodal rotary sections, per-head q/k norms):
    text-only requests give transformers' tokens."""
    from modular_b200.pipelines.context import SamplingParams

    torch.manual_seed(0)
    cfg = transformers.Qwen3VLConfig(
        text_config=dict(hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, vocab_size=320, max_position_embeddings=512, rope_theta=1e6,
                         rms_norm_eps=1e-6, tie_word_embeddings=False,
                         rope_scaling={"rope_type": "default", "mrope_section": [4, 6, 6], "mrope_interleaved": True}),
        vision_config=dict(depth=1, hidden_size=32, intermediate_size=64, num_heads=2, out_hidden_size=64, patch_size=16,
                           spatial_merge_size=2, temporal_patch_size=2, deepstack_visual_indexes=[0],
                           num_position_embeddings=16),
        image_token_id=300, video_token_id=301, vision_start_token_id=302, vision_end_token_id=303)
    hf = transformers.Qwen3VLForConditionalGeneration(cfg).eval()
    d = cfg.to_dict()
    d["architectures"] = ["Qwen3VLForConditionalGeneration"]
    _save(hf, d, tmp_path)
    llm = _engine(tmp_path)
    assert llm.weights.layers[0].q_norm is not None
    prompt = [5, 6, 7, 8, 9, 10, 11]
    rec = llm.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True))[0]
    with torch.no_grad():
        want = hf.generate(torch.tensor([prompt]), max_new_tokens=8, do_sample=False, pad_token_id=0,
                           eos_token_id=None)[0, len(prompt):].tolist()
    assert list(rec.tokens) == want
