"""Golden check against Hugging Face transformers on CPU: a randomly initialised HF model is saved as a checkpoint
directory, served by this engine through the registry, and both must produce the same greedy tokens. Covers the Llama layer and its variants: Mistral (same tensors), Qwen2 (projection bias), Qwen3 (RMSNorm on
every query and key head), Phi-3 (projections fused
in the checkpoint)."""

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


CASES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", dict(rope_theta=500000.0, rms_norm_eps=1e-5)),
    "mistral": ("MistralConfig", "MistralForCausalLM", dict(rope_theta=1e6, rms_norm_eps=1e-5, sliding_window=None)),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", dict(rope_theta=1e6, rms_norm_eps=1e-6, use_sliding_window=False)),
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(rope_theta=1e6, rms_norm_eps=1e-6, use_sliding_window=False,
                                                      head_dim=32)),
    "phi3": ("Phi3Config", "Phi3ForCausalLM", dict(rope_theta=10000.0, rms_norm_eps=1e-5, sliding_window=None,
                                                   pad_token_id=0)),
}


@pytest.mark.parametrize("family", sorted(CASES))
@pytest.mark.parametrize("tied", [False, True])
def test_greedy_tokens_match_transformers(tmp_path, family, tied):
    from modular_b200.pipelines.context import SamplingParams

    cfg_name, model_name, extra = CASES[family]
    torch.manual_seed(7)
    hf_cfg = getattr(transformers, cfg_name)(
        hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        vocab_size=320, max_position_embeddings=512, tie_word_embeddings=tied, **extra)
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
    prompts = [[5, 6, 7, 8, 9, 10, 11], [200, 3, 17]]
    n_new = 10
    recs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=n_new, ignore_eos=True))
    for prompt, rec in zip(prompts, recs):
        with torch.no_grad():
            want = hf.generate(torch.tensor([prompt]), max_new_tokens=n_new, do_sample=False, pad_token_id=0,
                               eos_token_id=None)[0, len(prompt):].tolist()
        assert list(rec.tokens) == want, (family, tied)
