"""GGUF: container round trip, block dequantisers against scalar restatements of the formats, and a
GGUF-stored tiny Llama that reproduces the original model's logits."""

import numpy as np
import pytest
import torch

from modular_b200.pipelines import gguf as G


def _f16(b):
    return float(np.frombuffer(bytes(b), dtype=np.float16)[0])


def _scalar_q4_k(block):
    d, dmin = _f16(block[0:2]), _f16(block[2:4])
    sc, qs = block[4:16], block[16:144]

    def scale_min(j):
        if j < 4:
            return sc[j] & 63, sc[j + 4] & 63
        return (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)

    y, q, is_ = [], 0, 0
    for _ in range(4):
        s1, m1 = scale_min(is_)
        s2, m2 = scale_min(is_ + 1)
        y += [d * s1 * (qs[q + l] & 0xF) - dmin * m1 for l in range(32)]
        y += [d * s2 * (qs[q + l] >> 4) - dmin * m2 for l in range(32)]
        q += 32
        is_ += 2
    return y


def _scalar_q6_k(block):
    ql, qh = block[0:128], block[128:192]
    sc = np.frombuffer(bytes(block[192:208]), dtype=np.int8)
    d = _f16(block[208:210])
    y = [0.0] * 256
    for half in range(2):
        L, H, S, Y = ql[64 * half:], qh[32 * half:], sc[8 * half:], 128 * half
        for l in range(32):
            i = l // 16
            q1 = ((L[l] & 0xF) | (((H[l] >> 0) & 3) << 4)) - 32
            q2 = ((L[l + 32] & 0xF) | (((H[l] >> 2) & 3) << 4)) - 32
            q3 = ((L[l] >> 4) | (((H[l] >> 4) & 3) << 4)) - 32
            q4 = ((L[l + 32] >> 4) | (((H[l] >> 6) & 3) << 4)) - 32
            y[Y + l] = d * S[i] * q1
            y[Y + l + 32] = d * S[i + 2] * q2
            y[Y + l + 64] = d * S[i + 4] * q3
            y[Y + l + 96] = d * S[i + 6] * q4
    return y


def test_k_quant_dequantisers_match_scalar_format_definitions():
    rng = np.random.default_rng(0)
    for t, scalar in ((G.GGML_Q4_K, _scalar_q4_k), (G.GGML_Q6_K, _scalar_q6_k)):
        per, size = G.BLOCK[t]
        raw = rng.integers(0, 256, size=(3, size), dtype=np.uint8)
        for b in raw:     # keep the fp16 scale fields finite
            for off in ((0, 2) if t == G.GGML_Q4_K else (208,)):
                b[off:off + 2] = np.frombuffer(np.float16(rng.uniform(0.01, 0.1)).tobytes(), dtype=np.uint8)
        got = G.dequantize(raw.reshape(-1), t, 3 * per)
        want = np.array([v for b in raw for v in scalar(b.tolist())], dtype=np.float32)
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6), t


def test_q8_q4_round_trip_error_bounds():
    x = np.random.default_rng(1).normal(size=(8, 64)).astype(np.float32)
    q8 = G.dequantize(np.frombuffer(G.quantize_q8_0(x), dtype=np.uint8), G.GGML_Q8_0, x.size).reshape(x.shape)
    q4 = G.dequantize(np.frombuffer(G.quantize_q4_0(x), dtype=np.uint8), G.GGML_Q4_0, x.size).reshape(x.shape)
    assert np.abs(q8 - x).max() < 0.02 and np.abs(q4 - x).max() < 0.35


def test_gguf_llama_checkpoint_reproduces_logits(tmp_path):
    from modular_b200.models.llama3 import Llama3Config, Llama3Model, Llama3Weights, adapt_hf_state_dict

    cfg = Llama3Config.tiny()
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=0, std=0.05)
    sd = w.to_hf_state_dict(cfg)
    inv = {v: k for k, v in G._TOP.items()}
    inv_layer = {v: k for k, v in G._LAYER.items()}
    tensors = {}
    for k, v in sd.items():
        if k in inv:
            name = inv[k]
        else:
            parts = k.split(".")        # model.layers.N.<module...>.weight
            name = f"blk.{parts[2]}.{inv_layer['.'.join(parts[3:-1])]}.{parts[-1]}"
        t = v.float()
        if k.endswith("q_proj.weight"):
            t = G._permute_qk(t, cfg.num_attention_heads)
        elif k.endswith("k_proj.weight"):
            t = G._permute_qk(t, cfg.num_key_value_heads)
        tensors[name] = (t.numpy(), G.GGML_F32 if t.ndim == 1 else G.GGML_F16)
    md = {"general.architecture": "llama", "llama.block_count": cfg.num_hidden_layers,
          "llama.embedding_length": cfg.hidden_size, "llama.attention.head_count": cfg.num_attention_heads,
          "llama.attention.head_count_kv": cfg.num_key_value_heads, "llama.feed_forward_length": cfg.intermediate_size,
          "llama.attention.layer_norm_rms_epsilon": cfg.rms_norm_eps, "llama.rope.freq_base": float(cfg.rope_theta),
          "llama.context_length": cfg.max_position_embeddings, "tokenizer.ggml.tokens": ["a", "b"]}
    path = str(tmp_path / "tiny.gguf")
    G.write_gguf(path, md, tensors)
    r = G.GGUFReader(path)
    hf = r.hf_config()
    assert hf["num_hidden_layers"] == cfg.num_hidden_layers and hf["num_key_value_heads"] == cfg.num_key_value_heads
    assert r.metadata["tokenizer.ggml.tokens"] == ["a", "b"]
    w2 = Llama3Weights.from_state_dict(cfg, adapt_hf_state_dict(r.to_hf_state_dict(torch.float32)), "cpu", torch.float32)
    T, page = 9, 16
    tok = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(0))
    i32 = lambda *a: torch.tensor(a, dtype=torch.int32)
    args = (tok, torch.arange(T, dtype=torch.int32), torch.arange(T) + page, i32([1, 0]), i32(0), i32(T), i32(T), i32(T - 1))
    kv = lambda: torch.zeros(3, 2, cfg.num_hidden_layers, cfg.num_key_value_heads, page, cfg.head_dim)
    a = Llama3Model(cfg, w, kv()).forward_tensors(*args)
    b = Llama3Model(cfg, w2, kv()).forward_tensors(*args)
    assert (a - b).abs().max() < 0.02 * a.abs().max()     # weights went through fp16


@pytest.mark.parametrize("arch", ["qwen2", "qwen3"])
def test_gguf_qwen_checkpoints_load_through_the_registry(tmp_path, arch):
    """qwen2 / qwen3 files: projection biases and per-head norm weights under the block names, Q / K rows in HF
    order; served through the registry from the .gguf alone, same greedy tokens as the source weights."""
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.models.llama3 import Llama3Weights, Qwen2Config, Qwen3Config
    from modular_b200.pipelines.config import PipelineArgs, PipelineConfig
    from modular_b200.pipelines.context import SamplingParams
    from modular_b200.pipelines.registry import PIPELINE_REGISTRY

    cfg = (Qwen2Config if arch == "qwen2" else Qwen3Config).tiny(tie_word_embeddings=False, vocab_size=512)
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=1, std=0.05)
    for l in w.layers:
        if l.q_norm is not None:
            l.q_norm.add_(torch.randn(l.q_norm.shape, generator=torch.Generator().manual_seed(2)) * 0.1)
            l.k_norm.add_(torch.randn(l.k_norm.shape, generator=torch.Generator().manual_seed(3)) * 0.1)
    inv = {v: k for k, v in G._TOP.items()}
    inv_layer = {v: k for k, v in G._LAYER.items()}
    tensors = {}
    for k, v in w.to_hf_state_dict(cfg).items():
        parts = k.split(".")
        name = inv[k] if k in inv else f"blk.{parts[2]}.{inv_layer['.'.join(parts[3:-1])]}.{parts[-1]}"
        tensors[name] = (v.float().numpy(), G.GGML_F32)
    md = {"general.architecture": arch, f"{arch}.block_count": cfg.num_hidden_layers,
          f"{arch}.embedding_length": cfg.hidden_size, f"{arch}.attention.head_count": cfg.num_attention_heads,
          f"{arch}.attention.head_count_kv": cfg.num_key_value_heads, f"{arch}.feed_forward_length": cfg.intermediate_size,
          f"{arch}.attention.layer_norm_rms_epsilon": cfg.rms_norm_eps, f"{arch}.rope.freq_base": float(cfg.rope_theta),
          f"{arch}.attention.key_length": cfg.head_dim, f"{arch}.context_length": 512}
    path = tmp_path / "m"
    path.mkdir()
    G.write_gguf(str(path / "tiny.gguf"), md, tensors)
    pc = PipelineConfig.from_args(PipelineArgs.from_flat_kwargs(
        None, model_path=str(path), devices="cpu", max_length=128, max_batch_size=2, max_batch_input_tokens=64,
        kv_cache_page_size=16, quantization_encoding="float32"))
    llm = PIPELINE_REGISTRY.retrieve(pc)[1]
    assert type(llm.cfg).__name__ == type(cfg).__name__
    assert (llm.weights.layers[0].qkv_bias is not None) == (arch == "qwen2")
    assert (llm.weights.layers[0].q_norm is not None) == (arch == "qwen3")
    sp = SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True)
    src = LLM(cfg, w, device="cpu", dtype=torch.float32, max_length=128, max_batch_size=2, max_batch_input_tokens=64,
              page_size=16)
    prompt = [5, 6, 7, 8, 9, 10]
    assert list(llm.generate([prompt], sp)[0].tokens) == list(src.generate([prompt], sp)[0].tokens)


def test_gguf_of_an_unknown_architecture_is_refused(tmp_path):
    G.write_gguf(str(tmp_path / "x.gguf"), {"general.architecture": "falcon"}, {})
    with pytest.raises(ValueError, match="falcon"):
        G.GGUFReader(str(tmp_path / "x.gguf")).hf_config()
