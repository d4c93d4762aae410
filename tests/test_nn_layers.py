"""Layer library on CPU: the layer-built Transformer equals the Llama model, sharded linears recombine."""

import torch

from modular_b200.models.llama3 import Llama3Config, Llama3Model, Llama3Weights
from modular_b200.nn.layers import (MLP, LayerNorm, Linear, RaggedBatch, RMSNorm, ShardingStrategy, Transformer,
                                    VocabParallelEmbedding)


def test_transformer_from_layers_matches_llama_model():
    cfg = Llama3Config.tiny()
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=0, std=0.05)
    page, T = 16, 21
    kv1 = torch.zeros(4, 2, cfg.num_hidden_layers, cfg.num_key_value_heads, page, cfg.head_dim)
    kv2 = torch.zeros_like(kv1)
    tok = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(0))
    i32 = lambda *a: torch.tensor(a, dtype=torch.int32)
    b = RaggedBatch(torch.arange(T, dtype=torch.int32), torch.arange(T) + page, i32([1, 2, 0]), i32(0), i32(T), i32(T))
    rows = i32(T - 1, 3)
    want = Llama3Model(cfg, w, kv1).forward_tensors(tok, b.positions, b.slots, b.block_table, b.q_start, b.q_len,
                                                    b.kv_len, rows)
    got = Transformer.from_llama_weights(cfg, w)(tok, kv2, b, rows)
    assert torch.allclose(got, want, atol=1e-5)
    assert torch.equal(kv1, kv2)


def test_sharded_linears_recombine():
    x = torch.randn(5, 64)
    row = Linear.random(64, 96, torch.float32, bias=True, strategy=ShardingStrategy.ROWWISE, seed=1)
    col = Linear.random(64, 48, torch.float32, bias=True, strategy=ShardingStrategy.COLUMNWISE, seed=2)
    assert torch.allclose(torch.cat([row.shard(r, 4)(x) for r in range(4)], dim=-1), row(x), atol=1e-5)
    parts = [col.shard(r, 4)(x[:, r * 16:(r + 1) * 16]) for r in range(4)]
    assert torch.allclose(sum(parts), col(x), atol=1e-5)
    qkv = Linear.random(64, 32 + 16 + 16, torch.float32, strategy=ShardingStrategy.STACKED_QKV, split_sizes=(32, 16, 16), seed=3)
    full = qkv(x)
    for r in range(2):
        want = torch.cat([full[:, r * 16:(r + 1) * 16], full[:, 32 + r * 8:32 + (r + 1) * 8], full[:, 48 + r * 8:48 + (r + 1) * 8]], -1)
        assert torch.allclose(qkv.shard(r, 2)(x), want, atol=1e-5)
    mlp = MLP.random(64, 128, torch.float32, seed=4)
    inter = [mlp.shard(r, 2) for r in range(2)]
    assert torch.allclose(sum(m(x) for m in inter), mlp(x), atol=1e-4)


def test_norms_fp8_linear_and_vocab_parallel_embedding():
    x = torch.randn(3, 7, 32)
    w = torch.rand(32) + 0.5
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert torch.allclose(RMSNorm(w)(x), ref, atol=1e-5)
    assert torch.allclose(RMSNorm(w - 1, weight_offset=1.0, multiply_before_cast=True)(x), ref, atol=1e-5)
    ln = LayerNorm(w, torch.ones(32) * 0.1)
    assert torch.allclose(ln(x), torch.nn.functional.layer_norm(x, (32,), w, torch.ones(32) * 0.1), atol=1e-5)
    lin = Linear.random(256, 128, torch.float32, std=0.05, seed=5)
    q = lin.quantize_fp8()
    xx = torch.randn(4, 256)
    assert (q(xx) - lin(xx)).abs().max() < 0.06 * lin(xx).abs().max()
    table = torch.randn(50, 8)
    ids = torch.tensor([[0, 13, 49], [25, 24, 7]])
    shards = [VocabParallelEmbedding.from_full(table, r, 2) for r in range(2)]
    assert torch.equal(sum(s(ids) for s in shards), table[ids])


def test_linear_with_nvfp4_and_mxfp8_weights_and_their_quant_configs():
    """Weight-only 4-bit (NVFP4) and micro-scaled 8-bit (MXFP8) linear layers against their dequantised weights, and
    the checkpoint quantisation configs that name them."""
    import torch

    from modular_b200.nn.layers import Linear
    from modular_b200.ops import reference as ref
    from modular_b200.pipelines.weights import parse_quant_config

    lin = Linear.random(256, 128, dtype=torch.float32, std=0.05, seed=3)
    x = torch.randn(5, 256)
    full = lin(x)
    for q, tol in ((lin.quantize_nvfp4(), 0.2), (lin.quantize_mxfp8(), 0.06)):
        assert q.in_dim == 256 and q.out_dim == 128
        y = q(x)
        assert torch.allclose(y, x @ q.dequantized_weight().float().t(), atol=1e-4)
        assert (y - full).norm() / full.norm() < tol
    p, bs, gs = ref.quant_nvfp4_weight(lin.weight)
    assert p.dtype == torch.uint8 and p.shape == (128, 128) and bs.dtype == torch.float8_e4m3fn and bs.shape == (128, 16)
    # every dequantised value is a representable e2m1 magnitude times its block scale
    d = ref.dequant_nvfp4_weight(p, bs, gs).view(128, 16, 16) / (bs.float() * gs).clamp_min(1e-30).unsqueeze(-1)
    assert set(d.abs().unique().round(decimals=3).tolist()) <= {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0}
    qc = parse_quant_config({"quantization_config": {"quant_method": "modelopt", "quant_algo": "NVFP4"}})
    assert qc.format == "nvfp4" and qc.activation_group == 16
    assert parse_quant_config({"quantization_config": {"quant_method": "mxfp8"}}).format == "mxfp8"
