"""Layer library: thin stateful wrappers over :mod:`modular_b200.ops` for building models.

Layers hold plain tensors (no autograd) and run this package's kernels on CUDA and the PyTorch
reference ops on CPU. ``shard(rank, world)`` returns the tensor-parallel slice of a layer under
its ``ShardingStrategy``.

Reference: max/python/max/nn/linear.py (``Linear``, ``ColumnParallelLinear``, ``MLP`` :1037-1084),
nn/embedding.py:130 (``Embedding``, ``VocabParallelEmbedding``), nn/norm/rms_norm.py:30-90,
nn/norm/layer_norm.py, nn/attention/attention_with_rope.py:498-557, nn/transformer/transformer.py.
"""

from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import ops
from .rotary_embedding import RopeScaling, cos_sin_table


class ShardingStrategy(enum.Enum):
    REPLICATE = "replicate"
    ROWWISE = "rowwise"          # split the output features (weight rows): column-parallel linear
    COLUMNWISE = "columnwise"    # split the input features (weight columns): row-parallel linear, partial sums
    STACKED_QKV = "stacked_qkv"  # rows = [q heads | k heads | v heads], each split by heads
    GATE_UP = "gate_up"          # rows = [gate | up], each split


def _rand(shape, std, dtype, device, gen):
    return (torch.randn(*shape, generator=gen) * std).to(dtype).to(device)


class Linear:
    """``y = x @ W.T (+ b)``; W is [out, in] in bf16, fp8 with 128x128 block scales, or weight-only NVFP4 / MXFP8
    (``weight_format``; reference: max/python/max/nn/linear.py:44 with the float8 / float4 configs of
    nn/quant_config.py). NVFP4 / MXFP8 weights run on the decode-step GEMM up to 256 rows (tiles dequantised in
    shared memory) and are expanded to bf16 for larger inputs."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 weight_scale: Optional[torch.Tensor] = None,
                 strategy: ShardingStrategy = ShardingStrategy.REPLICATE, split_sizes: Sequence[int] = (),
                 weight_format: Optional[str] = None, block_scale: Optional[torch.Tensor] = None,
                 global_scale: Optional[torch.Tensor] = None):
        self.weight, self.bias, self.weight_scale = weight, bias, weight_scale
        self.strategy, self.split_sizes = strategy, tuple(split_sizes)
        self.weight_format, self.block_scale, self.global_scale = weight_format, block_scale, global_scale
        self._expanded = None

    @classmethod
    def random(cls, in_dim, out_dim, dtype=torch.bfloat16, device="cpu", bias=False, std=0.02, seed=0, **kw):
        g = torch.Generator().manual_seed(seed)
        return cls(_rand((out_dim, in_dim), std, dtype, device, g),
                   _rand((out_dim,), std, dtype, device, g) if bias else None, **kw)

    @property
    def in_dim(self):
        return self.weight.shape[1] * (2 if self.weight_format == "nvfp4" else 1)

    @property
    def out_dim(self):
        return self.weight.shape[0]

    def quantize_fp8(self) -> "Linear":
        q, s = ops.reference.quant_fp8_weight_block128(self.weight.float())
        return Linear(q, self.bias, s, self.strategy, self.split_sizes)

    def quantize_nvfp4(self) -> "Linear":
        q, bs, gs = ops.reference.quant_nvfp4_weight(self.weight.float())
        return Linear(q, self.bias, None, self.strategy, self.split_sizes, "nvfp4", bs, gs)

    def quantize_mxfp8(self) -> "Linear":
        q, bs = ops.reference.quant_mxfp8_weight(self.weight.float())
        return Linear(q, self.bias, None, self.strategy, self.split_sizes, "mxfp8", bs)

    def dequantized_weight(self) -> torch.Tensor:
        """bf16 weights of a quantised layer (cached: the form that steps of more than 256 rows multiply with)."""
        if self._expanded is None:
            if self.weight_format == "nvfp4":
                w = ops.reference.dequant_nvfp4_weight(self.weight, self.block_scale, self.global_scale)
            elif self.weight_format == "mxfp8":
                w = ops.reference.dequant_mxfp8_weight(self.weight, self.block_scale)
            else:
                w = ops.reference.dequant_fp8_weight_block128(self.weight, self.weight_scale)
            self._expanded = w.to(torch.bfloat16 if self.weight.is_cuda else torch.float32)
        return self._expanded

    def __call__(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if self.weight_format in ("nvfp4", "mxfp8"):
            n, k = self.out_dim, self.in_dim
            if (x2.is_cuda and x2.dtype == torch.bfloat16 and x2.shape[0] <= ops.DECODE_GEMM_MAX_TOKENS
                    and n % 128 == 0 and k % 128 == 0):
                y = ops.linear_decode(x2.contiguous(), self.weight, w_format=self.weight_format,
                                      w_block_scale=self.block_scale, w_global_scale=self.global_scale)
                if residual is not None:
                    y = y + residual
            else:
                w = self.dequantized_weight().to(x2.dtype)
                y = ops.linear(x2, w, residual=residual) if x2.is_cuda else ops.reference.linear(x2, w, residual)
        elif self.weight_scale is not None:
            if x2.is_cuda:
                y = ops.linear_fp8(x2, self.weight, self.weight_scale, residual=residual)
            else:
                w = ops.reference.dequant_fp8_weight_block128(self.weight, self.weight_scale).to(x2.dtype)
                y = ops.reference.linear(x2, w, residual)
        else:
            y = ops.linear(x2, self.weight, residual=residual)
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*shape[:-1], self.out_dim)

    def shard(self, rank: int, world: int) -> "Linear":
        w, b, st = self.weight, self.bias, self.strategy
        if self.weight_scale is not None and st is not ShardingStrategy.REPLICATE:
            raise NotImplementedError("shard fp8 layers before quantising")
        if st is ShardingStrategy.REPLICATE or world == 1:
            return self
        if st is ShardingStrategy.ROWWISE:
            n = w.shape[0] // world
            return Linear(w[rank * n:(rank + 1) * n].contiguous(), None if b is None else b[rank * n:(rank + 1) * n], None, st)
        if st is ShardingStrategy.COLUMNWISE:
            n = w.shape[1] // world
            # the bias is added once, by rank 0, because the partial sums are added across ranks
            return Linear(w[:, rank * n:(rank + 1) * n].contiguous(), b if rank == 0 else None, None, st)
        sizes = self.split_sizes or ((w.shape[0] // 2,) * 2 if st is ShardingStrategy.GATE_UP else ())
        if not sizes or sum(sizes) != w.shape[0]:
            raise ValueError("split_sizes must cover the weight rows")
        parts, bparts, r0 = [], [], 0
        for sz in sizes:
            n = sz // world
            parts.append(w[r0 + rank * n:r0 + (rank + 1) * n])
            if b is not None:
                bparts.append(b[r0 + rank * n:r0 + (rank + 1) * n])
            r0 += sz
        return Linear(torch.cat(parts).contiguous(), torch.cat(bparts) if bparts else None, None, st,
                      tuple(s // world for s in sizes))


class ColumnParallelLinear(Linear):
    """Rowwise-sharded linear whose outputs are gathered along the feature axis (LM head)."""

    def __init__(self, weight, bias=None, collectives=None, **kw):
        super().__init__(weight, bias, strategy=ShardingStrategy.ROWWISE, **kw)
        self.collectives = collectives

    def __call__(self, x, residual=None):
        y = super().__call__(x, residual)
        if self.collectives is None:
            return y
        gathered = self.collectives.all_gather(y.t().contiguous())   # [world * out_local, tokens]
        return gathered.t().contiguous()


class MLP:
    """SwiGLU MLP with gate and up fused into one GEMM whose epilogue applies ``silu(gate) * up``."""

    def __init__(self, gate_up: Linear, down: Linear):
        self.gate_up, self.down = gate_up, down

    @classmethod
    def random(cls, hidden, inter, dtype=torch.bfloat16, device="cpu", std=0.02, seed=0):
        return cls(Linear.random(hidden, 2 * inter, dtype, device, std=std, seed=seed, strategy=ShardingStrategy.GATE_UP),
                   Linear.random(inter, hidden, dtype, device, std=std, seed=seed + 1, strategy=ShardingStrategy.COLUMNWISE))

    def __call__(self, x, residual=None):
        x2 = x.reshape(-1, x.shape[-1])
        if self.gate_up.weight_scale is None and self.gate_up.bias is None:
            act = ops.linear_swiglu(x2, self.gate_up.weight)
        else:
            act = ops.silu_mul(self.gate_up(x2))
        return self.down(act, residual=residual).reshape(x.shape)

    def shard(self, rank, world):
        return MLP(self.gate_up.shard(rank, world), self.down.shard(rank, world))


class Embedding:
    def __init__(self, weight: torch.Tensor):
        self.weight = weight

    def __call__(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(ids.reshape(-1), self.weight).reshape(*ids.shape, self.weight.shape[1])


class VocabParallelEmbedding:
    """Rows [vocab_start, vocab_start + n) of the table; ids outside produce zeros, and the sum over
    ranks (an all-reduce by the caller or ``collectives``) restores the full lookup."""

    def __init__(self, weight_shard: torch.Tensor, vocab_start: int, collectives=None):
        self.weight, self.vocab_start, self.collectives = weight_shard, vocab_start, collectives

    @classmethod
    def from_full(cls, weight: torch.Tensor, rank: int, world: int, collectives=None):
        n = (weight.shape[0] + world - 1) // world
        return cls(weight[rank * n:(rank + 1) * n].contiguous(), rank * n, collectives)

    def __call__(self, ids):
        y = ops.embedding(ids.reshape(-1), self.weight, vocab_start=self.vocab_start)
        if self.collectives is not None:
            y = self.collectives.all_reduce(y)
        return y.reshape(*ids.shape, self.weight.shape[1])


class RMSNorm:
    """``multiply_before_cast`` selects the Gemma rounding order (scale in fp32, then cast); Llama casts the
    normalised value first. ``weight_offset`` = 1 for checkpoints that store ``w - 1``."""

    def __init__(self, weight, eps=1e-6, weight_offset=0.0, multiply_before_cast=False):
        self.weight, self.eps, self.weight_offset, self.mbc = weight, eps, weight_offset, multiply_before_cast

    def __call__(self, x, residual=None):
        x2 = x.reshape(-1, x.shape[-1])
        if residual is not None:   # residual += x (in place); returns norm(residual)
            return ops.add_rms_norm(x2, residual.reshape(-1, x.shape[-1]), self.weight, self.eps,
                                    self.weight_offset, self.mbc).reshape(x.shape)
        return ops.rms_norm(x2, self.weight, self.eps, self.weight_offset, self.mbc).reshape(x.shape)


class LayerNorm:
    def __init__(self, weight, bias=None, eps=1e-5):
        self.weight, self.bias, self.eps = weight, bias, eps

    def __call__(self, x):
        xf = x.float()
        mu = xf.mean(-1, keepdim=True)
        var = (xf - mu).pow(2).mean(-1, keepdim=True)
        y = (xf - mu) * torch.rsqrt(var + self.eps) * self.weight.float()
        if self.bias is not None:
            y = y + self.bias.float()
        return y.to(x.dtype)


@dataclass
class RaggedBatch:
    """Device-side description of one ragged step (see pipelines.batch.BatchPacker.tensors)."""
    positions: torch.Tensor
    slots: torch.Tensor
    block_table: torch.Tensor
    q_start: torch.Tensor
    q_len: torch.Tensor
    kv_len: torch.Tensor
    plan: Optional[object] = None


class AttentionWithRope:
    """Fused QKV projection -> RoPE on Q,K + K/V store into the paged cache -> ragged paged attention
    -> output projection."""

    def __init__(self, qkv: Linear, o: Linear, n_q: int, n_kv: int, head_dim: int, layer_idx: int,
                 cos_sin: torch.Tensor, scale: Optional[float] = None, interleaved: bool = False):
        self.qkv, self.o, self.n_q, self.n_kv, self.head_dim = qkv, o, n_q, n_kv, head_dim
        self.layer_idx, self.cos_sin, self.interleaved = layer_idx, cos_sin, interleaved
        self.scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)

    def __call__(self, x, kv_cache: torch.Tensor, b: RaggedBatch, residual=None):
        kc, vc = kv_cache[:, 0, self.layer_idx], kv_cache[:, 1, self.layer_idx]
        qkv = self.qkv(x)
        ops.rope_kv_store(qkv, b.positions, b.slots, self.cos_sin, kc, vc, self.n_q, self.n_kv, self.head_dim,
                          self.interleaved)
        a = ops.paged_attention(qkv, kc, vc, b.block_table, b.q_start, b.q_len, b.kv_len, self.n_q, self.n_kv,
                                self.head_dim, self.scale, plan=b.plan)
        return self.o(a, residual=residual)

    def shard(self, rank, world):
        return AttentionWithRope(self.qkv.shard(rank, world), self.o.shard(rank, world), self.n_q // world,
                                 self.n_kv // world, self.head_dim, self.layer_idx, self.cos_sin, self.scale,
                                 self.interleaved)


class TransformerBlock:
    def __init__(self, attn_norm: RMSNorm, attn: AttentionWithRope, mlp_norm: RMSNorm, mlp):
        self.attn_norm, self.attn, self.mlp_norm, self.mlp = attn_norm, attn, mlp_norm, mlp

    def __call__(self, h, kv_cache, b: RaggedBatch):
        h = self.attn(self.attn_norm(h), kv_cache, b, residual=h)
        return self.mlp(self.mlp_norm(h), residual=h)


class Transformer:
    """Embedding -> blocks -> final norm -> LM head on the requested rows (last-token logits)."""

    def __init__(self, embedding: Embedding, blocks: Sequence[TransformerBlock], norm: RMSNorm, lm_head: Linear,
                 logits_scale: float = 1.0, softcap: Optional[float] = None):
        self.embedding, self.blocks, self.norm, self.lm_head = embedding, list(blocks), norm, lm_head
        self.logits_scale, self.softcap = logits_scale, softcap

    def __call__(self, tokens, kv_cache, b: RaggedBatch, logit_rows):
        h = self.embedding(tokens)
        for blk in self.blocks:
            h = blk(h, kv_cache, b)
        last = self.norm(h[logit_rows.long()])
        logits = ops.linear(last, self.lm_head.weight, out_dtype=torch.float32).float() * self.logits_scale
        if self.softcap:
            logits = torch.tanh(logits / self.softcap) * self.softcap
        return logits

    @classmethod
    def from_llama_weights(cls, cfg, w, max_position: Optional[int] = None) -> "Transformer":
        """The same network as models.llama3.Llama3Model, assembled from layers."""
        cs = cos_sin_table(cfg.head_dim, max_position or cfg.max_position_embeddings, cfg.rope_theta,
                           RopeScaling.from_hf(cfg.rope_scaling), w.embed.device)
        blocks = []
        for i, l in enumerate(w.layers):
            qkv = Linear(l.wqkv, strategy=ShardingStrategy.STACKED_QKV, split_sizes=(cfg.q_dim, cfg.kv_dim, cfg.kv_dim))
            attn = AttentionWithRope(qkv, Linear(l.wo, strategy=ShardingStrategy.COLUMNWISE), cfg.num_attention_heads,
                                     cfg.num_key_value_heads, cfg.head_dim, i, cs, cfg.attention_multiplier or None)
            mlp = MLP(Linear(l.wgu, strategy=ShardingStrategy.GATE_UP), Linear(l.wd, strategy=ShardingStrategy.COLUMNWISE))
            blocks.append(TransformerBlock(RMSNorm(l.attn_norm, cfg.rms_norm_eps), attn,
                                           RMSNorm(l.mlp_norm, cfg.rms_norm_eps), mlp))
        return cls(Embedding(w.embed), blocks, RMSNorm(w.final_norm, cfg.rms_norm_eps), Linear(w.lm_head))
