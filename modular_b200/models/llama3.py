"""Llama-3 family decoder (GQA attention, SwiGLU MLP, RMSNorm, RoPE) over a paged KV cache.

The model owns *fused* weights (``wqkv`` = [q; k; v] rows, ``wgu`` = [gate; up] rows) built
from an HF-layout state dict by :func:`adapt_hf_state_dict`, and runs one ragged batch
(``StepBatch``) per call:

* on CUDA the whole stack is issued by the native ``DecoderExecutor`` (one host call per
  step: embedding, per layer RMSNorm -> QKV GEMM -> RoPE + KV store -> paged attention ->
  O GEMM (+residual) -> RMSNorm -> gate/up GEMM with SwiGLU epilogue -> down GEMM
  (+residual), final norm, LM head on the requested rows);
* on CPU the same sequence runs op by op through the PyTorch reference ops in fp32/bf16.

Reference counterparts: max/python/max/pipelines/architectures/llama3/llama3.py:73,
model_config.py, weight_adapters.py:33; layer wiring max/python/max/nn/attention/
attention_with_rope.py:498-557 and nn/linear.py:1037-1084.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from .._native import lib as _lib
from ..nn.rotary_embedding import RopeScaling, cos_sin_table


@dataclass
class Llama3Config:
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: Optional[int] = None
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: Optional[dict] = None
    max_position_embeddings: int = 131072
    tie_word_embeddings: bool = False
    attention_multiplier: Optional[float] = None
    logits_scaling: float = 1.0       # Granite: logits are divided by it (folded into the LM head at load)
    embedding_multiplier: float = 1.0 # Granite: folded into the embedding table at load
    residual_multiplier: float = 1.0  # Granite: scale of every block output, folded into the o / down projections
    attention_bias: bool = False      # bias on the query / key / value projections (Qwen2)
    qk_norm: bool = False             # RMSNorm over head_dim on every query and key head before the rotation (Qwen3)
    qk_norm_full: bool = False        # with qk_norm: one RMSNorm over the whole query / key projection (OLMo 2)
    norm_after: bool = False          # norms on the block outputs (before the residual add) instead of the inputs (OLMo 2)
    sandwich_norm: bool = False       # Gemma 3: norms on block inputs AND outputs, weights stored as (w - 1), gelu-tanh MLP
    rope_local_theta: Optional[float] = None   # Gemma 3: rotary base of the sliding-window layers (no scaling there)
    local_layers: tuple = ()          # Gemma 3: indices of the sliding-window layers
    plain_layer_norm: bool = False    # LayerNorm without weight or bias (eps 1e-5) in place of every RMSNorm (OLMo)
    clip_qkv: Optional[float] = None  # queries, keys and values clamped to [-clip, clip] after the projection (OLMo)
    # mixture-of-experts feed-forward (Mixtral, Qwen3-MoE): 0 experts = dense SwiGLU MLP in every layer
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    decoder_sparse_step: int = 1
    mlp_only_layers: tuple = ()
    architectures: tuple = ("LlamaForCausalLM",)

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads

    @classmethod
    def from_hf(cls, d: dict) -> "Llama3Config":
        from ..pipelines.weights import normalize_hf_rope

        if isinstance(d.get("text_config"), dict) and "hidden_size" not in d:
            # a vision-language checkpoint nests the language model's settings; that model is what is served
            d = dict(d["text_config"], architectures=d.get("architectures", ()))
        d = normalize_hf_rope(d)
        rs = d.get("rope_scaling")
        if isinstance(rs, dict) and (rs.get("rope_type") or rs.get("type")) in ("mrope", "default"):
            # multimodal rotary sections: with text alone the three position streams coincide and the rotation is
            # the plain one
            d = dict(d, rope_scaling=None)
        act = d.get("hidden_act") or d.get("hidden_activation") or "silu"
        if act not in ("silu", "swish"):
            raise ValueError(f"activation {act!r} is not implemented by this family (SwiGLU layers only)")
        if d.get("mlp_bias"):
            raise ValueError("biases on the MLP projections are not implemented")
        keys = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in d.items() if k in keys}
        if "architectures" in kw:
            kw["architectures"] = tuple(kw["architectures"])
        if "mlp_only_layers" in kw:
            kw["mlp_only_layers"] = tuple(kw["mlp_only_layers"] or ())
        return cls(**kw)

    def to_hf(self) -> dict:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d["architectures"] = list(self.architectures)
        d["mlp_only_layers"] = list(self.mlp_only_layers)
        d["model_type"] = "llama"
        return d

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def is_moe_layer(self, i: int) -> bool:
        return (self.num_experts > 0 and i not in self.mlp_only_layers
                and (i + 1) % max(1, self.decoder_sparse_step) == 0)

    def moe_config(self):
        from ..nn.moe import MoEConfig

        return MoEConfig(self.hidden_size, self.moe_intermediate_size or self.intermediate_size, self.num_experts,
                         self.num_experts_per_tok, norm_topk_prob=self.norm_topk_prob, scoring_func="softmax")

    def param_count(self) -> int:
        attn = self.hidden_size * (self.q_dim + 2 * self.kv_dim) + self.q_dim * self.hidden_size + 2 * self.hidden_size
        dense = 3 * self.hidden_size * self.intermediate_size
        moe = self.num_experts * (3 * self.hidden_size * (self.moe_intermediate_size or self.intermediate_size)
                                  + self.hidden_size)
        n_moe = sum(self.is_moe_layer(i) for i in range(self.num_hidden_layers))
        emb = self.vocab_size * self.hidden_size
        return (self.num_hidden_layers * attn + n_moe * moe + (self.num_hidden_layers - n_moe) * dense
                + emb * (1 if self.tie_word_embeddings else 2) + self.hidden_size)

    # named presets used by benchmarks and tests
    @classmethod
    def llama31_8b(cls) -> "Llama3Config":
        return cls(rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                 "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})

    @classmethod
    def llama33_70b(cls) -> "Llama3Config":
        return cls(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                   num_attention_heads=64, num_key_value_heads=8,
                   rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                 "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})

    @classmethod
    def tiny(cls, **overrides) -> "Llama3Config":
        base = dict(hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=64, vocab_size=4096, rms_norm_eps=1e-5,
                    rope_theta=500000.0, max_position_embeddings=2048, tie_word_embeddings=True)
        base.update(overrides)
        return cls(**base)


def _cap_to_window(cfg, window):
    """Sliding-window attention equals full attention while the sequence is no longer than the window: serve such
    checkpoints with the context capped there instead of refusing them."""
    if window is not None and int(window) > 0:
        cfg.max_position_embeddings = min(cfg.max_position_embeddings, int(window))
    return cfg


@dataclass
class MistralConfig(Llama3Config):
    """Mistral checkpoints (``MistralForCausalLM``) share the Llama layer structure and tensor names. Every layer
    here attends to the whole prefix, so a checkpoint with a sliding attention window is served up to the window
    length (where the two are the same function). Reference: max/python/max/pipelines/architectures/mistral/."""

    rope_theta: float = 1000000.0
    max_position_embeddings: int = 32768
    architectures: tuple = ("MistralForCausalLM",)

    @classmethod
    def from_hf(cls, d: dict) -> "MistralConfig":
        return _cap_to_window(super().from_hf(d), (d.get("text_config") or d).get("sliding_window"))

    def to_hf(self) -> dict:
        d = super().to_hf()
        d["model_type"] = "mistral"
        d["sliding_window"] = None
        return d


@dataclass
class Qwen2Config(Llama3Config):
    """Qwen2 / Qwen2.5 (``Qwen2ForCausalLM``): the Llama layer with a bias on the query, key and value projections.
    Checkpoints that switch sliding-window attention on are refused.
    Reference: max/python/max/pipelines/architectures/qwen2/."""

    rope_theta: float = 1000000.0
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 32768
    attention_bias: bool = True
    architectures: tuple = ("Qwen2ForCausalLM",)

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen2Config":
        if d.get("use_sliding_window"):
            raise ValueError("sliding-window attention is not implemented")
        cfg = super().from_hf(d)
        cfg.attention_bias = True          # HF's Qwen2 layers always carry the bias; the key is not in its config
        return cfg

    @classmethod
    def tiny(cls, **kw) -> "Qwen2Config":
        base = dict(hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, vocab_size=4096, tie_word_embeddings=True, max_position_embeddings=2048)
        base.update(kw)
        return cls(**base)

    def to_hf(self) -> dict:
        d = super().to_hf()
        d["model_type"] = "qwen2"
        d["use_sliding_window"] = False
        return d


@dataclass
class Qwen3Config(Llama3Config):
    """Qwen3 dense models (``Qwen3ForCausalLM``): the Llama layer with an RMSNorm over ``head_dim`` on every query
    and key head between the projection and the rotary embedding, and an explicit ``head_dim``.
    Reference: max/python/max/pipelines/architectures/qwen3/."""

    rope_theta: float = 1000000.0
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 40960
    qk_norm: bool = True
    architectures: tuple = ("Qwen3ForCausalLM",)

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen3Config":
        if d.get("use_sliding_window"):
            raise ValueError("sliding-window attention is not implemented")
        cfg = super().from_hf(d)
        cfg.qk_norm = True
        cfg.attention_bias = bool(d.get("attention_bias", False))
        return cfg

    @classmethod
    def tiny(cls, **kw) -> "Qwen3Config":
        base = dict(hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=64, vocab_size=4096, tie_word_embeddings=True,
                    max_position_embeddings=2048)
        base.update(kw)
        return cls(**base)

    def to_hf(self) -> dict:
        d = super().to_hf()
        d["model_type"] = "qwen3"
        d["use_sliding_window"] = False
        return d


@dataclass
class GraniteConfig(Llama3Config):
    """IBM Granite 3.x dense models (``GraniteForCausalLM``): the Llama layer with four scalars - the embedding,
    every block output and the attention scores are multiplied by constants and the logits divided by one. The
    first, second and last are folded into the embedding table, the o / down projections and the LM head when the
    checkpoint is read, so the layers run unchanged; ``attention_multiplier`` is the softmax scale.
    Reference: max/python/max/pipelines/architectures/granite/."""

    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    architectures: tuple = ("GraniteForCausalLM",)

    def to_hf(self) -> dict:
        d = super().to_hf()
        d["model_type"] = "granite"
        return d


@dataclass
class Gemma3Config(Llama3Config):
    """Gemma 3 text models (``Gemma3ForCausalLM``): four RMSNorms per layer (block inputs and outputs) whose weights
    the checkpoint stores minus one, per-head query / key norms, a tanh-GELU gated MLP, embeddings scaled by
    ``sqrt(hidden)``, ``query_pre_attn_scalar ** -0.5`` as the softmax scale, and five sliding-window layers (rotary
    base 10 000, no scaling) for every full-attention layer (base 1 000 000, linear scaling on the larger models). Every
    layer here attends to the whole prefix, so the served context is capped at the window, where the two agree. The
    attention kernels cover head sizes 64 and 128: checkpoints with ``head_dim`` 256 run on CPU only.
    Reference: max/python/max/pipelines/architectures/gemma3/."""

    rope_theta: float = 1000000.0
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 131072
    tie_word_embeddings: bool = True
    qk_norm: bool = True
    sandwich_norm: bool = True
    architectures: tuple = ("Gemma3ForCausalLM",)

    @classmethod
    def from_hf(cls, d: dict) -> "Gemma3Config":
        # a vision-language checkpoint (Gemma3ForConditionalGeneration) nests the language model's settings
        d = dict(d.get("text_config") or d, architectures=d.get("architectures", ["Gemma3ForCausalLM"]))
        if d.get("attn_logit_softcapping") or d.get("final_logit_softcapping"):
            raise ValueError("logit soft-capping is not implemented")
        act = d.pop("hidden_activation", None) or d.pop("hidden_act", None) or "gelu_pytorch_tanh"
        d.pop("hidden_act", None)
        if act not in ("gelu_pytorch_tanh", "gelu_tanh"):
            raise ValueError(f"activation {act!r} is not implemented for this family")
        rp = d.pop("rope_parameters", None)
        local_theta = d.get("rope_local_base_freq", 10000.0)
        if isinstance(rp, dict) and "full_attention" in rp:
            g, loc = rp["full_attention"], rp.get("sliding_attention") or {}
            d["rope_theta"] = g.get("rope_theta", 1000000.0)
            kind = g.get("rope_type", "default")
            d["rope_scaling"] = None if kind in (None, "default") else {k: v for k, v in g.items() if k != "rope_theta"}
            local_theta = loc.get("rope_theta", local_theta)
        d.setdefault("tie_word_embeddings", True)
        cfg = super().from_hf(d)
        cfg.qk_norm = cfg.sandwich_norm = True
        cfg.rope_local_theta = float(local_theta)
        types = d.get("layer_types")
        if types is None:
            pat = int(d.get("sliding_window_pattern") or d.get("_sliding_window_pattern") or 6)
            types = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention" for i in range(cfg.num_hidden_layers)]
        cfg.local_layers = tuple(i for i, t in enumerate(types) if t == "sliding_attention")
        cfg.attention_multiplier = float(d.get("query_pre_attn_scalar", cfg.head_dim)) ** -0.5
        cfg.embedding_multiplier = float(cfg.hidden_size) ** 0.5
        if cfg.local_layers:
            _cap_to_window(cfg, d.get("sliding_window"))
        return cfg

    def to_hf(self) -> dict:
        d = super().to_hf()
        d.update(model_type="gemma3_text", hidden_activation="gelu_pytorch_tanh", rope_local_base_freq=self.rope_local_theta,
                 query_pre_attn_scalar=(self.attention_multiplier or self.head_dim ** -0.5) ** -2,
                 layer_types=["sliding_attention" if i in self.local_layers else "full_attention"
                              for i in range(self.num_hidden_layers)])
        d.pop("hidden_act", None)
        return d


@dataclass
class OlmoConfig(Llama3Config):
    """OLMo (``OlmoForCausalLM``): the Llama layer with a LayerNorm without weight or bias in place of every
    RMSNorm, and the query / key / value projections clamped to ``[-clip_qkv, clip_qkv]`` where the checkpoint
    asks for it. Reference: max/python/max/pipelines/architectures/olmo/."""

    rope_theta: float = 10000.0
    max_position_embeddings: int = 2048
    plain_layer_norm: bool = True
    architectures: tuple = ("OlmoForCausalLM",)

    @classmethod
    def from_hf(cls, d: dict) -> "OlmoConfig":
        cfg = super().from_hf(d)
        cfg.plain_layer_norm = True
        cfg.clip_qkv = float(d["clip_qkv"]) if d.get("clip_qkv") else None
        return cfg

    def to_hf(self) -> dict:
        d = super().to_hf()
        d["model_type"] = "olmo"
        return d


@dataclass
class Olmo2Config(Llama3Config):
    """OLMo 2 and OLMo 3 (``Olmo2ForCausalLM``, ``Olmo3ForCausalLM``): Llama projections in another order - no norm
    on the block inputs, an RMSNorm on every block output before it joins the residual stream, and one RMSNorm over
    the whole query and the whole key projection before the rotation. OLMo 3 adds a sliding window on three layers
    out of four, which is served up to the window length.
    Reference: max/python/max/pipelines/architectures/olmo2/, olmo3/."""

    rope_theta: float = 500000.0
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 4096
    qk_norm: bool = True
    qk_norm_full: bool = True
    norm_after: bool = True
    architectures: tuple = ("Olmo2ForCausalLM",)

    @classmethod
    def from_hf(cls, d: dict) -> "Olmo2Config":
        cfg = super().from_hf(d)
        cfg.qk_norm = cfg.qk_norm_full = cfg.norm_after = True
        if "sliding_attention" in (d.get("layer_types") or ()):
            _cap_to_window(cfg, d.get("sliding_window"))
        return cfg

    @classmethod
    def tiny(cls, **kw) -> "Olmo2Config":
        base = dict(hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, vocab_size=4096, max_position_embeddings=2048)
        base.update(kw)
        return cls(**base)

    def to_hf(self) -> dict:
        d = super().to_hf()
        d["model_type"] = "olmo2"
        return d


@dataclass
class MixtralConfig(Llama3Config):
    """Mixtral (``MixtralForCausalLM``): Llama attention with a mixture-of-experts feed-forward in every layer -
    softmax over all experts, top-k, weights renormalised. ``intermediate_size`` is the size of one expert.
    Reference: max/python/max/pipelines/architectures/mixtral/."""

    rope_theta: float = 1000000.0
    max_position_embeddings: int = 32768
    num_experts: int = 8
    num_experts_per_tok: int = 2
    architectures: tuple = ("MixtralForCausalLM",)

    @classmethod
    def from_hf(cls, d: dict) -> "MixtralConfig":
        d = dict(d)
        d["num_experts"] = d.get("num_local_experts", d.get("num_experts", 8))
        cfg = _cap_to_window(super().from_hf(d), d.get("sliding_window"))
        cfg.moe_intermediate_size = cfg.intermediate_size
        cfg.norm_topk_prob = True
        return cfg

    def __post_init__(self):
        super().__post_init__()
        if not self.moe_intermediate_size:
            self.moe_intermediate_size = self.intermediate_size

    @classmethod
    def tiny(cls, **kw) -> "MixtralConfig":
        base = dict(hidden_size=256, intermediate_size=384, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, vocab_size=4096, num_experts=4, num_experts_per_tok=2,
                    max_position_embeddings=2048)
        base.update(kw)
        return cls(**base)

    def to_hf(self) -> dict:
        d = super().to_hf()
        d["model_type"] = "mixtral"
        d["num_local_experts"] = self.num_experts
        d["sliding_window"] = None
        return d


@dataclass
class Qwen3MoeConfig(Qwen3Config):
    """Qwen3 mixture-of-experts models (``Qwen3MoeForCausalLM``): Qwen3 attention; layers selected by
    ``decoder_sparse_step`` / ``mlp_only_layers`` route to ``num_experts`` experts of ``moe_intermediate_size``
    (softmax, top-k, optional renormalisation), the others keep the dense MLP.
    Reference: max/python/max/pipelines/architectures/qwen3_moe/."""

    num_experts: int = 128
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    architectures: tuple = ("Qwen3MoeForCausalLM",)

    @classmethod
    def tiny(cls, **kw) -> "Qwen3MoeConfig":
        base = dict(hidden_size=256, intermediate_size=512, moe_intermediate_size=128, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=4096, num_experts=8,
                    num_experts_per_tok=2, tie_word_embeddings=False, max_position_embeddings=2048)
        base.update(kw)
        return cls(**base)

    def to_hf(self) -> dict:
        d = super().to_hf()
        d["model_type"] = "qwen3_moe"
        return d


@dataclass
class Phi3Config(Llama3Config):
    """Phi-3 / Phi-3.5 mini (``Phi3ForCausalLM``): the Llama layer with the q / k / v and the gate / up projections
    already fused in the checkpoint (``qkv_proj``, ``gate_up_proj``). The 128k variants scale the rotary
    frequencies with LongRoPE; partial rotary embeddings (Phi-4-mini) are refused. Reference: max/python/max/pipelines/architectures/phi3/."""

    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    architectures: tuple = ("Phi3ForCausalLM",)

    @classmethod
    def from_hf(cls, d: dict) -> "Phi3Config":
        from ..pipelines.weights import normalize_hf_rope

        d = normalize_hf_rope(d)
        if float(d.get("partial_rotary_factor", (d.get("rope_parameters") or {}).get("partial_rotary_factor", 1.0))) != 1.0:
            raise ValueError("partial rotary embeddings are not implemented")
        rs = d.get("rope_scaling")
        if rs:
            kind = rs.get("rope_type", rs.get("type"))
            if kind not in ("longrope", "su"):
                raise ValueError(f"rotary scaling {kind!r} is not implemented for this family")
            # LongRoPE (the 128k variants): per-frequency divisors for short and for long contexts and an attention
            # factor from the ratio of the two context lengths, which live at the top level of the config. The
            # table is built once: long divisors when the served context exceeds the original one, else short.
            orig = int(d.get("original_max_position_embeddings") or rs.get("original_max_position_embeddings")
                       or d["max_position_embeddings"])
            d = dict(d, rope_scaling=dict(rs, rope_type="longrope", original_max_position_embeddings=orig,
                                          factor=rs.get("factor") or d["max_position_embeddings"] / orig))
        return _cap_to_window(super().from_hf(d), (d.get("text_config") or d).get("sliding_window"))

    def to_hf(self) -> dict:
        d = super().to_hf()
        d["model_type"] = "phi3"
        d["sliding_window"] = None
        return d



@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    wqkv: torch.Tensor
    wo: torch.Tensor
    mlp_norm: torch.Tensor
    wgu: torch.Tensor
    wd: torch.Tensor
    # block-scaled fp8 layers: the four matrices are float8_e4m3fn and these hold one fp32 scale per
    # 128 x 128 block ([ceil(N/128), ceil(K/128)], the checkpoint's ``weight_scale_inv``); None = bf16
    wqkv_s: Optional[torch.Tensor] = None
    wo_s: Optional[torch.Tensor] = None
    wgu_s: Optional[torch.Tensor] = None
    wd_s: Optional[torch.Tensor] = None
    qkv_bias: Optional[torch.Tensor] = None      # [q; k; v] projection bias (Qwen2), in the activation dtype
    q_norm: Optional[torch.Tensor] = None        # [head_dim] weights of the per-head query / key RMSNorm (Qwen3)
    k_norm: Optional[torch.Tensor] = None
    moe: Optional[object] = None                 # nn.moe.MoE of a mixture-of-experts layer (wgu / wd are None then)
    attn_out_norm: Optional[torch.Tensor] = None  # Gemma 3: RMSNorm weights on the attention / MLP block outputs
    mlp_out_norm: Optional[torch.Tensor] = None

    @property
    def is_fp8(self) -> bool:
        return self.wqkv_s is not None

    def scales(self):
        return [self.wqkv_s, self.wo_s, self.wgu_s, self.wd_s] if self.is_fp8 else None


@dataclass
class Llama3Weights:
    embed: torch.Tensor
    layers: list
    final_norm: torch.Tensor
    lm_head: torch.Tensor

    @classmethod
    def random_init(cls, cfg: Llama3Config, device="cpu", dtype=torch.bfloat16, seed: int = 0,
                    std: float = 0.02) -> "Llama3Weights":
        g = torch.Generator(device="cpu").manual_seed(seed)
        dev = torch.device(device)

        def rnd(*shape):
            if dev.type == "cuda" and math.prod(shape) > (1 << 22):
                # large tensors: generate on the device (seeded per tensor)
                gd = torch.Generator(device=dev).manual_seed(int(torch.randint(0, 2**31, (1,), generator=g)))
                return (torch.randn(*shape, device=dev, dtype=torch.float32, generator=gd) * std).to(dtype)
            return (torch.randn(*shape, generator=g) * std).to(dtype).to(dev)

        embed = rnd(cfg.vocab_size, cfg.hidden_size)
        layers = []
        for li in range(cfg.num_hidden_layers):
            moe = None
            if cfg.is_moe_layer(li):
                from ..nn.moe import MoE

                moe = MoE.random_init(cfg.moe_config(), dev, dtype, seed=seed * 1009 + li + 1, std=std)
            layers.append(LayerWeights(
                attn_norm=torch.ones(cfg.hidden_size, dtype=dtype, device=dev),
                wqkv=rnd(cfg.q_dim + 2 * cfg.kv_dim, cfg.hidden_size),
                wo=rnd(cfg.hidden_size, cfg.q_dim),
                mlp_norm=torch.ones(cfg.hidden_size, dtype=dtype, device=dev),
                wgu=None if moe is not None else rnd(2 * cfg.intermediate_size, cfg.hidden_size),
                wd=None if moe is not None else rnd(cfg.hidden_size, cfg.intermediate_size), moe=moe,
                qkv_bias=rnd(cfg.q_dim + 2 * cfg.kv_dim) if cfg.attention_bias else None,
                q_norm=torch.ones(cfg.q_dim if cfg.qk_norm_full else cfg.head_dim, dtype=dtype, device=dev)
                if cfg.qk_norm else None,
                k_norm=torch.ones(cfg.kv_dim if cfg.qk_norm_full else cfg.head_dim, dtype=dtype, device=dev)
                if cfg.qk_norm else None,
                attn_out_norm=torch.ones(cfg.hidden_size, dtype=dtype, device=dev) if cfg.sandwich_norm else None,
                mlp_out_norm=torch.ones(cfg.hidden_size, dtype=dtype, device=dev) if cfg.sandwich_norm else None))
        final_norm = torch.ones(cfg.hidden_size, dtype=dtype, device=dev)
        lm_head = embed if cfg.tie_word_embeddings else rnd(cfg.vocab_size, cfg.hidden_size)
        return cls(embed, layers, final_norm, lm_head)

    @classmethod
    def random_init_shard(cls, cfg: Llama3Config, rank: int, world: int, device="cuda", dtype=torch.bfloat16,
                          seed: int = 0, std: float = 0.02, fp8: bool = False) -> "Llama3Weights":
        """Random weights of ONE tensor-parallel rank, created at shard size (a 70B model never exists whole
        on a GPU). Replicated tensors (embedding, norms) come from ``seed`` alone and are identical on every
        rank; sharded ones mix in the rank. ``fp8`` quantises each layer as it is made, so the peak footprint
        is one bf16 layer shard. The values are not a sharding of ``random_init(cfg, seed)``: this is for
        synthetic-weight benchmarks, where only shapes and dtypes matter."""
        from ..parallel.tp import shard_llama_config

        local = shard_llama_config(cfg, world) if world > 1 else cfg
        dev = torch.device(device)
        g_shared = torch.Generator(device=dev).manual_seed(seed)
        g_rank = torch.Generator(device=dev).manual_seed(seed * 1000003 + rank + 1)
        rnd = lambda g, *shape: (torch.randn(*shape, device=dev, dtype=torch.float32, generator=g) * std).to(dtype)
        embed = rnd(g_shared, cfg.vocab_size, cfg.hidden_size)
        ones = lambda: torch.ones(cfg.hidden_size, dtype=dtype, device=dev)
        layers = []
        for _ in range(cfg.num_hidden_layers):
            l = LayerWeights(ones(), rnd(g_rank, local.q_dim + 2 * local.kv_dim, cfg.hidden_size),
                             rnd(g_rank, cfg.hidden_size, local.q_dim), ones(),
                             rnd(g_rank, 2 * local.intermediate_size, cfg.hidden_size),
                             rnd(g_rank, cfg.hidden_size, local.intermediate_size),
                             qkv_bias=rnd(g_rank, local.q_dim + 2 * local.kv_dim) if cfg.attention_bias else None,
                             q_norm=torch.ones(cfg.head_dim, dtype=dtype, device=dev) if cfg.qk_norm else None,
                             k_norm=torch.ones(cfg.head_dim, dtype=dtype, device=dev) if cfg.qk_norm else None)
            if fp8:
                l = cls(embed, [l], ones(), embed).quantize_fp8().layers[0]
            layers.append(l)
        v_local = cfg.vocab_size // world
        lm_head = rnd(g_rank, v_local, cfg.hidden_size) if (world > 1 or not cfg.tie_word_embeddings) else embed
        return cls(embed, layers, ones(), lm_head)

    def quantize_fp8(self) -> "Llama3Weights":
        """Block-scaled fp8 copy of these weights: every projection becomes e4m3 with 128 x 128 scales
        (amax / 448); embeddings, norms and the LM head keep their dtype. Reference:
        max/python/max/pipelines/weights/quantize_checkpoint.py, quant config weights/quant.py:581."""
        def q(w):
            return ops.reference.quant_fp8_weight_block128(w)

        layers = []
        for l in self.layers:
            if l.is_fp8:
                layers.append(l)
                continue
            (a, a_s), (b, b_s), (c_, c_s), (d, d_s) = q(l.wqkv), q(l.wo), q(l.wgu), q(l.wd)
            layers.append(LayerWeights(l.attn_norm, a, b, l.mlp_norm, c_, d, a_s, b_s, c_s, d_s, l.qkv_bias,
                                       l.q_norm, l.k_norm))
        return Llama3Weights(self.embed, layers, self.final_norm, self.lm_head)

    def dequantize(self, dtype=torch.bfloat16) -> "Llama3Weights":
        """The same weights with fp8 layers expanded to ``dtype`` (what the fp8 kernels compute, up to the
        activation quantisation)."""
        d = lambda w, s: ops.reference.dequant_fp8_weight_block128(w, s).to(dtype)
        layers = [LayerWeights(l.attn_norm, d(l.wqkv, l.wqkv_s), d(l.wo, l.wo_s), l.mlp_norm, d(l.wgu, l.wgu_s),
                               d(l.wd, l.wd_s), qkv_bias=l.qkv_bias, q_norm=l.q_norm, k_norm=l.k_norm)
                  if l.is_fp8 else l for l in self.layers]
        return Llama3Weights(self.embed, layers, self.final_norm, self.lm_head)

    @classmethod
    def from_state_dict(cls, cfg: Llama3Config, sd: dict, device="cpu", dtype=torch.bfloat16, keep_fp8: bool = True):
        """``keep_fp8``: block-scaled fp8 projections (``<name>`` e4m3 + ``<name>_scale_inv``) stay fp8 when the
        fused row blocks line up with the 128-row scale blocks; otherwise they are expanded to ``dtype``."""
        sd = _split_fused_projections(cfg, adapt_hf_state_dict(sd))
        if cfg.sandwich_norm:
            # the checkpoint stores every norm weight minus one; the four norms of a layer: the two on the block
            # inputs go where Llama's are, the two on the block outputs get slots of their own
            ren = lambda k: (k.replace(".post_attention_layernorm.", ".attn_out_norm.")
                             .replace(".pre_feedforward_layernorm.", ".post_attention_layernorm.")
                             .replace(".post_feedforward_layernorm.", ".mlp_out_norm."))
            sd = {ren(k): (v.float() + 1.0 if k.endswith("norm.weight") else v) for k, v in sd.items()}
        if cfg.plain_layer_norm:
            # norms without parameters: nothing in the checkpoint; the slots hold ones and are not read
            one = torch.ones(cfg.hidden_size)
            sd = dict(sd)
            for i in range(cfg.num_hidden_layers):
                sd.setdefault(f"layers.{i}.input_layernorm.weight", one)
                sd.setdefault(f"layers.{i}.post_attention_layernorm.weight", one)
            sd.setdefault("norm.weight", one)
        if cfg.norm_after:
            # the two norms of a layer sit on the block outputs: the attention one is kept where the input norm of
            # the attention block is otherwise, the feed-forward one where the input norm of the MLP is
            sd = {k.replace(".post_attention_layernorm.", ".input_layernorm.")
                  .replace(".post_feedforward_layernorm.", ".post_attention_layernorm."): v for k, v in sd.items()}
        # parameters this family has no place for must not be dropped silently
        extra = [k for k in sd if k.endswith((".o_proj.bias", ".gate_proj.bias", ".up_proj.bias", ".down_proj.bias"))
                 and bool(torch.count_nonzero(sd[k]))]
        if extra:
            raise ValueError(f"checkpoint has biases that are not implemented: {extra[:3]}")
        dev = torch.device(device)
        fp8_names = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                     "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")

        def layer_is_fp8(p):
            return keep_fp8 and all(
                sd[p + n + ".weight"].dtype == torch.float8_e4m3fn and (p + n + ".weight_scale_inv") in sd
                and (n in ("self_attn.o_proj", "mlp.down_proj") or sd[p + n + ".weight"].shape[0] % 128 == 0)
                for n in fp8_names)

        def fp8_cat(p, names):
            w = torch.cat([sd[p + n + ".weight"] for n in names], dim=0).to(dev).contiguous()
            s_ = torch.cat([sd[p + n + ".weight_scale_inv"].float() for n in names], dim=0).to(dev).contiguous()
            return w, s_

        def raw(name):
            """Checkpoint tensor in floating point: fp8 tensors (block-scaled ``<name>_scale_inv`` [N/128, K/128],
            or per-tensor ``weight_scale``) are expanded with their scales; the GEMMs then run in ``dtype``."""
            w = sd[name]
            if w.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
                if name + "_scale_inv" in sd:
                    return ops.reference.dequant_fp8_weight_block128(w, sd[name + "_scale_inv"].float())
                scale = sd.get(name.replace(".weight", ".weight_scale"))
                return w.float() * (scale.float() if scale is not None else 1.0)
            return w

        def get(name):
            return raw(name).to(device=dev, dtype=dtype).contiguous()

        def bias(p):
            names = [p + f"self_attn.{n}_proj.bias" for n in "qkv"]
            if not all(n in sd for n in names):
                return None
            return torch.cat([sd[n].float() for n in names]).to(device=dev, dtype=dtype).contiguous()

        def opt(name):
            return get(name) if name in sd else None

        layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            if layer_is_fp8(p):
                a, a_s = fp8_cat(p, ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"))
                b, b_s = fp8_cat(p, ("self_attn.o_proj",))
                c_, c_s = fp8_cat(p, ("mlp.gate_proj", "mlp.up_proj"))
                d, d_s = fp8_cat(p, ("mlp.down_proj",))
                layers.append(LayerWeights(get(p + "input_layernorm.weight"), a, b,
                                           get(p + "post_attention_layernorm.weight"), c_, d, a_s, b_s, c_s, d_s,
                                           bias(p), opt(p + "self_attn.q_norm.weight"),
                                           opt(p + "self_attn.k_norm.weight")))
                continue
            wqkv = torch.cat([raw(p + "self_attn.q_proj.weight"), raw(p + "self_attn.k_proj.weight"),
                              raw(p + "self_attn.v_proj.weight")], dim=0)
            moe = _moe_from_state_dict(cfg, sd, p, dev, dtype) if cfg.is_moe_layer(i) else None
            wgu = None
            if moe is None:
                wgu = torch.cat([raw(p + "mlp.gate_proj.weight"), raw(p + "mlp.up_proj.weight")], dim=0)
                wgu = wgu.to(device=dev, dtype=dtype).contiguous()
            layers.append(LayerWeights(
                attn_norm=get(p + "input_layernorm.weight"),
                wqkv=wqkv.to(device=dev, dtype=dtype).contiguous(),
                wo=get(p + "self_attn.o_proj.weight"),
                mlp_norm=get(p + "post_attention_layernorm.weight"),
                wgu=wgu, wd=None if moe is not None else get(p + "mlp.down_proj.weight"), moe=moe,
                qkv_bias=bias(p),
                q_norm=opt(p + "self_attn.q_norm.weight"), k_norm=opt(p + "self_attn.k_norm.weight"),
                attn_out_norm=opt(p + "attn_out_norm.weight"), mlp_out_norm=opt(p + "mlp_out_norm.weight")))
        embed = get("embed_tokens.weight")
        lm_head = embed if (cfg.tie_word_embeddings or "lm_head.weight" not in sd) else get("lm_head.weight")
        if cfg.embedding_multiplier != 1.0 or cfg.logits_scaling != 1.0 or cfg.residual_multiplier != 1.0:
            # Granite's scalars go into the weights (computed in fp32, rounded once); a tied LM head becomes its own
            # tensor because table and head are scaled differently
            scaled = lambda w, f: (w.float() * f).to(dtype) if f != 1.0 else w
            lm_head = scaled(lm_head, 1.0 / cfg.logits_scaling)
            embed = scaled(embed, cfg.embedding_multiplier)
            for l in layers:
                if l.is_fp8 or l.moe is not None:
                    raise ValueError("residual / embedding multipliers are folded into bf16 dense layers only")
                l.wo, l.wd = scaled(l.wo, cfg.residual_multiplier), scaled(l.wd, cfg.residual_multiplier)
        return cls(embed, layers, get("norm.weight"), lm_head)

    def to_hf_state_dict(self, cfg: Llama3Config) -> dict:
        """Inverse of :meth:`from_state_dict` (used to write checkpoints in tests and tools)."""
        sd = {"model.embed_tokens.weight": self.embed, "model.norm.weight": self.final_norm}
        if not cfg.tie_word_embeddings:
            sd["lm_head.weight"] = self.lm_head
        for i, l in enumerate(self.layers):
            p = f"model.layers.{i}."
            if l.q_norm is not None:
                sd.update({p + "self_attn.q_norm.weight": l.q_norm, p + "self_attn.k_norm.weight": l.k_norm})
            if l.qkv_bias is not None:
                bq, bk, bv = torch.split(l.qkv_bias, [cfg.q_dim, cfg.kv_dim, cfg.kv_dim])
                sd.update({p + "self_attn.q_proj.bias": bq, p + "self_attn.k_proj.bias": bk,
                           p + "self_attn.v_proj.bias": bv})
            if l.is_fp8:
                # e4m3 tensors cannot be split by torch.split on every build: slice through the byte view
                rows = lambda w, a, b: w.view(torch.uint8)[a:b].view(torch.float8_e4m3fn)
                qd, kd, I = cfg.q_dim, cfg.kv_dim, cfg.intermediate_size
                parts = {"self_attn.q_proj": (l.wqkv, l.wqkv_s, 0, qd), "self_attn.k_proj": (l.wqkv, l.wqkv_s, qd, qd + kd),
                         "self_attn.v_proj": (l.wqkv, l.wqkv_s, qd + kd, qd + 2 * kd),
                         "self_attn.o_proj": (l.wo, l.wo_s, 0, l.wo.shape[0]),
                         "mlp.gate_proj": (l.wgu, l.wgu_s, 0, I), "mlp.up_proj": (l.wgu, l.wgu_s, I, 2 * I),
                         "mlp.down_proj": (l.wd, l.wd_s, 0, l.wd.shape[0])}
                for n, (w, s_, a, b) in parts.items():
                    sd[p + n + ".weight"] = rows(w, a, b)
                    sd[p + n + ".weight_scale_inv"] = s_[a // 128:(b + 127) // 128]
                sd[p + "input_layernorm.weight"] = l.attn_norm
                sd[p + "post_attention_layernorm.weight"] = l.mlp_norm
                continue
            q, k, v = torch.split(l.wqkv, [cfg.q_dim, cfg.kv_dim, cfg.kv_dim], dim=0)
            sd.update({p + "input_layernorm.weight": l.attn_norm, p + "self_attn.q_proj.weight": q,
                       p + "self_attn.k_proj.weight": k, p + "self_attn.v_proj.weight": v,
                       p + "self_attn.o_proj.weight": l.wo,
                       p + "post_attention_layernorm.weight": l.mlp_norm})
            if l.moe is not None:
                sd.update({p + "mlp.gate.weight": l.moe.gate.to(l.wo.dtype), p + "mlp.experts.gate_up_proj": l.moe.w_gate_up,
                           p + "mlp.experts.down_proj": l.moe.w_down})
                continue
            g, u = torch.split(l.wgu, cfg.intermediate_size, dim=0)
            sd.update({p + "mlp.gate_proj.weight": g, p + "mlp.up_proj.weight": u,
                       p + "mlp.down_proj.weight": l.wd})
        if cfg.sandwich_norm:
            for i, l in enumerate(self.layers):
                sd[f"model.layers.{i}.attn_out_norm.weight"] = l.attn_out_norm
                sd[f"model.layers.{i}.mlp_out_norm.weight"] = l.mlp_out_norm
            ren = lambda k: (k.replace(".post_attention_layernorm.", ".pre_feedforward_layernorm.")
                             .replace(".attn_out_norm.", ".post_attention_layernorm.")
                             .replace(".mlp_out_norm.", ".post_feedforward_layernorm."))
            sd = {ren(k): (v.float() - 1.0).to(v.dtype) if k.endswith("norm.weight") else v for k, v in sd.items()}
            if cfg.embedding_multiplier != 1.0:
                sd["model.embed_tokens.weight"] = (self.embed.float() / cfg.embedding_multiplier).to(self.embed.dtype)
        if cfg.plain_layer_norm:
            sd = {k: v for k, v in sd.items() if not k.endswith(("layernorm.weight", "model.norm.weight"))}
        if cfg.norm_after:
            sd = {k.replace(".post_attention_layernorm.", ".post_feedforward_layernorm.")
                  .replace(".input_layernorm.", ".post_attention_layernorm."): v for k, v in sd.items()}
        return {k: v.contiguous() for k, v in sd.items()}


def _moe_from_state_dict(cfg, sd: dict, p: str, dev, dtype):
    """The mixture-of-experts feed-forward of layer prefix ``p``. Three checkpoint layouts: all experts in two
    tensors (``mlp.experts.gate_up_proj`` [E, 2 I, H] and ``mlp.experts.down_proj`` [E, H, I], what transformers >= 5
    writes), one set per expert (``mlp.experts.N.{gate,up,down}_proj``, Qwen3-MoE on the hub), and Mixtral's
    ``block_sparse_moe.experts.N.{w1,w3,w2}`` (gate, up, down)."""
    from ..nn.moe import MoE

    E = cfg.num_experts
    to = lambda t: t.to(device=dev, dtype=dtype).contiguous()
    if p + "mlp.experts.gate_up_proj" in sd:
        gate = sd[p + "mlp.gate.weight"]
        gu, dn = to(sd[p + "mlp.experts.gate_up_proj"]), to(sd[p + "mlp.experts.down_proj"])
    elif p + "block_sparse_moe.gate.weight" in sd:
        m = p + "block_sparse_moe."
        gate = sd[m + "gate.weight"]
        gu = to(torch.stack([torch.cat((sd[f"{m}experts.{e}.w1.weight"], sd[f"{m}experts.{e}.w3.weight"])) for e in range(E)]))
        dn = to(torch.stack([sd[f"{m}experts.{e}.w2.weight"] for e in range(E)]))
    else:
        m = p + "mlp."
        gate = sd[m + "gate.weight"]
        gu = to(torch.stack([torch.cat((sd[f"{m}experts.{e}.gate_proj.weight"], sd[f"{m}experts.{e}.up_proj.weight"]))
                             for e in range(E)]))
        dn = to(torch.stack([sd[f"{m}experts.{e}.down_proj.weight"] for e in range(E)]))
    return MoE(cfg.moe_config(), gate.float().to(dev), gu, dn)


def _split_fused_projections(cfg, sd: dict) -> dict:
    """Checkpoints that store ``qkv_proj`` / ``gate_up_proj`` (Phi-3) -> the separate tensors the loader expects
    (views, no copies)."""
    if not any(k.endswith("self_attn.qkv_proj.weight") for k in sd):
        return sd
    out = {}
    for k, v in sd.items():
        if k.endswith("self_attn.qkv_proj.weight"):
            p = k[: -len("qkv_proj.weight")]
            q, kk, vv = torch.split(v, [cfg.q_dim, cfg.kv_dim, cfg.kv_dim], dim=0)
            out[p + "q_proj.weight"], out[p + "k_proj.weight"], out[p + "v_proj.weight"] = q, kk, vv
        elif k.endswith("mlp.gate_up_proj.weight"):
            p = k[: -len("gate_up_proj.weight")]
            g, u = torch.split(v, cfg.intermediate_size, dim=0)
            out[p + "gate_proj.weight"], out[p + "up_proj.weight"] = g, u
        else:
            out[k] = v
    return out


def adapt_hf_state_dict(sd: dict) -> dict:
    """HF checkpoint names -> internal names: strips the ``model.`` prefix, keeps ``lm_head``. Of a vision-language
    checkpoint the language model is kept (``language_model.`` wrappers stripped) and the vision tower and projector
    are dropped: such checkpoints are served for text."""
    out = {}
    for k, v in sd.items():
        if any(part in k for part in ("vision_tower.", "vision_model.", "multi_modal_projector.", "visual.",
                                      "model.connector.")):
            continue
        for pre in ("model.language_model.", "language_model.model.", "language_model.", "model.text_model.", "model."):
            if k.startswith(pre):
                k = k[len(pre):]
                break
        out[k] = v
    return out


class Llama3Model:
    """Runs ragged batches of a Llama-3 decoder against a paged KV cache."""

    def __init__(self, cfg: Llama3Config, weights: Llama3Weights, kv_cache: torch.Tensor,
                 max_tokens: int = 8192, max_seqs: int = 256, max_position: Optional[int] = None,
                 use_executor: Optional[bool] = None, fuse_swiglu: bool = True, tp=None):
        # under tensor parallelism `cfg` and `weights` are this rank's shard (heads, FFN and
        # LM-head rows divided by the TP degree; hidden and vocab sizes stay global)
        self.cfg = cfg
        self.tp = tp
        self.w = weights
        self.kv = kv_cache
        self.device = weights.embed.device
        self.dtype = weights.embed.dtype
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs
        self.page_size = kv_cache.shape[4]
        self.scale = cfg.attention_multiplier or 1.0 / math.sqrt(cfg.head_dim)
        max_position = max_position or cfg.max_position_embeddings
        self.cos_sin = cos_sin_table(cfg.head_dim, max_position, cfg.rope_theta,
                                     RopeScaling.from_hf(cfg.rope_scaling), self.device)
        self.cos_sin_local = None
        if cfg.rope_local_theta:
            self.cos_sin_local = cos_sin_table(cfg.head_dim, max_position, cfg.rope_local_theta, None, self.device)
        on_gpu = self.device.type == "cuda"
        self.use_executor = on_gpu and self.dtype == torch.bfloat16 if use_executor is None else use_executor
        if any(l.moe is not None for l in weights.layers):
            # mixture-of-experts layers run op by op (router, grouped GEMMs of nn.moe); the native step executor
            # knows dense layers only
            self.use_executor = False
            if tp is not None and tp.world > 1:
                raise ValueError("tensor parallelism is not implemented for mixture-of-experts layers of this family")
        if cfg.norm_after or cfg.qk_norm_full or cfg.plain_layer_norm or cfg.clip_qkv or cfg.sandwich_norm:
            # another layer order than the native step executor runs
            self.use_executor = False
            if tp is not None and tp.world > 1:
                raise ValueError("tensor parallelism is not implemented for the OLMo and Gemma layer variants")
        self.fuse_swiglu = fuse_swiglu
        self.executor = None
        self.logits_buf = None
        if self.use_executor:
            self._build_executor()

    # ------------------------------------------------------------ native path
    def _build_executor(self) -> None:
        c, dev, dt = self.cfg, self.device, self.dtype
        L = _lib()
        ex = L.DecoderExecutor(dict(
            n_layers=c.num_hidden_layers, hidden=c.hidden_size, n_q=c.num_attention_heads,
            n_kv=c.num_key_value_heads, head_dim=c.head_dim, inter=c.intermediate_size,
            vocab=c.vocab_size, eps=c.rms_norm_eps, page_size=self.page_size,
            attn_scale=self.scale, fuse_swiglu=int(self.fuse_swiglu),
            gemm_impl={"tiled": 0, "persistent": 1}.get(ops.GEMM_IMPL, 2),
            use_pdl=int(os.environ.get("MB200_PDL", "0")),
            attn_impl=int(os.environ.get("MB200_ATTN_TMA", "1")),
            # steps of up to this many tokens run the decode-step GEMMs (fused all-reduce + residual + norm)
            dec_max_tokens=self._dec_tokens(),
            # weights are static: the tiled GEMMs may request their first tiles while the previous kernel drains
            prefetch_weights=int(os.environ.get("MB200_PREFETCH_W", "1") not in ("", "0"))))
        ex.set_globals(self.w.embed, self.w.final_norm, self.w.lm_head, self.cos_sin)
        self.is_fp8 = any(l.is_fp8 for l in self.w.layers)
        if self.is_fp8 and not all(l.is_fp8 for l in self.w.layers):
            raise ValueError("mixed fp8 / bf16 layers are not supported by the executor")
        for l in self.w.layers:
            ex.add_layer(l.attn_norm, l.wqkv, l.wo, l.mlp_norm, l.wgu, l.wd, l.scales(), l.qkv_bias, l.q_norm, l.k_norm)
        ex.set_kv_cache(self.kv)
        T, B = self.max_tokens, self.max_seqs
        mk = lambda *s, dtype=dt: torch.empty(*s, dtype=dtype, device=dev)
        self.logits_buf = mk(B, c.vocab_size, dtype=torch.float32)
        self.sampled = torch.zeros(B, dtype=torch.long, device=dev)
        self._bufs = dict(
            h=mk(T, c.hidden_size), xn=mk(T, c.hidden_size), qkv=mk(T, c.q_dim + 2 * c.kv_dim),
            attn=mk(T, c.q_dim), act=mk(T, c.intermediate_size),
            gu=None if self.fuse_swiglu else mk(T, 2 * c.intermediate_size),
            last_h=mk(B, c.hidden_size), last_xn=mk(B, c.hidden_size))
        b = self._bufs
        ex.set_buffers(b["h"], b["xn"], b["qkv"], b["attn"], b["act"], b["gu"], b["last_h"],
                       b["last_xn"], self.logits_buf, self.sampled, ops.gemm_workspace(dev),
                       *ops.persistent_gemm_workspace(dev))
        if self.is_fp8:
            # quantised activations (e4m3 + one fp32 scale per token and 128-wide K group) and the unfused
            # gate/up product
            kmax = max(c.hidden_size, c.intermediate_size, c.q_dim)
            self._fp8_bufs = (torch.empty(T, kmax, dtype=torch.uint8, device=dev),
                              torch.empty((kmax + 127) // 128, T, dtype=torch.float32, device=dev),
                              b["gu"] if b["gu"] is not None else mk(T, 2 * c.intermediate_size))
            ex.set_fp8_buffers(*self._fp8_bufs)
        ex.set_dec(*ops.decode_gemm_workspace(dev))
        ops.ensure_attention_split_workspace(dev)
        if self.tp is not None and self.tp.world > 1:
            # symmetric buffers for the fused reduce-scatter + norm + all-gather and the logits
            tp, W = self.tp, self.tp.world
            vocab_local = self.w.lm_head.shape[0]
            # fused GEMM+collective path: partial slots [slot][rows_per_rank][hidden]; W * rows_per_rank
            # can exceed T by W - 1 rows
            # bit0: GEMM -> reduce-scatter pushes, bit1: flag-gated all-gather -> GEMM
            fused = int(os.environ.get("MB200_TP_FUSED", "2"))
            partial_rows = T + W
            sym_partial = tp.alloc_symmetric(partial_rows * c.hidden_size, dt)
            sym_xn = tp.alloc_symmetric(T * c.hidden_size, dt)
            sym_logits = tp.alloc_symmetric(B * c.vocab_size, torch.float32)
            sym_flags = tp.alloc_symmetric(max(64, L.tp_flag_ints()), torch.int32, zero=True)
            self._tp_bufs = (sym_partial, sym_xn, sym_logits, sym_flags)
            h_local = mk((T + W - 1) // W, c.hidden_size)
            logits_local = mk(B, vocab_local, dtype=torch.float32)
            self.logits_buf = sym_logits.tensor.view(B, c.vocab_size)
            tp.barrier()  # flags are zeroed everywhere before any kernel can touch them
            ex.set_tp(W, tp.rank, sym_partial.peer_ptrs, sym_xn.peer_ptrs, sym_logits.peer_ptrs,
                      sym_flags.peer_ptrs, h_local, logits_local, vocab_local, fused, partial_rows)
            # decode steps: receive buffers of the fused GEMM + all-reduce + norm, every word a bf16 -0.0
            # ("nothing has arrived"); the kernels restore that state themselves after each use
            lam_rows = min(T, self._dec_tokens(), L.gemm_dec_sizes()[2])
            if lam_rows > 0:
                sym_lam = tp.alloc_symmetric(L.gemm_dec_lamport_elems(W, lam_rows, c.hidden_size), dt)
                sym_lam.tensor.view(torch.int16).fill_(-32768)
                self._tp_bufs += (sym_lam,)
                tp.barrier()
                ex.set_tp_lamport(sym_lam.peer_ptrs, lam_rows)
        self.executor = ex

    def _dec_tokens(self) -> int:
        """Largest step (tokens) that takes the decode-step GEMM path. Under tensor parallelism it replaces two
        collective launches per layer and wins at every decode size; on one GPU the tiled kernels with
        split-K measured faster (106 against 117 us per layer of GEMMs at 64 tokens), so it is off there.
        ``MB200_DEC_TOKENS`` overrides."""
        env = os.environ.get("MB200_DEC_TOKENS")
        if env is not None:
            return int(env)
        return 256 if (self.tp is not None and self.tp.world > 1) else 0

    def forward_packed(self, meta: torch.Tensor, offsets: dict, T: int, B: int, bt_stride: int,
                       n_tiles: int, n_decode: int, n_logits: int, has_future: bool = False,
                       do_sample: bool = False, sample_step: int = 0) -> torch.Tensor:
        """Native step from a packed device metadata buffer. Returns fp32 logits
        ``[n_logits, vocab]`` (a view of a persistent buffer, valid until the next call). With
        ``do_sample`` the sampled ids land in ``self.sampled[:n_logits]``; with ``has_future``
        token ids flagged in the batch are first taken from the previous step's ``sampled``."""
        if T > self.max_tokens or n_logits > self.max_seqs:
            raise ValueError(f"batch of {T} tokens / {n_logits} logit rows exceeds the executor's "
                             f"buffers ({self.max_tokens}, {self.max_seqs})")
        self.executor.forward(meta, offsets, T, B, bt_stride, n_tiles, n_decode, n_logits,
                              has_future, do_sample, sample_step)
        return self.logits_buf[:n_logits]

    # ------------------------------------------------------------ op-by-op path
    def forward_tensors(self, tokens, positions, slots, block_table, q_start, q_len, kv_len,
                        logit_rows, plan=None, lora=None) -> torch.Tensor:
        """Same computation through :mod:`modular_b200.ops` one op at a time (CPU, and the
        cross-check for the executor on GPU). Returns fp32 logits [len(logit_rows), vocab]."""
        h = self.forward_hidden(tokens, positions, slots, block_table, q_start, q_len, kv_len, plan=plan, lora=lora)
        last = h[logit_rows.long()]
        xn = self._norm(last, self.w.final_norm)
        logits = ops.linear(xn, self.w.lm_head, out_dtype=torch.float32)
        return logits.float()

    def forward_hidden(self, tokens, positions, slots, block_table, q_start, q_len, kv_len, plan=None,
                       kv=None, lora=None) -> torch.Tensor:
        """Residual stream after the last layer, before the final norm: [T, hidden]. ``lora`` is a
        :class:`modular_b200.pipelines.lora.LoRABatch`; its per-module deltas are added to the base outputs."""
        c = self.cfg
        if lora is not None and not lora.active:
            lora = None
        if lora is not None:
            if c.norm_after or c.plain_layer_norm or c.clip_qkv or c.sandwich_norm:
                raise ValueError("LoRA adapters are not implemented for the OLMo and Gemma layer variants")
            return self._forward_hidden_lora(tokens, positions, slots, block_table, q_start, q_len, kv_len, plan,
                                             self.kv if kv is None else kv, lora)
        kv = self.kv if kv is None else kv
        if c.sandwich_norm:
            return self._forward_hidden_gemma(tokens, positions, slots, block_table, q_start, q_len, kv_len, plan, kv)
        if c.norm_after or c.plain_layer_norm or c.clip_qkv:
            return self._forward_hidden_olmo(tokens, positions, slots, block_table, q_start, q_len, kv_len, plan, kv)
        h = ops.embedding(tokens, self.w.embed)
        for li, l in enumerate(self.w.layers):
            kc, vc = kv[:, 0, li], kv[:, 1, li]
            x = ops.rms_norm(h, l.attn_norm, c.rms_norm_eps)
            if l.is_fp8:
                # block-scaled fp8 projections: activations quantised per token group in front of every GEMM
                qkv = ops.linear_fp8(x, l.wqkv, l.wqkv_s)
                if l.qkv_bias is not None:
                    qkv += l.qkv_bias
                self._qk_norm(qkv, l)
                ops.rope_kv_store(qkv, positions, slots, self.cos_sin, kc, vc, c.num_attention_heads,
                                  c.num_key_value_heads, c.head_dim, False)
                a = ops.paged_attention(qkv, kc, vc, block_table, q_start, q_len, kv_len, c.num_attention_heads,
                                        c.num_key_value_heads, c.head_dim, self.scale, plan=plan)
                h = ops.linear_fp8(a, l.wo, l.wo_s, residual=h)
                x = ops.rms_norm(h, l.mlp_norm, c.rms_norm_eps)
                act = ops.silu_mul(ops.linear_fp8(x, l.wgu, l.wgu_s))
                h = ops.linear_fp8(act, l.wd, l.wd_s, residual=h)
                continue
            qkv = ops.linear(x, l.wqkv)
            if l.qkv_bias is not None:
                qkv += l.qkv_bias
            self._qk_norm(qkv, l)
            ops.rope_kv_store(qkv, positions, slots, self.cos_sin, kc, vc, c.num_attention_heads,
                              c.num_key_value_heads, c.head_dim, False)
            a = ops.paged_attention(qkv, kc, vc, block_table, q_start, q_len, kv_len,
                                    c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                                    self.scale, plan=plan)
            h = ops.linear(a, l.wo, residual=h)
            x = ops.rms_norm(h, l.mlp_norm, c.rms_norm_eps)
            if l.moe is not None:
                h = h + l.moe(x)
                continue
            if self.fuse_swiglu:
                act = ops.linear_swiglu(x, l.wgu)
            else:
                act = ops.silu_mul(ops.linear(x, l.wgu))
            h = ops.linear(act, l.wd, residual=h)
        return h

    def _norm(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """The model's norm: RMSNorm with weight ``w``, or (OLMo) a LayerNorm without parameters, computed in fp32."""
        if self.cfg.plain_layer_norm:
            return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), None, None, 1e-5).to(x.dtype)
        return ops.rms_norm(x, w, self.cfg.rms_norm_eps)

    def _forward_hidden_olmo(self, tokens, positions, slots, block_table, q_start, q_len, kv_len, plan, kv):
        """The OLMo layer variants, op by op. OLMo: input norms without parameters and clamped projections.
        OLMo 2 / 3: no input norms, ``h += norm(attn(h)); h += norm(mlp(h))`` with the norms on the block outputs.
        Reference: max/python/max/pipelines/architectures/olmo/, olmo2/."""
        c = self.cfg
        h = ops.embedding(tokens, self.w.embed)
        for li, l in enumerate(self.w.layers):
            if l.is_fp8 or l.moe is not None or l.qkv_bias is not None:
                raise ValueError("the OLMo layer variants are implemented for dense bf16 / fp32 weights without bias")
            kc, vc = kv[:, 0, li], kv[:, 1, li]
            x = h if c.norm_after else self._norm(h, l.attn_norm)
            qkv = ops.linear(x, l.wqkv)
            if c.clip_qkv:
                qkv.clamp_(-c.clip_qkv, c.clip_qkv)
            self._qk_norm(qkv, l)
            ops.rope_kv_store(qkv, positions, slots, self.cos_sin, kc, vc, c.num_attention_heads,
                              c.num_key_value_heads, c.head_dim, False)
            a = ops.paged_attention(qkv, kc, vc, block_table, q_start, q_len, kv_len, c.num_attention_heads,
                                    c.num_key_value_heads, c.head_dim, self.scale, plan=plan)
            if c.norm_after:
                h = h + self._norm(ops.linear(a, l.wo), l.attn_norm)
                x = h
            else:
                h = ops.linear(a, l.wo, residual=h)
                x = self._norm(h, l.mlp_norm)
            act = ops.linear_swiglu(x, l.wgu) if self.fuse_swiglu else ops.silu_mul(ops.linear(x, l.wgu))
            if c.norm_after:
                h = h + self._norm(ops.linear(act, l.wd), l.mlp_norm)
            else:
                h = ops.linear(act, l.wd, residual=h)
        return h

    def _forward_hidden_gemma(self, tokens, positions, slots, block_table, q_start, q_len, kv_len, plan, kv):
        """Gemma 3 text layers, op by op: ``h += norm(attn(norm(h))); h += norm(mlp(norm(h)))`` with a tanh-GELU
        gate in the MLP, per-head query / key norms, and a rotary base of their own on the sliding-window layers.
        The checkpoint's ``w - 1`` norm weights and the ``sqrt(hidden)`` embedding scale were folded in at load.
        Reference: max/python/max/pipelines/architectures/gemma3/."""
        c = self.cfg
        I = c.intermediate_size
        h = ops.embedding(tokens, self.w.embed)
        for li, l in enumerate(self.w.layers):
            if l.is_fp8 or l.moe is not None or l.qkv_bias is not None:
                raise ValueError("Gemma layers are implemented for dense bf16 / fp32 weights without bias")
            kc, vc = kv[:, 0, li], kv[:, 1, li]
            cos_sin = self.cos_sin_local if (li in c.local_layers and self.cos_sin_local is not None) else self.cos_sin
            qkv = ops.linear(ops.rms_norm(h, l.attn_norm, c.rms_norm_eps), l.wqkv)
            self._qk_norm(qkv, l)
            ops.rope_kv_store(qkv, positions, slots, cos_sin, kc, vc, c.num_attention_heads, c.num_key_value_heads,
                              c.head_dim, False)
            a = ops.paged_attention(qkv, kc, vc, block_table, q_start, q_len, kv_len, c.num_attention_heads,
                                    c.num_key_value_heads, c.head_dim, self.scale, plan=plan)
            h = h + ops.rms_norm(ops.linear(a, l.wo), l.attn_out_norm, c.rms_norm_eps)
            gu = ops.linear(ops.rms_norm(h, l.mlp_norm, c.rms_norm_eps), l.wgu)
            act = torch.nn.functional.gelu(gu[:, :I], approximate="tanh") * gu[:, I:]
            h = h + ops.rms_norm(ops.linear(act.contiguous(), l.wd), l.mlp_out_norm, c.rms_norm_eps)
        return h

    def _qk_norm(self, qkv: torch.Tensor, l) -> None:
        """RMSNorm of the queries and keys of a fused projection, in place: per head (Qwen3) or over the whole
        projection (OLMo 2)."""
        if l.q_norm is None:
            return
        c = self.cfg
        if c.qk_norm_full:
            qd, kd = c.q_dim, c.kv_dim
            qkv[:, :qd] = ops.rms_norm(qkv[:, :qd].contiguous(), l.q_norm, c.rms_norm_eps)
            qkv[:, qd:qd + kd] = ops.rms_norm(qkv[:, qd:qd + kd].contiguous(), l.k_norm, c.rms_norm_eps)
            return
        ops.qk_norm(qkv, l.q_norm, l.k_norm, c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.rms_norm_eps)

    def _forward_hidden_lora(self, tokens, positions, slots, block_table, q_start, q_len, kv_len, plan, kv, lora):
        """Same network with LoRA deltas on the seven projection modules (separate gate/up products so the
        deltas enter before the activation)."""
        c = self.cfg
        I = c.intermediate_size

        def add(y, delta, lo=None, hi=None):
            if delta is not None:
                if lo is None:
                    y += delta
                else:
                    y[:, lo:hi] += delta
            return y

        h = ops.embedding(tokens, self.w.embed)
        for li, l in enumerate(self.w.layers):
            kc, vc = kv[:, 0, li], kv[:, 1, li]
            x = ops.rms_norm(h, l.attn_norm, c.rms_norm_eps)
            qkv = ops.linear(x, l.wqkv)
            if l.qkv_bias is not None:
                qkv += l.qkv_bias
            self._qk_norm(qkv, l)
            add(qkv, lora.delta(li, "q_proj", x), 0, c.q_dim)
            add(qkv, lora.delta(li, "k_proj", x), c.q_dim, c.q_dim + c.kv_dim)
            add(qkv, lora.delta(li, "v_proj", x), c.q_dim + c.kv_dim, c.q_dim + 2 * c.kv_dim)
            ops.rope_kv_store(qkv, positions, slots, self.cos_sin, kc, vc, c.num_attention_heads,
                              c.num_key_value_heads, c.head_dim, False)
            a = ops.paged_attention(qkv, kc, vc, block_table, q_start, q_len, kv_len, c.num_attention_heads,
                                    c.num_key_value_heads, c.head_dim, self.scale, plan=plan)
            h = add(ops.linear(a, l.wo, residual=h), lora.delta(li, "o_proj", a))
            x = ops.rms_norm(h, l.mlp_norm, c.rms_norm_eps)
            gu = ops.linear(x, l.wgu)
            add(gu, lora.delta(li, "gate_proj", x), 0, I)
            add(gu, lora.delta(li, "up_proj", x), I, 2 * I)
            act = ops.silu_mul(gu)
            h = add(ops.linear(act, l.wd, residual=h), lora.delta(li, "down_proj", act))
        return h

    def encode(self, token_lists, pooling: str = "last", normalize: bool = True) -> torch.Tensor:
        """Sentence embeddings: run the prompts as one ragged prefill over a private scratch cache and
        pool the final-normed hidden states (``last`` token or ``mean``). Returns fp32 [n, hidden].
        Reference: max/python/max/pipelines/lib/embeddings_pipeline.py."""
        c, dev, page = self.cfg, self.device, self.page_size
        lens = [len(t) for t in token_lists]
        if not lens or min(lens) < 1:
            raise ValueError("encode needs non-empty token lists")
        pages_per = [(n + page - 1) // page for n in lens]
        kv = torch.zeros(sum(pages_per) + 1, 2, c.num_hidden_layers, c.num_key_value_heads, page, c.head_dim,
                         dtype=self.dtype, device=dev)
        bt = torch.zeros(len(lens), max(pages_per), dtype=torch.int32)
        slots, positions, nxt = [], [], 1
        for i, (n, pp) in enumerate(zip(lens, pages_per)):
            bt[i, :pp] = torch.arange(nxt, nxt + pp)
            slots.append(torch.arange(n) + nxt * page)
            positions.append(torch.arange(n))
            nxt += pp
        q_len = torch.tensor(lens, dtype=torch.int32)
        q_start = torch.cumsum(q_len, 0, dtype=torch.int32) - q_len
        tokens = torch.tensor([t for tl in token_lists for t in tl], dtype=torch.long, device=dev)
        h = self.forward_hidden(tokens, torch.cat(positions).int().to(dev), torch.cat(slots).to(dev), bt.to(dev),
                                q_start.to(dev), q_len.to(dev), q_len.to(dev), kv=kv)
        hn = self._norm(h, self.w.final_norm).float()
        out = torch.empty(len(lens), c.hidden_size, dtype=torch.float32, device=dev)
        for i, (s0, n) in enumerate(zip(q_start.tolist(), lens)):
            out[i] = hn[s0 + n - 1] if pooling == "last" else hn[s0:s0 + n].mean(0)
        if normalize:
            out = out / out.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        return out
