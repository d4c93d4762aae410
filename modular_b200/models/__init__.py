"""Model families. A family bundles what the engine needs to serve an architecture: config,
weights and model classes, the KV-cache geometry and an activation-memory estimate.

Reference: max/python/max/pipelines/architectures/__init__.py (one ``SupportedArchitecture`` per
model directory) and lib/arch_lookup.py:70.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch


@dataclass
class ModelFamily:
    name: str
    config_class: Any
    weights_class: Any
    model_class: Any
    kv_params: Callable        # (cfg, page_size, dtype, prefix_caching) -> KVCacheParams
    activation_bytes: Callable  # (cfg, max_tokens, max_seqs) -> int
    supports_tp: bool = False
    supports_ep: bool = False       # expert parallelism: routed experts sharded, every rank serves its own requests


def _llama_family() -> ModelFamily:
    from ..kv_cache import KVCacheParams
    from .llama3 import Llama3Config, Llama3Model, Llama3Weights

    def kv(cfg, page, dtype, prefix):
        return KVCacheParams(cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.head_dim, page, dtype, False, prefix)

    def act(cfg, T, B):
        return (T * (3 * cfg.hidden_size + 2 * cfg.q_dim + 3 * cfg.intermediate_size) * 2
                + B * cfg.vocab_size * 4 + (256 << 20))

    return ModelFamily("llama", Llama3Config, Llama3Weights, Llama3Model, kv, act, supports_tp=True)


def _deepseek_family() -> ModelFamily:
    from ..kv_cache import KVCacheParams
    from .deepseek_v3 import DeepseekV3Config, DeepseekV3Model, DeepseekV3Weights

    def kv(cfg, page, dtype, prefix):
        return KVCacheParams(cfg.num_hidden_layers, 1, cfg.latent_dim, page, dtype, True, prefix)

    def act(cfg, T, B):
        h = cfg.num_attention_heads
        per_tok = (4 * cfg.hidden_size + 2 * h * (cfg.qk_head_dim + cfg.kv_lora_rank + cfg.v_head_dim)
                   + 3 * max(cfg.intermediate_size, cfg.num_experts_per_tok * cfg.moe_intermediate_size))
        return T * per_tok * 2 + B * cfg.vocab_size * 4 + (256 << 20)

    return ModelFamily("deepseek_v3", DeepseekV3Config, DeepseekV3Weights, DeepseekV3Model, kv, act, supports_ep=True)


def _mamba_family() -> ModelFamily:
    from ..kv_cache import KVCacheParams
    from .mamba import STATE_PAGE_TOKENS, MambaConfig, MambaModel, MambaWeights

    def kv(cfg, page, dtype, prefix):
        # a bookkeeping cache only (one 8-element row per token): the recurrent state lives in the model, one slot
        # per first page, so pages are large and never shared by prefix
        return KVCacheParams(1, 1, 8, max(page, STATE_PAGE_TOKENS), dtype, True, False)

    def act(cfg, T, B):
        return (T * (2 * cfg.hidden_size + 6 * cfg.intermediate_size) * 4 + B * cfg.vocab_size * 4
                + 4 * B * cfg.state_bytes_per_slot() + (256 << 20))

    return ModelFamily("mamba", MambaConfig, MambaWeights, MambaModel, kv, act)


def _lfm2_family() -> ModelFamily:
    from ..kv_cache import KVCacheParams
    from .lfm2 import Lfm2Config, Lfm2Model, Lfm2Weights

    def kv(cfg, page, dtype, prefix):
        # keys and values for the attention layers only; no prefix sharing (it cannot restore the convolution tails)
        return KVCacheParams(max(len(cfg.attention_layers), 1), cfg.num_key_value_heads, cfg.head_dim, page, dtype,
                             False, False)

    def act(cfg, T, B):
        return (T * (8 * cfg.hidden_size + 3 * cfg.intermediate_size) * 2 + B * cfg.vocab_size * 4
                + 4 * B * cfg.state_bytes_per_slot() + (256 << 20))

    return ModelFamily("lfm2", Lfm2Config, Lfm2Weights, Lfm2Model, kv, act)


def _bert_family() -> ModelFamily:
    from ..kv_cache import KVCacheParams
    from .bert import BertConfig, BertModel, BertWeights

    def kv(cfg, page, dtype, prefix):
        # encoders keep nothing between requests: a token-sized dummy cache for the engine's bookkeeping
        return KVCacheParams(1, 1, 8, page, dtype, True, False)

    def act(cfg, T, B):
        return T * (8 * cfg.hidden_size + 2 * cfg.intermediate_size) * 4 + (256 << 20)

    return ModelFamily("bert", BertConfig, BertWeights, BertModel, kv, act)


def family_for(config) -> ModelFamily:
    """The family that serves `config` (matched on the config class)."""
    for make in (_llama_family, _deepseek_family, _mamba_family, _lfm2_family, _bert_family):
        fam = make()
        if isinstance(config, fam.config_class):
            return fam
    raise TypeError(f"no model family registered for config type {type(config).__name__}")
