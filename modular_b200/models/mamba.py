"""Mamba (``MambaForCausalLM``): a stack of selective state-space blocks, no attention and no KV cache.

Each layer is ``h += mixer(rms_norm(h))`` with the Mamba-1 mixer of :mod:`modular_b200.nn.state_space` (causal
depthwise conv1d and selective scan kernels on CUDA in bf16, their PyTorch forms elsewhere). What a request carries
from step to step is a fixed-size state per layer - the last ``conv_kernel - 1`` inputs of the convolution and the
``[d_inner, state_size]`` scan state - instead of keys and values that grow with the sequence.

The engine's schedulers, chunked prefill and preemption work on pages of a paged cache, so the family keeps a
token-sized dummy cache for that bookkeeping and stores the real state in slots indexed by the FIRST page of a
request: pages are exclusive to a request while prefix caching is off (the family turns it off - a state cannot be
shared by prefix the way KV pages can), and a request whose step starts at position 0 starts from a zero state, which
is also what a preempted request does when it is recomputed.

Reference: max/python/max/pipelines/architectures/mamba/ (model and state cache) over max/python/max/nn/state_space/.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..nn.state_space import MambaMixer

STATE_PAGE_TOKENS = 2048      # tokens per bookkeeping page: bounds the number of pages, and with it the state slots


@dataclass
class MambaConfig:
    hidden_size: int = 768
    state_size: int = 16
    num_hidden_layers: int = 24
    vocab_size: int = 50280
    expand: int = 2
    conv_kernel: int = 4
    time_step_rank: Optional[int] = None          # None = ceil(hidden_size / 16)
    intermediate_size: Optional[int] = None       # None = expand * hidden_size
    layer_norm_epsilon: float = 1e-5
    tie_word_embeddings: bool = True
    max_position_embeddings: int = 1 << 20         # no positional limit; the engine's max_length bounds a request
    architectures: tuple = ("MambaForCausalLM",)
    # the batch packer plans attention work per head group; there is none here
    num_attention_heads: int = 1
    num_key_value_heads: int = 1

    def __post_init__(self):
        if self.intermediate_size is None:
            self.intermediate_size = self.expand * self.hidden_size
        if self.time_step_rank in (None, "auto"):
            self.time_step_rank = math.ceil(self.hidden_size / 16)

    @classmethod
    def from_hf(cls, d: dict) -> "MambaConfig":
        if d.get("use_bias"):
            raise ValueError("biases on the in / out projections are not implemented")
        if d.get("use_conv_bias") is False:
            raise ValueError("a convolution without bias is not implemented")
        if (d.get("hidden_act") or "silu") != "silu":
            raise ValueError(f"activation {d.get('hidden_act')!r} is not implemented")
        keys = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in d.items() if k in keys and k != "max_position_embeddings"}
        if "architectures" in kw:
            kw["architectures"] = tuple(kw["architectures"])
        return cls(**kw)

    def to_hf(self) -> dict:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d.pop("num_attention_heads"), d.pop("num_key_value_heads"), d.pop("max_position_embeddings")
        d.update(architectures=list(self.architectures), model_type="mamba", use_bias=False, use_conv_bias=True,
                 hidden_act="silu")
        return d

    @classmethod
    def tiny(cls, **kw) -> "MambaConfig":
        base = dict(hidden_size=256, num_hidden_layers=2, vocab_size=4096, state_size=16)
        base.update(kw)
        return cls(**base)

    @classmethod
    def mamba_130m(cls) -> "MambaConfig":
        return cls()

    @classmethod
    def mamba_2_8b(cls) -> "MambaConfig":
        return cls(hidden_size=2560, num_hidden_layers=64)

    def param_count(self) -> int:
        H, D, N, R, W = self.hidden_size, self.intermediate_size, self.state_size, self.time_step_rank, self.conv_kernel
        per_layer = H + H * 2 * D + D * W + D + D * (R + 2 * N) + R * D + D + D * N + D + D * H
        head = 0 if self.tie_word_embeddings else self.vocab_size * H
        return self.vocab_size * H + self.num_hidden_layers * per_layer + H + head

    def state_bytes_per_slot(self) -> int:
        return self.num_hidden_layers * self.intermediate_size * (self.conv_kernel - 1 + self.state_size) * 4


@dataclass
class MambaLayerWeights:
    norm: torch.Tensor
    mixer: MambaMixer


@dataclass
class MambaWeights:
    embed: torch.Tensor
    layers: list
    final_norm: torch.Tensor
    lm_head: torch.Tensor

    @staticmethod
    def _mixer(cfg: MambaConfig, dtype, dev) -> MambaMixer:
        return MambaMixer(cfg.hidden_size, cfg.intermediate_size, cfg.state_size, cfg.conv_kernel, cfg.time_step_rank,
                          dtype=dtype, device=dev)

    @classmethod
    def random_init(cls, cfg: MambaConfig, device="cpu", dtype=torch.bfloat16, seed: int = 0, std: float = 0.02):
        g = torch.Generator(device="cpu").manual_seed(seed)
        dev = torch.device(device)
        rnd = lambda *shape, s=std: (torch.randn(*shape, generator=g) * s).to(dtype).to(dev)
        layers = []
        for _ in range(cfg.num_hidden_layers):
            m = cls._mixer(cfg, dtype, dev)
            with torch.no_grad():
                m.in_proj.weight.copy_(rnd(*m.in_proj.weight.shape))
                m.x_proj.weight.copy_(rnd(*m.x_proj.weight.shape))
                m.dt_proj.weight.copy_(rnd(*m.dt_proj.weight.shape, s=cfg.time_step_rank ** -0.5))
                # time steps in [1e-3, 1e-1] after the softplus, as the published checkpoints are initialised
                dt = torch.exp(torch.rand(cfg.intermediate_size, generator=g) * (math.log(0.1) - math.log(1e-3))
                               + math.log(1e-3))
                m.dt_proj.bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(dtype))
                m.out_proj.weight.copy_(rnd(*m.out_proj.weight.shape))
                m.conv_w.copy_(rnd(*m.conv_w.shape, s=0.2))
            layers.append(MambaLayerWeights(torch.ones(cfg.hidden_size, dtype=dtype, device=dev), m))
        embed = rnd(cfg.vocab_size, cfg.hidden_size)
        lm_head = embed if cfg.tie_word_embeddings else rnd(cfg.vocab_size, cfg.hidden_size)
        return cls(embed, layers, torch.ones(cfg.hidden_size, dtype=dtype, device=dev), lm_head)

    @classmethod
    def from_state_dict(cls, cfg: MambaConfig, sd: dict, device="cpu", dtype=torch.bfloat16):
        """Hugging Face ``MambaForCausalLM`` tensors (``backbone.*``; ``lm_head.weight`` absent when tied)."""
        dev = torch.device(device)
        sd = {(k[len("backbone."):] if k.startswith("backbone.") else k): v for k, v in sd.items()}
        get = lambda n: sd[n].to(device=dev, dtype=dtype).contiguous()
        f32 = lambda n: sd[n].to(device=dev, dtype=torch.float32).contiguous()
        layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}.mixer."
            if p + "in_proj.bias" in sd or p + "out_proj.bias" in sd:
                raise ValueError("biases on the in / out projections are not implemented")
            m = cls._mixer(cfg, dtype, dev)
            with torch.no_grad():
                m.in_proj.weight.copy_(get(p + "in_proj.weight"))
                m.conv_w.copy_(get(p + "conv1d.weight").reshape(cfg.intermediate_size, cfg.conv_kernel))
                m.conv_b.copy_(get(p + "conv1d.bias"))
                m.x_proj.weight.copy_(get(p + "x_proj.weight"))
                m.dt_proj.weight.copy_(get(p + "dt_proj.weight"))
                m.dt_proj.bias.copy_(get(p + "dt_proj.bias"))
                m.A_log.copy_(f32(p + "A_log"))
                m.D.copy_(f32(p + "D"))
                m.out_proj.weight.copy_(get(p + "out_proj.weight"))
            layers.append(MambaLayerWeights(get(f"layers.{i}.norm.weight"), m))
        embed = get("embeddings.weight")
        lm_head = embed if (cfg.tie_word_embeddings or "lm_head.weight" not in sd) else get("lm_head.weight")
        return cls(embed, layers, get("norm_f.weight"), lm_head)

    def to_hf_state_dict(self, cfg: MambaConfig) -> dict:
        sd = {"backbone.embeddings.weight": self.embed, "backbone.norm_f.weight": self.final_norm}
        if not cfg.tie_word_embeddings:
            sd["lm_head.weight"] = self.lm_head
        for i, l in enumerate(self.layers):
            p, m = f"backbone.layers.{i}.mixer.", l.mixer
            sd[f"backbone.layers.{i}.norm.weight"] = l.norm
            sd.update({p + "in_proj.weight": m.in_proj.weight, p + "conv1d.weight": m.conv_w.unsqueeze(1),
                       p + "conv1d.bias": m.conv_b, p + "x_proj.weight": m.x_proj.weight,
                       p + "dt_proj.weight": m.dt_proj.weight, p + "dt_proj.bias": m.dt_proj.bias,
                       p + "A_log": m.A_log, p + "D": m.D, p + "out_proj.weight": m.out_proj.weight})
        return {k: v.detach().contiguous() for k, v in sd.items()}


class MambaModel:
    """Serves :class:`MambaConfig` behind the engine's model interface (``forward_tensors``; no step executor and
    no CUDA graphs: every step is launched op by op)."""

    use_executor = False
    executor = None
    logits_buf = None

    def __init__(self, cfg: MambaConfig, weights: MambaWeights, kv_cache: torch.Tensor, max_tokens: int = 8192,
                 max_seqs: int = 256, max_position: Optional[int] = None):
        self.cfg, self.w, self.kv = cfg, weights, kv_cache
        self.device, self.dtype = weights.embed.device, weights.embed.dtype
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.page_size = kv_cache.shape[4]
        slots = kv_cache.shape[0]
        need = slots * cfg.state_bytes_per_slot()
        if self.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.device)
            if need > free:
                raise ValueError(f"the recurrent state of {slots} request slots takes {need >> 20} MiB, more than "
                                 f"the {free >> 20} MiB that are free: lower max_batch_size or pass num_kv_pages")
        # one (conv, scan) state per layer and first-page id
        self.state = [l.mixer.alloc_state(slots, self.device) for l in weights.layers]

    @torch.no_grad()
    def forward_hidden(self, tokens, block_table, q_start, q_len, kv_len) -> torch.Tensor:
        c = self.cfg
        n = q_len.shape[0]
        cu = torch.zeros(n + 1, dtype=torch.int32, device=self.device)
        cu[1:] = torch.cumsum(q_len, 0)
        state_idx = block_table[:, 0].to(torch.int32).contiguous()
        has_init = (kv_len > q_len).to(torch.int32)       # something of this request was processed before this step
        h = ops.embedding(tokens, self.w.embed)
        for l, st in zip(self.w.layers, self.state):
            x = ops.rms_norm(h, l.norm, c.layer_norm_epsilon)
            h = h + l.mixer(x, cu, st, state_idx, has_init)
        return h

    @torch.no_grad()
    def forward_tensors(self, tokens, positions, slots, block_table, q_start, q_len, kv_len, logit_rows,
                        **unused) -> torch.Tensor:
        """Logits [n_logit_rows, vocab] of a ragged step. ``positions`` and ``slots`` address a KV cache and are not
        used: the order of the tokens inside each sequence is all the recurrence needs."""
        if unused.get("lora") is not None:
            raise ValueError("LoRA adapters are not implemented for state-space layers")
        h = self.forward_hidden(tokens, block_table, q_start, q_len, kv_len)
        last = h.index_select(0, logit_rows.long())
        xn = ops.rms_norm(last, self.w.final_norm, self.cfg.layer_norm_epsilon)
        return ops.linear(xn, self.w.lm_head, out_dtype=torch.float32)
