"""LFM2 (``Lfm2ForCausalLM``): a hybrid decoder - most layers are gated short convolutions, a few are grouped-query
attention layers with per-head query / key RMSNorm and rotary positions; every layer ends in a SwiGLU MLP.

A convolution layer computes ``out_proj(C * causal_conv1d(B * x))`` with ``B, C, x = in_proj(h)``: a depthwise
convolution over the last ``conv_L_cache`` tokens, so what it carries between steps is ``conv_L_cache - 1`` inputs per
channel. The attention layers use the engine's paged KV cache (one cache layer per attention layer); the convolution
tails live in slots indexed by a request's first page, which is exclusive to it because the family turns prefix
caching off (a cached prefix restores keys and values, not convolution tails). A step that starts at position 0
starts from an empty tail. Runs op by op on the GEMM, norm, rotary, attention and conv1d kernels.

Reference: max/python/max/pipelines/architectures/lfm2/.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..nn.rotary_embedding import RopeScaling, cos_sin_table
from ..nn.state_space import causal_conv1d_varlen


@dataclass
class Lfm2Config:
    hidden_size: int = 2048
    intermediate_size: int = 8192          # width of the SwiGLU MLP as it is in the weights
    num_hidden_layers: int = 16
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    vocab_size: int = 65536
    norm_eps: float = 1e-5
    rope_theta: float = 1000000.0
    rope_scaling: Optional[dict] = None
    max_position_embeddings: int = 128000
    conv_L_cache: int = 3
    conv_bias: bool = False
    layer_types: tuple = ()                # "conv" | "full_attention" per layer
    tie_word_embeddings: bool = True
    architectures: tuple = ("Lfm2ForCausalLM",)

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = tuple("full_attention" if i % 3 == 2 else "conv" for i in range(self.num_hidden_layers))
        self.layer_types = tuple(self.layer_types)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def attention_layers(self) -> tuple:
        return tuple(i for i, t in enumerate(self.layer_types) if t == "full_attention")

    @classmethod
    def from_hf(cls, d: dict) -> "Lfm2Config":
        from ..pipelines.weights import normalize_hf_rope

        d = normalize_hf_rope(d)
        keys = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in d.items() if k in keys and v is not None}
        kw["norm_eps"] = d.get("norm_eps", d.get("block_norm_eps", 1e-5))
        if "architectures" in kw:
            kw["architectures"] = tuple(kw["architectures"])
        if "layer_types" not in kw and d.get("full_attn_idxs") is not None:
            full = set(d["full_attn_idxs"])
            kw["layer_types"] = tuple("full_attention" if i in full else "conv" for i in range(d["num_hidden_layers"]))
        ff = int(d.get("intermediate_size", d.get("block_ff_dim", 0)))
        if d.get("block_auto_adjust_ff_dim", False):
            # the checkpoint's MLP is two thirds of the nominal width, scaled and rounded up to a block multiple
            ff = int(2 * ff / 3)
            if d.get("block_ffn_dim_multiplier"):
                ff = int(d["block_ffn_dim_multiplier"] * ff)
            m = int(d.get("block_multiple_of", 256))
            ff = m * ((ff + m - 1) // m)
        kw["intermediate_size"] = ff
        return cls(**kw)

    def to_hf(self) -> dict:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d.update(architectures=list(self.architectures), layer_types=list(self.layer_types), model_type="lfm2",
                 block_auto_adjust_ff_dim=False)
        return d

    @classmethod
    def tiny(cls, **kw) -> "Lfm2Config":
        base = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=4, num_attention_heads=4,
                    num_key_value_heads=2, vocab_size=4096, max_position_embeddings=2048,
                    layer_types=("conv", "conv", "full_attention", "conv"))
        base.update(kw)
        return cls(**base)

    def param_count(self) -> int:
        H, I, hd = self.hidden_size, self.intermediate_size, self.head_dim
        attn = H * hd * (2 * self.num_attention_heads + 2 * self.num_key_value_heads) + 2 * hd
        conv = 4 * H * H + H * self.conv_L_cache
        n_attn = len(self.attention_layers)
        return (self.vocab_size * H * (1 if self.tie_word_embeddings else 2) + H
                + self.num_hidden_layers * (3 * H * I + 2 * H) + n_attn * attn + (self.num_hidden_layers - n_attn) * conv)

    def state_bytes_per_slot(self) -> int:
        return (self.num_hidden_layers - len(self.attention_layers)) * self.hidden_size * (self.conv_L_cache - 1) * 4


@dataclass
class Lfm2LayerWeights:
    op_norm: torch.Tensor
    ffn_norm: torch.Tensor
    wgu: torch.Tensor                       # [2I, H]: gate (w1) over up (w3)
    wd: torch.Tensor                        # [H, I]  (w2)
    # attention layers
    wqkv: Optional[torch.Tensor] = None
    wo: Optional[torch.Tensor] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    # convolution layers
    w_in: Optional[torch.Tensor] = None     # [3H, H] -> B, C, x
    b_in: Optional[torch.Tensor] = None
    conv_w: Optional[torch.Tensor] = None   # [H, L]
    conv_b: Optional[torch.Tensor] = None
    w_out: Optional[torch.Tensor] = None
    b_out: Optional[torch.Tensor] = None


@dataclass
class Lfm2Weights:
    embed: torch.Tensor
    layers: list
    final_norm: torch.Tensor
    lm_head: torch.Tensor

    @classmethod
    def random_init(cls, cfg: Lfm2Config, device="cpu", dtype=torch.bfloat16, seed: int = 0, std: float = 0.02):
        g = torch.Generator(device="cpu").manual_seed(seed)
        dev = torch.device(device)
        rnd = lambda *s, sc=std: (torch.randn(*s, generator=g) * sc).to(dtype).to(dev)
        one = lambda n: torch.ones(n, dtype=dtype, device=dev)
        H, I, hd = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
        layers = []
        for t in cfg.layer_types:
            l = Lfm2LayerWeights(one(H), one(H), rnd(2 * I, H), rnd(H, I))
            if t == "full_attention":
                l.wqkv = rnd((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * hd, H)
                l.wo, l.q_norm, l.k_norm = rnd(H, cfg.num_attention_heads * hd), one(hd), one(hd)
            else:
                l.w_in, l.conv_w, l.w_out = rnd(3 * H, H), rnd(H, cfg.conv_L_cache, sc=0.3), rnd(H, H)
                if cfg.conv_bias:
                    l.b_in, l.conv_b, l.b_out = rnd(3 * H), rnd(H), rnd(H)
            layers.append(l)
        embed = rnd(cfg.vocab_size, H)
        return cls(embed, layers, one(H), embed if cfg.tie_word_embeddings else rnd(cfg.vocab_size, H))

    @classmethod
    def from_state_dict(cls, cfg: Lfm2Config, sd: dict, device="cpu", dtype=torch.bfloat16):
        dev = torch.device(device)
        sd = {(k[len("model."):] if k.startswith("model.") else k): v for k, v in sd.items()}
        get = lambda n: sd[n].to(device=dev, dtype=dtype).contiguous()
        opt = lambda n: get(n) if n in sd else None
        cat = lambda names: torch.cat([sd[n] for n in names], 0).to(device=dev, dtype=dtype).contiguous()
        layers = []
        for i, t in enumerate(cfg.layer_types):
            p = f"layers.{i}."
            l = Lfm2LayerWeights(get(p + "operator_norm.weight"), get(p + "ffn_norm.weight"),
                                 cat([p + "feed_forward.w1.weight", p + "feed_forward.w3.weight"]),
                                 get(p + "feed_forward.w2.weight"))
            if l.wd.shape[1] != cfg.intermediate_size:
                raise ValueError(f"MLP width {l.wd.shape[1]} in the weights, {cfg.intermediate_size} in the config")
            if t == "full_attention":
                a = p + "self_attn."
                l.wqkv = cat([a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight"])
                l.wo, l.q_norm, l.k_norm = get(a + "out_proj.weight"), get(a + "q_layernorm.weight"), get(a + "k_layernorm.weight")
            else:
                c = p + "conv."
                l.w_in, l.b_in = get(c + "in_proj.weight"), opt(c + "in_proj.bias")
                l.conv_w = get(c + "conv.weight").reshape(cfg.hidden_size, cfg.conv_L_cache)
                l.conv_b = opt(c + "conv.bias")
                l.w_out, l.b_out = get(c + "out_proj.weight"), opt(c + "out_proj.bias")
            layers.append(l)
        embed = get("embed_tokens.weight")
        lm_head = embed if (cfg.tie_word_embeddings or "lm_head.weight" not in sd) else get("lm_head.weight")
        return cls(embed, layers, get("embedding_norm.weight"), lm_head)


class Lfm2Model:
    """Serves :class:`Lfm2Config` behind the engine's model interface (``forward_tensors``, op by op)."""

    use_executor = False
    executor = None
    logits_buf = None

    def __init__(self, cfg: Lfm2Config, weights: Lfm2Weights, kv_cache: torch.Tensor, max_tokens: int = 8192,
                 max_seqs: int = 256, max_position: Optional[int] = None):
        self.cfg, self.w, self.kv = cfg, weights, kv_cache
        self.device, self.dtype = weights.embed.device, weights.embed.dtype
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.page_size = kv_cache.shape[4]
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self.cos_sin = cos_sin_table(cfg.head_dim, max_position or cfg.max_position_embeddings, cfg.rope_theta,
                                     RopeScaling.from_hf(cfg.rope_scaling), self.device)
        self.kv_layer = {li: j for j, li in enumerate(cfg.attention_layers)}      # layer -> plane of the KV cache
        slots, width = kv_cache.shape[0], cfg.conv_L_cache - 1
        # convolution tails, one slot per first-page id: fp32 [slots, hidden, L - 1] per convolution layer
        self.conv_state = {li: torch.zeros(slots, cfg.hidden_size, width, dtype=torch.float32, device=self.device)
                           for li, t in enumerate(cfg.layer_types) if t != "full_attention"}

    @torch.no_grad()
    def forward_hidden(self, tokens, positions, slots, block_table, q_start, q_len, kv_len, plan=None) -> torch.Tensor:
        c, H = self.cfg, self.cfg.hidden_size
        cu = torch.zeros(q_len.shape[0] + 1, dtype=torch.int32, device=self.device)
        cu[1:] = torch.cumsum(q_len, 0)
        state_idx = block_table[:, 0].to(torch.int32).contiguous()
        has_init = (kv_len > q_len).to(torch.int32)
        h = ops.embedding(tokens, self.w.embed)
        for li, l in enumerate(self.w.layers):
            x = ops.rms_norm(h, l.op_norm, c.norm_eps)
            if l.wqkv is not None:
                j = self.kv_layer[li]
                kc, vc = self.kv[:, 0, j], self.kv[:, 1, j]
                qkv = ops.linear(x, l.wqkv)
                ops.qk_norm(qkv, l.q_norm, l.k_norm, c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.norm_eps)
                ops.rope_kv_store(qkv, positions, slots, self.cos_sin, kc, vc, c.num_attention_heads,
                                  c.num_key_value_heads, c.head_dim, False)
                a = ops.paged_attention(qkv, kc, vc, block_table, q_start, q_len, kv_len, c.num_attention_heads,
                                        c.num_key_value_heads, c.head_dim, self.scale, plan=plan)
                h = ops.linear(a, l.wo, residual=h)
            else:
                bcx = ops.linear(x, l.w_in)
                if l.b_in is not None:
                    bcx = bcx + l.b_in
                gated = (bcx[:, :H] * bcx[:, 2 * H:]).contiguous()
                bias = l.conv_b if l.conv_b is not None else torch.zeros(H, dtype=gated.dtype, device=self.device)
                y = causal_conv1d_varlen(gated, l.conv_w, bias, cu, self.conv_state[li], state_idx, has_init, silu=False)
                y = (bcx[:, H: 2 * H] * y).contiguous()
                h = ops.linear(y, l.w_out, residual=h)
                if l.b_out is not None:
                    h = h + l.b_out
            x = ops.rms_norm(h, l.ffn_norm, c.norm_eps)
            h = ops.linear(ops.silu_mul(ops.linear(x, l.wgu)), l.wd, residual=h)
        return h

    @torch.no_grad()
    def forward_tensors(self, tokens, positions, slots, block_table, q_start, q_len, kv_len, logit_rows, plan=None,
                        lora=None) -> torch.Tensor:
        """fp32 logits [len(logit_rows), vocab] of a ragged step."""
        if lora is not None:
            raise ValueError("LoRA adapters are not implemented for this family")
        h = self.forward_hidden(tokens, positions, slots, block_table, q_start, q_len, kv_len, plan)
        xn = ops.rms_norm(h.index_select(0, logit_rows.long()), self.w.final_norm, self.cfg.norm_eps)
        return ops.linear(xn, self.w.lm_head, out_dtype=torch.float32).float()
