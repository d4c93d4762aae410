"""Encoder-only embedding models: BERT (``BertModel``) and MPNet (``MPNetModel`` / ``MPNetForMaskedLM``).

Bidirectional attention over the whole sequence, learned absolute positions, post-LayerNorm blocks with biased
projections and a GELU feed-forward; MPNet adds one table of relative-position biases (log-spaced distance buckets)
shared by all layers and counts positions from its padding index. These models produce sentence embeddings only
(``encode``: CLS, mean or last pooling over the final hidden states); there is nothing to decode, so the engine's
generation entry points refuse them. The layers run on PyTorch operators (library GEMMs and softmax) on whichever
device holds the weights: embedding requests are one forward pass over short sequences, not a serving hot loop.

Reference: max/python/max/pipelines/architectures/bert/, mpnet/ (encoders behind the embeddings pipeline,
max/python/max/pipelines/lib/embeddings_pipeline.py).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    hidden_act: str = "gelu"
    pad_token_id: int = 0
    relative_attention_num_buckets: int = 0       # MPNet: 32; 0 = no relative-position bias (BERT)
    architectures: tuple = ("BertModel",)
    num_key_value_heads: int = 1                  # read by the batch packer; unused

    @property
    def is_mpnet(self) -> bool:
        return self.relative_attention_num_buckets > 0

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @classmethod
    def from_hf(cls, d: dict) -> "BertConfig":
        if d.get("hidden_act", "gelu") not in ("gelu", "gelu_new", "gelu_pytorch_tanh", "relu"):
            raise ValueError(f"activation {d.get('hidden_act')!r} is not implemented")
        if d.get("position_embedding_type", "absolute") != "absolute":
            raise ValueError("only absolute position embeddings are implemented")
        keys = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in d.items() if k in keys}
        if "architectures" in kw:
            kw["architectures"] = tuple(kw["architectures"])
        if d.get("model_type") == "mpnet" or any("MPNet" in a for a in d.get("architectures", ())):
            kw.setdefault("relative_attention_num_buckets", 32)
            kw["type_vocab_size"] = 0
            kw.setdefault("pad_token_id", 1)
            kw.setdefault("layer_norm_eps", 1e-5)
        return cls(**kw)

    def to_hf(self) -> dict:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d.pop("num_key_value_heads")
        d.update(architectures=list(self.architectures), model_type="mpnet" if self.is_mpnet else "bert")
        return d

    @classmethod
    def tiny(cls, **kw) -> "BertConfig":
        base = dict(vocab_size=4096, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                    intermediate_size=256, max_position_embeddings=512)
        base.update(kw)
        return cls(**base)

    def param_count(self) -> int:
        H, I = self.hidden_size, self.intermediate_size
        per_layer = 4 * (H * H + H) + 2 * H * I + I + H + 4 * H
        return (self.vocab_size + self.max_position_embeddings + self.type_vocab_size) * H + 2 * H \
            + self.num_hidden_layers * per_layer + self.relative_attention_num_buckets * self.num_attention_heads


@dataclass
class BertLayerWeights:
    wqkv: torch.Tensor          # [3H, H]
    bqkv: torch.Tensor
    wo: torch.Tensor
    bo: torch.Tensor
    attn_ln: tuple              # (weight, bias)
    w1: torch.Tensor            # [I, H]
    b1: torch.Tensor
    w2: torch.Tensor            # [H, I]
    b2: torch.Tensor
    out_ln: tuple


@dataclass
class BertWeights:
    embed: torch.Tensor
    pos_embed: torch.Tensor
    type_embed: Optional[torch.Tensor]
    embed_ln: tuple
    layers: list
    rel_bias: Optional[torch.Tensor]      # [buckets, heads] (MPNet)

    @classmethod
    def random_init(cls, cfg: BertConfig, device="cpu", dtype=torch.float32, seed: int = 0, std: float = 0.02):
        g = torch.Generator(device="cpu").manual_seed(seed)
        dev = torch.device(device)
        rnd = lambda *s: (torch.randn(*s, generator=g) * std).to(dtype).to(dev)
        ln = lambda: (torch.ones(cfg.hidden_size, dtype=dtype, device=dev), rnd(cfg.hidden_size))
        H, I = cfg.hidden_size, cfg.intermediate_size
        layers = [BertLayerWeights(rnd(3 * H, H), rnd(3 * H), rnd(H, H), rnd(H), ln(), rnd(I, H), rnd(I), rnd(H, I),
                                   rnd(H), ln()) for _ in range(cfg.num_hidden_layers)]
        return cls(rnd(cfg.vocab_size, H), rnd(cfg.max_position_embeddings, H),
                   rnd(cfg.type_vocab_size, H) if cfg.type_vocab_size else None, ln(), layers,
                   rnd(cfg.relative_attention_num_buckets, cfg.num_attention_heads) if cfg.is_mpnet else None)

    @classmethod
    def from_state_dict(cls, cfg: BertConfig, sd: dict, device="cpu", dtype=torch.float32):
        """Hugging Face tensors, with or without the ``bert.`` / ``mpnet.`` prefix; pooler and LM heads are dropped."""
        dev = torch.device(device)
        for pre in ("bert.", "mpnet."):
            if any(k.startswith(pre) for k in sd):
                sd = {(k[len(pre):] if k.startswith(pre) else k): v for k, v in sd.items()}
        get = lambda n: sd[n].to(device=dev, dtype=dtype).contiguous()
        ln = lambda p: (get(p + ".weight"), get(p + ".bias"))
        cat = lambda names: torch.cat([sd[n] for n in names], 0).to(device=dev, dtype=dtype).contiguous()
        layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"encoder.layer.{i}."
            if cfg.is_mpnet:
                a, qkv, o, aln = p + "attention.attn.", ("q", "k", "v"), p + "attention.attn.o", p + "attention.LayerNorm"
            else:
                a, qkv, o, aln = (p + "attention.self.", ("query", "key", "value"), p + "attention.output.dense",
                                  p + "attention.output.LayerNorm")
            layers.append(BertLayerWeights(
                cat([a + n + ".weight" for n in qkv]), cat([a + n + ".bias" for n in qkv]),
                get(o + ".weight"), get(o + ".bias"), ln(aln),
                get(p + "intermediate.dense.weight"), get(p + "intermediate.dense.bias"),
                get(p + "output.dense.weight"), get(p + "output.dense.bias"), ln(p + "output.LayerNorm")))
        return cls(get("embeddings.word_embeddings.weight"), get("embeddings.position_embeddings.weight"),
                   get("embeddings.token_type_embeddings.weight") if cfg.type_vocab_size else None,
                   ln("embeddings.LayerNorm"), layers,
                   get("encoder.relative_attention_bias.weight") if cfg.is_mpnet else None)


def relative_bucket(delta: torch.Tensor, num_buckets: int = 32, max_distance: int = 128) -> torch.Tensor:
    """Bucket of a signed key-minus-query distance: half of the buckets per direction; in each half the first
    ``num_buckets / 4`` distances get a bucket each and the rest share log-spaced buckets up to ``max_distance``."""
    half = num_buckets // 2
    exact = half // 2
    n = -delta
    side = (n < 0).long() * half
    n = n.abs()
    far = exact + (torch.log(n.float().clamp_min(1) / exact) / math.log(max_distance / exact) * (half - exact)).long()
    return side + torch.where(n < exact, n, far.clamp_max(half - 1))


class BertModel:
    """Sentence-embedding encoder behind the engine's model interface (``encode`` only)."""

    use_executor = False
    executor = None
    logits_buf = None
    default_pooling = "mean"
    generates = False           # schedulers refuse generation requests before they reach a step

    def __init__(self, cfg: BertConfig, weights: BertWeights, kv_cache: torch.Tensor = None, max_tokens: int = 8192,
                 max_seqs: int = 256, max_position: Optional[int] = None):
        self.cfg, self.w, self.kv = cfg, weights, kv_cache
        self.device, self.dtype = weights.embed.device, weights.embed.dtype
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.page_size = kv_cache.shape[4] if kv_cache is not None else 0

    def forward_tensors(self, *args, **kwargs):
        raise NotImplementedError("encoder-only model: it serves embeddings (/v1/embeddings), not generation")

    def _act(self, x):
        a = self.cfg.hidden_act
        if a == "relu":
            return F.relu(x)
        return F.gelu(x, approximate="tanh" if a in ("gelu_new", "gelu_pytorch_tanh") else "none")

    @torch.no_grad()
    def hidden_states(self, tokens: list) -> torch.Tensor:
        """Final hidden states [n, hidden] of one sequence."""
        c, w = self.cfg, self.w
        n = len(tokens)
        first = c.pad_token_id + 1 if c.is_mpnet else 0       # MPNet counts positions from its padding index
        if n + first > c.max_position_embeddings:
            raise ValueError(f"{n} tokens exceed the model's {c.max_position_embeddings - first} positions")
        ids = torch.tensor(tokens, dtype=torch.long, device=self.device)
        h = w.embed[ids] + w.pos_embed[first: first + n]
        if w.type_embed is not None:
            h = h + w.type_embed[0]
        h = F.layer_norm(h, (c.hidden_size,), *w.embed_ln, c.layer_norm_eps)
        bias = None
        if w.rel_bias is not None:
            pos = torch.arange(n, device=self.device)
            bucket = relative_bucket(pos[None, :] - pos[:, None], c.relative_attention_num_buckets)
            bias = w.rel_bias[bucket].permute(2, 0, 1).to(h.dtype)          # [heads, q, k]
        nh, hd = c.num_attention_heads, c.head_dim
        for l in w.layers:
            q, k, v = (F.linear(h, l.wqkv, l.bqkv).view(n, 3, nh, hd).permute(1, 2, 0, 3))
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=bias).permute(1, 0, 2).reshape(n, nh * hd)
            h = F.layer_norm(F.linear(a, l.wo, l.bo) + h, (c.hidden_size,), *l.attn_ln, c.layer_norm_eps)
            m = F.linear(self._act(F.linear(h, l.w1, l.b1)), l.w2, l.b2)
            h = F.layer_norm(m + h, (c.hidden_size,), *l.out_ln, c.layer_norm_eps)
        return h

    @torch.no_grad()
    def encode(self, token_lists, pooling: str = "mean", normalize: bool = True) -> torch.Tensor:
        """Pooled embeddings, fp32 [n, hidden]: ``cls`` (first token), ``mean`` or ``last``."""
        if not token_lists or min(len(t) for t in token_lists) < 1:
            raise ValueError("encode needs non-empty token lists")
        if pooling not in ("cls", "mean", "last"):
            raise ValueError(f"unknown pooling {pooling!r} (cls | mean | last)")
        out = torch.empty(len(token_lists), self.cfg.hidden_size, dtype=torch.float32, device=self.device)
        for i, toks in enumerate(token_lists):
            h = self.hidden_states(list(toks)).float()
            out[i] = h[0] if pooling == "cls" else h[-1] if pooling == "last" else h.mean(0)
        if normalize:
            out = out / out.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        return out
