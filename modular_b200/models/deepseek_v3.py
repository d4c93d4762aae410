"""DeepSeek-V3 / R1 decoder: multi-head latent attention (MLA) + mixture-of-experts FFN.

Attention keeps only a *latent* row per token in the paged cache (``kv_lora_rank`` compressed
KV values + the shared rotary key, 512 + 64 numbers), and runs in the absorbed form for prefill
and decode alike: queries are multiplied by ``W_uk`` into latent space, attention is MQA-shaped
(all heads share the one latent "KV head"), and the result is multiplied by ``W_uv`` afterwards.
Both absorptions are per-head batched GEMMs on the grouped tcgen05 kernel.

The first ``first_k_dense_replace`` layers use a dense SwiGLU MLP, the rest a routed MoE with
group-limited sigmoid routing and shared experts (:mod:`modular_b200.nn.moe`); with expert
parallelism the routed experts are sharded over ranks (:mod:`modular_b200.parallel.ep`).

Weights may be bf16 or block-scaled fp8 (128x128 blocks, ``weight_scale_inv`` in the
checkpoint); fp8 linears run on the block-scaled tcgen05 GEMM, expert weights are kept in bf16
for the grouped GEMM.

Reference: max/python/max/pipelines/architectures/deepseekV3/deepseekV3.py (DeepseekV3, decoder
layer :173-392, EP modes :583-649), layers/moe_gate.py:36, nn/attention/multi_latent_attention.py,
model_config.py; HF ``DeepseekV3ForCausalLM`` naming for checkpoints.
"""

from __future__ import annotations

import contextlib
import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..nn.moe import Fp8ExpertWeights, MoE, MoEConfig
from ..nn.rotary_embedding import RopeScaling, cos_sin_table



@contextlib.contextmanager
def _no_gc_during_capture():
    """Collect dead reference cycles now and keep the cyclic collector off while a CUDA graph is captured. The
    step below runs as Python code that allocates many temporaries; a collection triggered in the middle of it
    can destroy CUDA graphs of an engine that is no longer referenced, and destroying a graph is not permitted
    while a stream captures (the capture is invalidated and the next launch fails)."""
    import gc

    gc.collect()
    was_on = gc.isenabled()
    gc.disable()
    try:
        yield
    finally:
        if was_on:
            gc.enable()

@dataclass
class DeepseekV3Config:
    vocab_size: int = 129280
    hidden_size: int = 7168
    intermediate_size: int = 18432
    moe_intermediate_size: int = 2048
    num_hidden_layers: int = 61
    num_attention_heads: int = 128
    q_lora_rank: Optional[int] = 1536
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    n_routed_experts: int = 256
    n_shared_experts: int = 1
    num_experts_per_tok: int = 8
    n_group: int = 8
    topk_group: int = 4
    norm_topk_prob: bool = True
    routed_scaling_factor: float = 2.5
    scoring_func: str = "sigmoid"
    first_k_dense_replace: int = 3
    moe_layer_freq: int = 1
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = field(default_factory=lambda: dict(
        type="yarn", factor=40.0, original_max_position_embeddings=4096, beta_fast=32, beta_slow=1,
        mscale=1.0, mscale_all_dim=1.0))
    max_position_embeddings: int = 163840
    tie_word_embeddings: bool = False

    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def latent_dim(self) -> int:
        return self.kv_lora_rank + self.qk_rope_head_dim

    # what the generic engine code asks of any config
    architectures = ("DeepseekV3ForCausalLM",)

    @property
    def num_key_value_heads(self) -> int:
        return 1          # one shared latent row per token

    @property
    def head_dim(self) -> int:
        return self.latent_dim

    def to_hf(self) -> dict:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d["architectures"] = list(self.architectures)
        d["model_type"] = "deepseek_v3"
        return d

    def param_count(self) -> int:
        H, h = self.hidden_size, self.num_attention_heads
        attn = (H * (self.q_lora_rank or 0) + (self.q_lora_rank or H) * h * self.qk_head_dim + H * self.latent_dim
                + self.kv_lora_rank * h * (self.qk_nope_head_dim + self.v_head_dim) + h * self.v_head_dim * H)
        dense = 3 * H * self.intermediate_size
        moe = 3 * H * self.moe_intermediate_size * (self.n_routed_experts + self.n_shared_experts) + H * self.n_routed_experts
        n_moe = sum(self.is_moe_layer(i) for i in range(self.num_hidden_layers))
        return (self.num_hidden_layers * attn + n_moe * moe + (self.num_hidden_layers - n_moe) * dense
                + 2 * self.vocab_size * H)

    def is_moe_layer(self, i: int) -> bool:
        return (self.n_routed_experts > 0 and i >= self.first_k_dense_replace
                and i % self.moe_layer_freq == 0)

    def moe_config(self) -> MoEConfig:
        return MoEConfig(self.hidden_size, self.moe_intermediate_size, self.n_routed_experts,
                         self.num_experts_per_tok, self.n_shared_experts, self.n_group, self.topk_group,
                         self.norm_topk_prob, self.routed_scaling_factor, self.scoring_func)

    def softmax_scale(self) -> float:
        s = 1.0 / math.sqrt(self.qk_head_dim)
        rs = self.rope_scaling or {}
        if rs.get("mscale_all_dim") and rs.get("factor", 1.0) > 1.0:
            m = 0.1 * rs["mscale_all_dim"] * math.log(rs["factor"]) + 1.0
            s *= m * m
        return s

    @classmethod
    def deepseek_v3(cls) -> "DeepseekV3Config":
        return cls()

    @classmethod
    def tiny(cls, **kw) -> "DeepseekV3Config":
        base = dict(vocab_size=512, hidden_size=256, intermediate_size=512, moe_intermediate_size=128,
                    num_hidden_layers=3, num_attention_heads=4, q_lora_rank=128, kv_lora_rank=128,
                    qk_nope_head_dim=64, qk_rope_head_dim=64, v_head_dim=64, n_routed_experts=8,
                    n_shared_experts=1, num_experts_per_tok=2, n_group=2, topk_group=1,
                    first_k_dense_replace=1, max_position_embeddings=2048,
                    rope_scaling=dict(type="yarn", factor=4.0, original_max_position_embeddings=512,
                                      beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0))
        base.update(kw)
        return cls(**base)

    @classmethod
    def from_hf(cls, d: dict) -> "DeepseekV3Config":
        from ..pipelines.weights import normalize_hf_rope

        d = normalize_hf_rope(d)
        names = cls.__dataclass_fields__.keys()
        kw = {k: v for k, v in d.items() if k in names}
        if "DeepseekV2ForCausalLM" in (d.get("architectures") or ()) or d.get("model_type") == "deepseek_v2":
            # DeepSeek-V2 / V2-Lite: same attention and layer layout; the router is a softmax over the experts with a
            # plain top-k ("greedy", V2-Lite) or a top-k inside the groups with the largest single score
            # ("group_limited_greedy", V2 / V2.5)
            method = d.get("topk_method", "greedy")
            if method not in ("greedy", "group_limited_greedy"):
                raise ValueError(f"router method {method!r} of DeepSeek-V2 is not implemented")
            kw["scoring_func"] = "softmax"
            if method == "greedy":
                kw.update(n_group=1, topk_group=1)
            kw.setdefault("norm_topk_prob", False)
            kw.setdefault("routed_scaling_factor", 1.0)
            if "rope_scaling" not in kw:
                kw["rope_scaling"] = None
        return cls(**kw)


class Fp8Weight:
    """Block-scaled fp8 weight: q [N, K] float8_e4m3fn, scale fp32 [ceil(N/128), ceil(K/128)]."""

    def __init__(self, q: torch.Tensor, scale: torch.Tensor):
        self.q, self.scale = q, scale

    @property
    def shape(self):
        return self.q.shape

    def dequant(self) -> torch.Tensor:
        return ops.reference.dequant_fp8_weight_block128(self.q, self.scale)


def _linear(x, w, residual=None):
    if isinstance(w, Fp8Weight):
        if x.is_cuda:
            return ops.linear_fp8(x, w.q, w.scale, residual=residual)
        y = ops.reference.linear(x, w.dequant().to(x.dtype), residual)
        return y
    return ops.linear(x, w, residual=residual)


@dataclass
class DSLayer:
    attn_norm: torch.Tensor
    q_a: Optional[object]            # [q_lora, H]     (None when q_lora_rank is None)
    q_a_norm: Optional[torch.Tensor]
    q_b: object                      # [h * qk_head_dim, q_lora]  (or q_proj [h * qk_head_dim, H])
    kv_a: object                     # [kv_lora + rope, H]
    kv_a_norm: torch.Tensor
    w_uk: torch.Tensor               # [h, kv_lora, nope]   absorbed on the query side   (N=kv_lora, K=nope)
    w_uv: torch.Tensor               # [h, v_dim, kv_lora]  applied to the latent output  (N=v_dim, K=kv_lora)
    wo: object                       # [H, h * v_dim]
    mlp_norm: torch.Tensor
    w_a: Optional[torch.Tensor] = None   # [q_lora + kv_lora + rope, H]: q_a and kv_a stacked (bf16 weights only)
    wgu: Optional[object] = None     # dense layers: [2 * inter, H]
    wd: Optional[object] = None      # dense layers: [H, inter]
    moe: Optional[MoE] = None


class DeepseekV3Weights:
    def __init__(self, cfg: DeepseekV3Config, embed, layers, final_norm, lm_head):
        self.cfg, self.embed, self.layers, self.final_norm, self.lm_head = cfg, embed, layers, final_norm, lm_head

    @staticmethod
    def split_kv_b(cfg: DeepseekV3Config, kv_b: torch.Tensor):
        """kv_b_proj.weight [h * (nope + v), kv_lora] -> (w_uk [h, kv_lora, nope], w_uv [h, v, kv_lora])."""
        h = cfg.num_attention_heads
        w = kv_b.view(h, cfg.qk_nope_head_dim + cfg.v_head_dim, cfg.kv_lora_rank)
        w_uk = w[:, : cfg.qk_nope_head_dim].transpose(1, 2).contiguous()
        w_uv = w[:, cfg.qk_nope_head_dim:].contiguous()
        return w_uk, w_uv

    @classmethod
    def random_init(cls, cfg: DeepseekV3Config, device="cpu", dtype=torch.bfloat16, seed=0, std=0.02,
                    e_begin: int = 0, e_end: Optional[int] = None) -> "DeepseekV3Weights":
        g = torch.Generator().manual_seed(seed)
        r = lambda *s: (torch.randn(*s, generator=g) * std).to(dtype).to(device)
        ones = lambda n: torch.ones(n, dtype=dtype, device=device)
        H, h = cfg.hidden_size, cfg.num_attention_heads
        layers = []
        for i in range(cfg.num_hidden_layers):
            kv_b = r(h * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank)
            w_uk, w_uv = cls.split_kv_b(cfg, kv_b)
            if cfg.q_lora_rank:
                q_a, q_a_norm, q_b = r(cfg.q_lora_rank, H), ones(cfg.q_lora_rank), r(h * cfg.qk_head_dim, cfg.q_lora_rank)
            else:
                q_a, q_a_norm, q_b = None, None, r(h * cfg.qk_head_dim, H)
            lw = DSLayer(ones(H), q_a, q_a_norm, q_b, r(cfg.latent_dim, H), ones(cfg.kv_lora_rank), w_uk, w_uv,
                         r(H, h * cfg.v_head_dim), ones(H))
            if cfg.is_moe_layer(i):
                lw.moe = MoE.random_init(cfg.moe_config(), device, dtype, seed=seed * 1000 + i + 1, std=std,
                                         e_begin=e_begin, e_end=e_end)
            else:
                lw.wgu, lw.wd = r(2 * cfg.intermediate_size, H), r(H, cfg.intermediate_size)
            layers.append(lw)
        embed = r(cfg.vocab_size, H)
        return cls(cfg, embed, layers, ones(H), embed if cfg.tie_word_embeddings else r(cfg.vocab_size, H))

    @classmethod
    def random_init_ep(cls, cfg: DeepseekV3Config, rank: int, world: int, device="cuda", dtype=torch.bfloat16,
                       seed: int = 0, std: float = 0.02, fp8_experts: bool = True) -> "DeepseekV3Weights":
        """Random weights of ONE expert-parallel rank, generated on the device: attention, dense layers, router and
        shared experts replicated (same seed on every rank), routed experts [rank * E/world, (rank + 1) * E/world)
        only, quantised to block-scaled fp8 layer by layer when ``fp8_experts`` (the full model holds 671 B
        parameters; a rank's slice is ~82 GB in fp8). For synthetic-weight benchmarks."""
        from ..nn.moe import Fp8ExpertWeights

        dev = torch.device(device)
        g_all = torch.Generator(device=dev).manual_seed(seed)
        g_rank = torch.Generator(device=dev).manual_seed(seed * 1000003 + rank + 1)
        rnd = lambda g, *s: (torch.randn(*s, device=dev, dtype=torch.float32, generator=g) * std).to(dtype)
        ones = lambda n: torch.ones(n, dtype=dtype, device=dev)
        H, h = cfg.hidden_size, cfg.num_attention_heads
        mc = cfg.moe_config()
        E, I = cfg.n_routed_experts, cfg.moe_intermediate_size
        El = E // world
        layers = []
        for i in range(cfg.num_hidden_layers):
            kv_b = rnd(g_all, h * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank)
            w_uk, w_uv = cls.split_kv_b(cfg, kv_b)
            if cfg.q_lora_rank:
                q_a, q_a_norm, q_b = rnd(g_all, cfg.q_lora_rank, H), ones(cfg.q_lora_rank), rnd(g_all, h * cfg.qk_head_dim, cfg.q_lora_rank)
            else:
                q_a, q_a_norm, q_b = None, None, rnd(g_all, h * cfg.qk_head_dim, H)
            lw = DSLayer(ones(H), q_a, q_a_norm, q_b, rnd(g_all, cfg.latent_dim, H), ones(cfg.kv_lora_rank), w_uk, w_uv,
                         rnd(g_all, H, h * cfg.v_head_dim), ones(H))
            if cfg.is_moe_layer(i):
                gate = rnd(g_all, E, H).float()
                bias = (torch.randn(E, device=dev, generator=g_all) * 0.1) if mc.scoring_func == "sigmoid" else None
                shared = mc.n_shared_experts * I
                sgu = rnd(g_all, 2 * shared, H) if shared else None
                sd_ = rnd(g_all, H, shared) if shared else None
                wgu, wd = rnd(g_rank, El, 2 * I, H), rnd(g_rank, El, H, I)
                if fp8_experts:
                    wgu, wd = Fp8ExpertWeights.quantize(wgu), Fp8ExpertWeights.quantize(wd)
                lw.moe = MoE(mc, gate, wgu, wd, bias, sgu, sd_, e_begin=rank * El, e_end=(rank + 1) * El)
            else:
                lw.wgu, lw.wd = rnd(g_all, 2 * cfg.intermediate_size, H), rnd(g_all, H, cfg.intermediate_size)
            layers.append(lw)
        embed = rnd(g_all, cfg.vocab_size, H)
        return cls(cfg, embed, layers, ones(H), embed if cfg.tie_word_embeddings else rnd(g_all, cfg.vocab_size, H))

    @classmethod
    def from_state_dict(cls, cfg: DeepseekV3Config, sd: dict, device="cpu", dtype=torch.bfloat16,
                        e_begin: int = 0, e_end: Optional[int] = None, keep_fp8: bool = True):
        """HF ``DeepseekV3ForCausalLM`` names (with or without the ``model.`` prefix). fp8 tensors come
        with ``<name>_scale_inv``; they stay fp8 for plain linears and are dequantised for experts,
        ``kv_b_proj`` (absorbed) and the router."""
        sd = {(k[6:] if k.startswith("model.") else k): v for k, v in sd.items()}
        e_end = cfg.n_routed_experts if e_end is None else e_end

        def W(name, allow_fp8=True):
            w = sd[name + ".weight"]
            sc = sd.get(name + ".weight_scale_inv")
            if sc is not None:
                fw = Fp8Weight(w.to(device), sc.float().to(device))
                return fw if (allow_fp8 and keep_fp8) else fw.dequant().to(dtype)
            return w.to(dtype).to(device)

        V = lambda name: sd[name].to(dtype).to(device)
        layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            a = p + "self_attn."
            w_uk, w_uv = cls.split_kv_b(cfg, W(a + "kv_b_proj", allow_fp8=False))
            if cfg.q_lora_rank:
                q_a, q_a_norm, q_b = W(a + "q_a_proj"), V(a + "q_a_layernorm.weight"), W(a + "q_b_proj")
            else:
                q_a, q_a_norm, q_b = None, None, W(a + "q_proj")
            lw = DSLayer(V(p + "input_layernorm.weight"), q_a, q_a_norm, q_b, W(a + "kv_a_proj_with_mqa"),
                         V(a + "kv_a_layernorm.weight"), w_uk, w_uv, W(a + "o_proj"),
                         V(p + "post_attention_layernorm.weight"))
            m = p + "mlp."
            if cfg.is_moe_layer(i):
                cat = lambda x, y: torch.cat((x, y), dim=0).contiguous()
                # routed experts stay in block-scaled fp8 when the checkpoint has them so and the row counts
                # are whole 128-row scale blocks (gate and up then stack without re-blocking)
                ex_fp8 = (keep_fp8 and f"{m}experts.{e_begin}.gate_proj.weight_scale_inv" in sd
                          and cfg.moe_intermediate_size % 128 == 0 and cfg.hidden_size % 128 == 0)
                if ex_fp8:
                    def stack8(names):
                        parts = [[W(f"{m}experts.{e}.{n}") for n in names] for e in range(e_begin, e_end)]
                        return Fp8ExpertWeights(torch.stack([torch.cat([p.q for p in ps]) for ps in parts]),
                                                torch.stack([torch.cat([p.scale for p in ps]) for ps in parts]))
                    gu, dn = stack8(("gate_proj", "up_proj")), stack8(("down_proj",))
                elif m + "experts.gate_up_proj" in sd:
                    # all experts of a layer in two tensors ([E, 2 I, H] gate rows then up rows, [E, H, I]): the
                    # layout transformers >= 5 keeps in memory and writes back
                    gu = sd[m + "experts.gate_up_proj"][e_begin:e_end].to(dtype).to(device).contiguous()
                    dn = sd[m + "experts.down_proj"][e_begin:e_end].to(dtype).to(device).contiguous()
                else:
                    gu = torch.stack([cat(W(f"{m}experts.{e}.gate_proj", False), W(f"{m}experts.{e}.up_proj", False))
                                      for e in range(e_begin, e_end)])
                    dn = torch.stack([W(f"{m}experts.{e}.down_proj", False) for e in range(e_begin, e_end)])
                sh_gu = sh_d = None
                if cfg.n_shared_experts:
                    sh_gu = cat(W(m + "shared_experts.gate_proj", False), W(m + "shared_experts.up_proj", False))
                    sh_d = W(m + "shared_experts.down_proj", False)
                bias = sd.get(m + "gate.e_score_correction_bias")
                lw.moe = MoE(cfg.moe_config(), sd[m + "gate.weight"].float().to(device), gu, dn,
                             None if bias is None else bias.float().to(device), sh_gu, sh_d,
                             e_begin=e_begin, e_end=e_end)
            else:
                def dense(n):
                    w = W(m + n)
                    return w
                g_, u_ = dense("gate_proj"), dense("up_proj")
                if isinstance(g_, Fp8Weight):   # rows of gate and up stay block-aligned when stacked
                    lw.wgu = Fp8Weight(torch.cat((g_.q, u_.q)), torch.cat((g_.scale, u_.scale)))
                else:
                    lw.wgu = torch.cat((g_, u_)).contiguous()
                lw.wd = dense("down_proj")
            layers.append(lw)
        embed = V("embed_tokens.weight")
        lm = embed if cfg.tie_word_embeddings or "lm_head.weight" not in sd else V("lm_head.weight")
        return cls(cfg, embed, layers, V("norm.weight"), lm)

    def to_hf_state_dict(self) -> dict:
        """bf16 weights back to HF names (for round-trip tests)."""
        cfg, sd = self.cfg, {}
        sd["model.embed_tokens.weight"] = self.embed
        sd["model.norm.weight"] = self.final_norm
        if not cfg.tie_word_embeddings:
            sd["lm_head.weight"] = self.lm_head
        for i, l in enumerate(self.layers):
            p, a = f"model.layers.{i}.", f"model.layers.{i}.self_attn."
            kv_b = torch.cat((l.w_uk.transpose(1, 2), l.w_uv), dim=1).reshape(-1, cfg.kv_lora_rank)
            sd[p + "input_layernorm.weight"] = l.attn_norm
            sd[p + "post_attention_layernorm.weight"] = l.mlp_norm
            if l.q_a is not None:
                sd[a + "q_a_proj.weight"], sd[a + "q_a_layernorm.weight"], sd[a + "q_b_proj.weight"] = l.q_a, l.q_a_norm, l.q_b
            else:
                sd[a + "q_proj.weight"] = l.q_b
            sd[a + "kv_a_proj_with_mqa.weight"], sd[a + "kv_a_layernorm.weight"] = l.kv_a, l.kv_a_norm
            sd[a + "kv_b_proj.weight"], sd[a + "o_proj.weight"] = kv_b, l.wo
            m = p + "mlp."
            if l.moe is not None:
                I = cfg.moe_intermediate_size
                sd[m + "gate.weight"] = l.moe.gate
                if l.moe.bias is not None:
                    sd[m + "gate.e_score_correction_bias"] = l.moe.bias
                for j in range(l.moe.w_gate_up.shape[0]):
                    e = l.moe.e_begin + j
                    sd[f"{m}experts.{e}.gate_proj.weight"] = l.moe.w_gate_up[j, :I]
                    sd[f"{m}experts.{e}.up_proj.weight"] = l.moe.w_gate_up[j, I:]
                    sd[f"{m}experts.{e}.down_proj.weight"] = l.moe.w_down[j]
                if l.moe.shared_gate_up is not None:
                    S = l.moe.shared_gate_up.shape[0] // 2
                    sd[m + "shared_experts.gate_proj.weight"] = l.moe.shared_gate_up[:S]
                    sd[m + "shared_experts.up_proj.weight"] = l.moe.shared_gate_up[S:]
                    sd[m + "shared_experts.down_proj.weight"] = l.moe.shared_down
            else:
                inter = l.wgu.shape[0] // 2
                sd[m + "gate_proj.weight"], sd[m + "up_proj.weight"], sd[m + "down_proj.weight"] = \
                    l.wgu[:inter], l.wgu[inter:], l.wd
        return {k: v.contiguous() for k, v in sd.items()}


class DeepseekV3Model:
    """Runs ragged batches of a DeepSeek-V3 decoder against a paged *latent* KV cache.

    ``kv_cache``: ``[pages, 1, layers, 1, page_size, kv_lora_rank + rope_dim]``. With ``ep`` (an
    :class:`modular_b200.parallel.ep.EPContext`) the routed experts of every MoE layer are this
    rank's slice and tokens are exchanged by the dispatch / combine kernels.
    """

    use_executor = False      # the step is a sequence of this package's kernels driven from Python

    def __init__(self, cfg: DeepseekV3Config, weights: DeepseekV3Weights, kv_cache: torch.Tensor,
                 max_tokens: int = 8192, max_seqs: int = 256, max_position: Optional[int] = None, ep=None):
        self.cfg, self.w, self.kv = cfg, weights, kv_cache
        self.device, self.dtype = weights.embed.device, weights.embed.dtype
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.page_size = kv_cache.shape[4]
        self.scale = cfg.softmax_scale()
        rs = dict(cfg.rope_scaling or {})
        if rs.get("type", rs.get("rope_type")) == "yarn":
            rs["rope_type"] = "deepseek_yarn"
            rs.pop("type", None)
        max_position = max_position or min(cfg.max_position_embeddings, 1 << 17)
        self.cos_sin = cos_sin_table(cfg.qk_rope_head_dim, max_position, cfg.rope_theta,
                                     RopeScaling.from_hf(rs) if rs else None, self.device)
        # q_a and kv_a read the same input: one GEMM over their stacked rows (the layer keeps views of the stack)
        for l in weights.layers:
            if getattr(l, "w_a", None) is None and torch.is_tensor(l.kv_a) and (l.q_a is None or torch.is_tensor(l.q_a)):
                l.w_a = torch.cat([l.q_a, l.kv_a]) if l.q_a is not None else l.kv_a
                if l.q_a is not None:
                    ql = l.q_a.shape[0]
                    l.q_a, l.kv_a = l.w_a[:ql], l.w_a[ql:]
        self.ep = ep
        self._ep_layers = {}
        if ep is not None:
            from ..parallel.ep import EPMoE
            for i, l in enumerate(weights.layers):
                if l.moe is not None:
                    self._ep_layers[i] = EPMoE(l.moe, ep if self.device.type == "cuda" else None)
        self.sampled = torch.zeros(max_seqs, dtype=torch.long, device=self.device)
        self._graphs: dict = {}             # decode batch size -> (graph, static inputs, static logits)
        self.forward_calls = 0              # steps taken (eager or replayed)
        self._graph_calls: dict = {}        # native calls recorded in each graph (0 unless calls are counted)
        self.graph_replays = 0
        self.replayed_calls = 0

    # ------------------------------------------------------------ CUDA graphs of decode steps
    def capture_decode_graphs(self, batch_sizes: Sequence[int]) -> None:
        """Capture one graph per decode batch size (one query token per sequence). The whole step, MoE exchange
        included, is one replay: the exchange kernels keep their epochs in device memory. With expert
        parallelism every rank must call this with the same sizes at the same point (the warm-up run of every
        size exchanges rows)."""
        if self.device.type != "cuda":
            return
        dev, pages = self.device, self.kv.shape[0]
        max_pages = -(-min(self.cos_sin.shape[0], pages * self.page_size) // self.page_size)
        for B in sorted(set(int(b) for b in batch_sizes)):
            if B in self._graphs or B > self.max_seqs:
                continue
            i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
            st = dict(tokens=torch.zeros(B, dtype=torch.long, device=dev), positions=i32(B),
                      slots=torch.full((B,), -1, dtype=torch.long, device=dev), block_table=i32(B, max_pages),
                      q_start=torch.arange(B, dtype=torch.int32, device=dev), q_len=i32(B) + 1, kv_len=i32(B) + 1,
                      logit_rows=torch.arange(B, dtype=torch.int32, device=dev))
            args = tuple(st[k] for k in ("tokens", "positions", "slots", "block_table", "q_start", "q_len",
                                         "kv_len", "logit_rows"))
            if self.ep is not None:
                self.ep.set_step_tokens(B)
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._forward(*args)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            from .._native import native_calls

            g = torch.cuda.CUDAGraph()
            n0 = native_calls()
            with _no_gc_during_capture():
                with torch.cuda.graph(g):
                    logits = self._forward(*args)
            self._graph_calls[B] = native_calls() - n0
            self._graphs[B] = (g, st, logits)
        torch.cuda.synchronize()

    def _graph_for(self, T: int, n_seqs: int, n_logits: int):
        """The graph size for this step, or 0. Expert-parallel ranks first agree on the largest token count of
        the step: all of them then address the exchange buffers with the same bound, whichever path each takes."""
        sizes = sorted(self._graphs)
        if self.ep is not None and self.device.type == "cuda":
            if self.ep.host_group is None:
                return 0        # no agreement between the ranks: every step runs eagerly with the full bound
            bound = self.ep.set_step_tokens(T)
            fit = next((b for b in sizes if b >= bound), 0)
            self.ep.set_step_tokens_local(fit or bound)
        else:
            fit = next((b for b in sizes if b >= T), 0)
        return fit if (fit and T == n_seqs == n_logits) else 0

    def forward_tensors(self, tokens, positions, slots, block_table, q_start, q_len, kv_len,
                        logit_rows, plan=None) -> torch.Tensor:
        """One ragged step. Returns fp32 logits ``[len(logit_rows), vocab]``. Decode-only steps replay a captured
        graph when one of a fitting size exists (sequences beyond the real ones are dummies that write no KV)."""
        T, n = tokens.shape[0], q_len.shape[0]
        self.forward_calls += 1
        B = self._graph_for(T, n, logit_rows.shape[0]) if (self._graphs or self.ep is not None) else 0
        if not B:
            return self._forward(tokens, positions, slots, block_table, q_start, q_len, kv_len, logit_rows)
        g, st, logits = self._graphs[B]
        st["tokens"][:n].copy_(tokens)
        st["positions"][:n].copy_(positions)
        st["slots"][:n].copy_(slots)
        st["slots"][n:].fill_(-1)
        st["kv_len"][:n].copy_(kv_len)
        st["kv_len"][n:].fill_(1)
        w = min(block_table.shape[1], st["block_table"].shape[1])
        st["block_table"][:n, :w].copy_(block_table[:, :w])
        g.replay()
        self.graph_replays += 1
        self.replayed_calls += self._graph_calls.get(B, 0)
        return logits[:n]

    def expert_load(self):
        """Rows routed to each local expert of every MoE layer so far: int64 numpy [moe layers, experts per rank]
        (None unless the expert-parallel context collects the load). Idle steps and graph warm-ups count too: one
        dummy token each."""
        layers = [self._ep_layers[i] for i in sorted(self._ep_layers)]
        if not layers or layers[0].load is None:
            return None
        return torch.stack([l.load for l in layers]).cpu().numpy()

    def idle_step(self) -> None:
        """A step with one dummy token that writes no cache entry: what an expert-parallel rank without requests
        runs while other ranks work, so that it takes part in their exchanges (and serves its experts)."""
        dev = self.device
        i32 = lambda v: torch.tensor([v], dtype=torch.int32, device=dev)
        self.forward_tensors(torch.zeros(1, dtype=torch.long, device=dev), i32(0),
                             torch.full((1,), -1, dtype=torch.long, device=dev),
                             torch.zeros(1, 1, dtype=torch.int32, device=dev), i32(0), i32(1), i32(1), i32(0))

    # ------------------------------------------------------------ attention
    def _attention_fused(self, li: int, l: DSLayer, x, positions, slots, block_table, q_start, q_len, kv_len):
        """The CUDA path for bf16 attention weights: one down-projection GEMM, one kernel for both norms, the key
        rotation and the cache store, per-head absorption GEMMs that address the heads in place (no transposes)."""
        from .._native import lib

        c, L = self.cfg, lib()
        T, h, R = x.shape[0], c.num_attention_heads, c.kv_lora_rank
        lin = ops.linear_decode if T <= ops.DECODE_GEMM_MAX_TOKENS else ops.linear
        dev = x.device
        cache = self.kv[:, 0, li, 0]
        ql = c.q_lora_rank or 0
        qkv_a = lin(x, l.w_a)
        q_a = torch.empty(T, ql, dtype=x.dtype, device=dev) if ql else None
        L.mla_post_down(qkv_a, ql, l.q_a_norm, l.kv_a_norm, c.rms_norm_eps, positions, self.cos_sin, slots, q_a, cache)
        q = lin(q_a if ql else x, l.q_b)                                      # [T, h * (nope + rope)]
        q_rope = torch.empty(T, h, c.qk_rope_head_dim, dtype=x.dtype, device=dev)
        L.mla_q_rope(q, h, c.qk_nope_head_dim, positions, self.cos_sin, q_rope)
        q_lat = torch.empty(T, h * R, dtype=x.dtype, device=dev)
        ops.batched_linear_heads(q, l.w_uk, q_lat, c.qk_head_dim, R)          # absorb W_uk per head
        o_lat = ops.mla_paged_attention(q_lat.view(T, h, R), q_rope, cache, block_table, q_start, q_len, kv_len,
                                        self.scale)
        o = torch.empty(T, h * c.v_head_dim, dtype=x.dtype, device=dev)
        ops.batched_linear_heads(o_lat.view(T, h * R), l.w_uv, o, R, c.v_head_dim)   # apply W_uv per head
        return o

    def _attention(self, li: int, l: DSLayer, x, positions, slots, block_table, q_start, q_len, kv_len):
        c = self.cfg
        if (x.is_cuda and x.dtype == torch.bfloat16 and l.w_a is not None and torch.is_tensor(l.q_b)
                and c.qk_rope_head_dim == 64 and positions.dtype == torch.int32):
            return self._attention_fused(li, l, x, positions, slots, block_table, q_start, q_len, kv_len)
        T, h = x.shape[0], c.num_attention_heads
        if l.q_a is not None:
            q = _linear(ops.rms_norm(_linear(x, l.q_a), l.q_a_norm, c.rms_norm_eps), l.q_b)
        else:
            q = _linear(x, l.q_b)
        q = q.view(T, h, c.qk_head_dim)
        kv_a = _linear(x, l.kv_a)
        c_kv = ops.rms_norm(kv_a[:, : c.kv_lora_rank].contiguous(), l.kv_a_norm, c.rms_norm_eps)
        half = c.qk_rope_head_dim // 2
        cs = self.cos_sin[positions.long()]
        cos, sin = cs[:, :half], cs[:, half:]
        k_rope = ops.reference.apply_rope(kv_a[:, c.kv_lora_rank:].unsqueeze(1), cos, sin, True).squeeze(1)
        q_rope = ops.reference.apply_rope(q[..., c.qk_nope_head_dim:], cos, sin, True).contiguous()
        cache = self.kv[:, 0, li, 0]
        ops.mla_kv_store(c_kv, k_rope, slots, cache)
        # absorb W_uk: per-head  q_nope [T, nope] @ w_uk[h]^T -> [T, kv_lora]
        q_nope = q[..., : c.qk_nope_head_dim].transpose(0, 1)
        q_lat = ops.batched_linear(q_nope, l.w_uk).transpose(0, 1).contiguous()
        o_lat = ops.mla_paged_attention(q_lat, q_rope, cache, block_table, q_start, q_len, kv_len, self.scale)
        # apply W_uv: per-head  o_lat [T, kv_lora] @ w_uv[h]^T -> [T, v]
        o = ops.batched_linear(o_lat.transpose(0, 1), l.w_uv).transpose(0, 1).reshape(T, h * c.v_head_dim)
        return o.contiguous()

    def _mlp(self, li: int, l: DSLayer, x):
        if l.moe is None:
            if isinstance(l.wgu, Fp8Weight):
                return _linear(ops.silu_mul(_linear(x, l.wgu)), l.wd)
            return ops.linear(ops.linear_swiglu(x, l.wgu), l.wd)
        if li in self._ep_layers:
            return self._ep_layers[li](x)
        return l.moe(x)

    # ------------------------------------------------------------ step
    def _forward(self, tokens, positions, slots, block_table, q_start, q_len, kv_len, logit_rows) -> torch.Tensor:
        c, eps = self.cfg, self.cfg.rms_norm_eps
        layers = self.w.layers
        h = ops.embedding(tokens, self.w.embed)
        # decode-sized steps on the GPU use the GEMM that carries the residual add and the next norm in its tail
        small = h.is_cuda and h.dtype == torch.bfloat16 and h.shape[0] <= ops.DECODE_GEMM_MAX_TOKENS
        x = ops.rms_norm(h, layers[0].attn_norm, eps)
        for li, l in enumerate(layers):
            a = self._attention(li, l, x, positions, slots, block_table, q_start, q_len, kv_len)
            if small and torch.is_tensor(l.wo):
                x, h = ops.linear_decode(a, l.wo, "add_norm", h=h, gamma=l.mlp_norm, eps=eps)
            else:
                h = _linear(a, l.wo, residual=h)
                x = ops.rms_norm(h, l.mlp_norm, eps)
            gamma_next = layers[li + 1].attn_norm if li + 1 < len(layers) else self.w.final_norm
            if l.moe is None and small and torch.is_tensor(l.wgu):
                x, h = ops.linear_decode(ops.linear_decode(x, l.wgu, "swiglu"), l.wd, "add_norm", h=h, gamma=gamma_next,
                                         eps=eps)
                continue
            if li in self._ep_layers and h.is_cuda:
                h = self._ep_layers[li](x, residual=h)            # the combine adds the residual
            else:
                y = self._mlp(li, l, x)
                h = (h.float() + y.float()).to(h.dtype) if not h.is_cuda else h + y
            x = ops.rms_norm(h, gamma_next, eps)
        return ops.linear(x[logit_rows.long()], self.w.lm_head, out_dtype=torch.float32).float()


def hf_reference_forward(cfg: DeepseekV3Config, sd: dict, tokens: torch.Tensor) -> torch.Tensor:
    """Straightforward (non-absorbed, dense, fp32) DeepSeek-V3 forward of one sequence from an HF-named
    state dict: the oracle for tests. Returns logits [T, vocab]."""
    sd = {(k[6:] if k.startswith("model.") else k): v.float() for k, v in sd.items()}
    T, h = tokens.shape[0], cfg.num_attention_heads
    rms = lambda x, w: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w
    rs = dict(cfg.rope_scaling or {})
    if rs.get("type", rs.get("rope_type")) == "yarn":
        rs["rope_type"] = "deepseek_yarn"
        rs.pop("type", None)
    cs = cos_sin_table(cfg.qk_rope_head_dim, T, cfg.rope_theta, RopeScaling.from_hf(rs) if rs else None)
    half = cfg.qk_rope_head_dim // 2
    cos, sin = cs[:, :half], cs[:, half:]
    x = sd["embed_tokens.weight"][tokens]
    mcfg = cfg.moe_config()
    from ..nn.moe import route
    for i in range(cfg.num_hidden_layers):
        p, a = f"layers.{i}.", f"layers.{i}.self_attn."
        xn = rms(x, sd[p + "input_layernorm.weight"])
        if cfg.q_lora_rank:
            q = rms(xn @ sd[a + "q_a_proj.weight"].t(), sd[a + "q_a_layernorm.weight"]) @ sd[a + "q_b_proj.weight"].t()
        else:
            q = xn @ sd[a + "q_proj.weight"].t()
        q = q.view(T, h, cfg.qk_head_dim)
        kv_a = xn @ sd[a + "kv_a_proj_with_mqa.weight"].t()
        c_kv = rms(kv_a[:, : cfg.kv_lora_rank], sd[a + "kv_a_layernorm.weight"])
        k_rope = ops.reference.apply_rope(kv_a[:, cfg.kv_lora_rank:].unsqueeze(1), cos, sin, True)
        q_rope = ops.reference.apply_rope(q[..., cfg.qk_nope_head_dim:], cos, sin, True)
        kv = (c_kv @ sd[a + "kv_b_proj.weight"].t()).view(T, h, cfg.qk_nope_head_dim + cfg.v_head_dim)
        k = torch.cat((kv[..., : cfg.qk_nope_head_dim], k_rope.expand(T, h, -1)), dim=-1)
        v = kv[..., cfg.qk_nope_head_dim:]
        qf = torch.cat((q[..., : cfg.qk_nope_head_dim], q_rope), dim=-1)
        s = torch.einsum("qhd,khd->hqk", qf, k) * cfg.softmax_scale()
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(T, -1)
        x = x + o @ sd[a + "o_proj.weight"].t()
        xn = rms(x, sd[p + "post_attention_layernorm.weight"])
        m = p + "mlp."
        ffn = lambda z, pre: (torch.nn.functional.silu(z @ sd[pre + "gate_proj.weight"].t()) *
                              (z @ sd[pre + "up_proj.weight"].t())) @ sd[pre + "down_proj.weight"].t()
        if cfg.is_moe_layer(i):
            ids, w = route(xn @ sd[m + "gate.weight"].t(), sd.get(m + "gate.e_score_correction_bias"), mcfg)
            y = ffn(xn, m + "shared_experts.") if cfg.n_shared_experts else torch.zeros_like(xn)
            for t in range(T):
                for j in range(ids.shape[1]):
                    y[t] += w[t, j] * ffn(xn[t:t + 1], f"{m}experts.{int(ids[t, j])}.")[0]
            x = x + y
        else:
            x = x + ffn(xn, m)
    x = rms(x, sd["norm.weight"])
    lm = sd.get("lm_head.weight", sd["embed_tokens.weight"])
    return x @ lm.t()
