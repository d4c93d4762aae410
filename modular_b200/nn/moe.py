"""Mixture-of-experts layer: routing, expert GEMMs, weighted combine.

``MoE.forward`` runs
    router logits -> top-k (group-limited sigmoid routing for DeepSeek-V3, softmax top-k otherwise)
    -> sort (token, slot) pairs by expert -> gather rows in expert order
    -> grouped gate/up GEMM with SwiGLU epilogue -> grouped down GEMM
    -> un-permute + router-weighted sum (+ shared experts).
On CUDA every stage is one of this package's kernels (``moe.cu`` and the grouped mode of the
tcgen05 GEMM); on CPU the same stages run in PyTorch. ``e_begin`` / ``e_end`` restrict the layer
to the experts this rank owns (expert parallelism): pairs routed elsewhere contribute nothing
locally and are handled by the dispatch / combine exchange in :mod:`modular_b200.parallel.ep`.

Reference: max/python/max/nn/moe/moe.py:221 (``MoE``, forward :743-865), ``MoEGate`` :118,
architectures/deepseekV3/layers/moe_gate.py:36 (group-limited router).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from .. import ops
from .._native import lib as _lib


@dataclass
class MoEConfig:
    hidden_size: int
    moe_intermediate_size: int
    n_routed_experts: int
    num_experts_per_tok: int
    n_shared_experts: int = 0
    n_group: int = 1
    topk_group: int = 1
    norm_topk_prob: bool = True
    routed_scaling_factor: float = 1.0
    scoring_func: str = "sigmoid"       # sigmoid (DeepSeek-V3) | softmax


# ---------------------------------------------------------------------- reference routing
def route_group_limited_ref(logits, bias, cfg: MoEConfig):
    scores = torch.sigmoid(logits.float())
    choice = scores + (bias.float() if bias is not None else 0.0)
    T, E = scores.shape
    g = choice.view(T, cfg.n_group, E // cfg.n_group)
    gscore = g.topk(min(2, g.shape[-1]), dim=-1).values.sum(-1)
    gidx = gscore.topk(cfg.topk_group, dim=-1).indices
    gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, gidx, True)
    masked = choice.masked_fill(~gmask.unsqueeze(-1).expand_as(g).reshape(T, E), float("-inf"))
    ids = masked.topk(cfg.num_experts_per_tok, dim=-1).indices
    w = scores.gather(1, ids)
    if cfg.norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return ids.int(), w * cfg.routed_scaling_factor


def route_softmax_ref(logits, cfg: MoEConfig):
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = p.topk(cfg.num_experts_per_tok, dim=-1)
    if cfg.norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return ids.int(), w * cfg.routed_scaling_factor


def route_softmax_group_limited(logits, cfg: MoEConfig):
    """DeepSeek-V2's ``group_limited_greedy``: softmax over all experts, the ``topk_group`` groups with the largest
    single score stay, top-k among their experts (torch ops on either device: this router has no kernel of its own)."""
    p = torch.softmax(logits.float(), dim=-1)
    T, E = p.shape
    g = p.view(T, cfg.n_group, E // cfg.n_group)
    gidx = g.amax(dim=-1).topk(cfg.topk_group, dim=-1).indices
    gmask = torch.zeros(T, cfg.n_group, dtype=torch.bool, device=p.device).scatter_(1, gidx, True)
    masked = p.masked_fill(~gmask.unsqueeze(-1).expand_as(g).reshape(T, E), 0.0)
    w, ids = masked.topk(cfg.num_experts_per_tok, dim=-1)
    if cfg.norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return ids.int(), (w * cfg.routed_scaling_factor).contiguous()


def route(logits, bias, cfg: MoEConfig):
    """Returns (topk_ids int32 [T, k], topk_weights fp32 [T, k])."""
    if cfg.scoring_func != "sigmoid" and cfg.n_group > 1:
        return route_softmax_group_limited(logits, cfg)
    if not logits.is_cuda:
        if cfg.scoring_func == "sigmoid":
            return route_group_limited_ref(logits, bias, cfg)
        return route_softmax_ref(logits, cfg)
    T, k = logits.shape[0], cfg.num_experts_per_tok
    ids = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    lg = logits.float().contiguous()
    if cfg.scoring_func == "sigmoid":
        _lib().moe_router_group_limited(lg, bias.float() if bias is not None else None, ids, w, cfg.n_group,
                                        cfg.topk_group, cfg.norm_topk_prob, cfg.routed_scaling_factor)
    else:
        _lib().moe_router_softmax_topk(lg, ids, w, cfg.norm_topk_prob)
        if cfg.routed_scaling_factor != 1.0:
            w *= cfg.routed_scaling_factor
    return ids, w


class Fp8ExpertWeights:
    """Block-scaled fp8 weights of a stack of experts: ``q`` [E, N, K] float8_e4m3fn and ``scale`` fp32
    [E, N/128, ceil(K/128)] (the checkpoint's ``weight_scale_inv`` per 128x128 block); N % 128 == 0.
    Reference: max/python/max/nn/moe/moe_fp8.py:48 with the fp8-blockwise strategy of quant_strategy.py."""

    def __init__(self, q: torch.Tensor, scale: torch.Tensor):
        self.q, self.scale = q.contiguous(), scale.float().contiguous()

    @classmethod
    def quantize(cls, w: torch.Tensor) -> "Fp8ExpertWeights":
        qs = [ops.reference.quant_fp8_weight_block128(w[e]) for e in range(w.shape[0])]
        return cls(torch.stack([q for q, _ in qs]), torch.stack([s for _, s in qs]))

    @property
    def shape(self):
        return self.q.shape

    def __getitem__(self, e):
        """Integer: dequantised weight of expert ``e`` (reference paths). Slice: that range of experts."""
        if isinstance(e, slice):
            return Fp8ExpertWeights(self.q[e], self.scale[e])
        return ops.reference.dequant_fp8_weight_block128(self.q[e], self.scale[e])

    def contiguous(self):
        return self


class MoE:
    """Weights: ``gate`` [E, H] router, ``w_gate_up`` [E_local, 2I, H], ``w_down`` [E_local, H, I] (bf16
    tensors or :class:`Fp8ExpertWeights`), optional shared experts fused as one MLP (``shared_gate_up``
    [2 I_s, H], ``shared_down`` [H, I_s])."""

    def __init__(self, cfg: MoEConfig, gate, w_gate_up, w_down, e_score_bias=None, shared_gate_up=None,
                 shared_down=None, e_begin: int = 0, e_end: Optional[int] = None):
        self.cfg = cfg
        self.gate, self.bias = gate, e_score_bias
        self.w_gate_up, self.w_down = w_gate_up, w_down
        self.shared_gate_up, self.shared_down = shared_gate_up, shared_down
        self.e_begin = e_begin
        self.e_end = cfg.n_routed_experts if e_end is None else e_end
        self._scratch = None

    @classmethod
    def random_init(cls, cfg: MoEConfig, device="cpu", dtype=torch.bfloat16, seed=0, std=0.02, **kw):
        g = torch.Generator().manual_seed(seed)
        r = lambda *s: (torch.randn(*s, generator=g) * std).to(dtype).to(device)
        E, H, I = cfg.n_routed_experts, cfg.hidden_size, cfg.moe_intermediate_size
        e0, e1 = kw.get("e_begin", 0), kw.get("e_end") or E
        full_gu, full_d = r(E, 2 * I, H), r(E, H, I)
        shared = cfg.n_shared_experts * I
        return cls(cfg, r(E, H).float().to(device), full_gu[e0:e1].contiguous(), full_d[e0:e1].contiguous(),
                   (torch.randn(E, generator=g) * 0.1).to(device) if cfg.scoring_func == "sigmoid" else None,
                   r(2 * shared, H) if shared else None, r(H, shared) if shared else None, **kw)

    # ------------------------------------------------------------ pieces
    def router_logits(self, x):
        """fp32 router scores [T, E]. On the GPU the product runs on this package's GEMM with a bf16 copy of the
        router matrix (checkpoints store it in bf16, so nothing is lost) and fp32 accumulation and output."""
        if x.is_cuda and x.dtype == torch.bfloat16 and self.gate.shape[0] % 64 == 0:
            if getattr(self, "_gate_bf16", None) is None:
                self._gate_bf16 = self.gate.to(torch.bfloat16).contiguous()
            return ops.linear(x, self._gate_bf16, out_dtype=torch.float32)
        return x.float() @ self.gate.float().t()

    def shared_forward(self, x):
        if self.shared_gate_up is None:
            return None
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[0] <= ops.DECODE_GEMM_MAX_TOKENS:
            return ops.linear_decode(ops.linear_decode(x, self.shared_gate_up, "swiglu"), self.shared_down)
        return ops.linear(ops.linear_swiglu(x, self.shared_gate_up), self.shared_down)

    def experts_forward(self, x, ids, w, shared_out=None):
        """Local experts on tokens x with routing (ids, w); returns y [T, H]."""
        if not x.is_cuda:
            return self._experts_ref(x, ids, w, shared_out)
        cfg, dev = self.cfg, x.device
        T, k = ids.shape
        E = self.e_end - self.e_begin
        if self._scratch is None or self._scratch[0].device != dev:
            self._scratch = (torch.zeros(2 * E, dtype=torch.int32, device=dev),
                             torch.empty(E + 1, dtype=torch.int32, device=dev))
        scratch, offsets = self._scratch
        order = torch.empty(T * k, dtype=torch.int32, device=dev)
        inverse = torch.empty(T * k, dtype=torch.int32, device=dev)
        L = _lib()
        L.moe_create_indices(ids, self.e_begin, self.e_end, scratch, offsets, order, inverse)
        n_local = offsets[E:E + 1]
        xp = torch.empty(T * k, cfg.hidden_size, dtype=x.dtype, device=dev)
        L.moe_permute_rows(x, order, n_local, xp, k)
        out = self.local_gemms(xp, offsets)
        y = torch.empty(T, cfg.hidden_size, dtype=x.dtype, device=dev)
        L.moe_combine(out, inverse, w, shared_out, y, k)
        return y

    def local_gemms(self, xp, offsets, act=None, out=None, max_rows: int = 0, expected_rows: int = 0):
        """Both grouped GEMMs of the local experts on rows already in expert order (``offsets`` int32
        [E_local + 1]). ``xp``: bf16 rows, or ``(xq, xs)`` = e4m3 rows [n, H] (any row stride) with fp32
        scales [H/128, n] for fp8 experts that receive quantised rows. Returns bf16 [n, H]. ``n`` may be an
        upper bound of the rows (the true count is ``offsets[-1]`` on the device); ``max_rows`` bounds the rows
        of one expert and ``expected_rows`` is the typical count per expert (it picks the token tile)."""
        cfg, L = self.cfg, _lib()
        fp8_in = isinstance(xp, tuple)
        n = (xp[0] if fp8_in else xp).shape[0]
        dev = (xp[0] if fp8_in else xp).device
        if out is None:
            out = torch.empty(n, cfg.hidden_size, dtype=torch.bfloat16, device=dev)
        if isinstance(self.w_gate_up, Fp8ExpertWeights):
            # quantise per 1x128 group, grouped block-scaled GEMM, SwiGLU, quantise again, second grouped
            # GEMM (rows past the local count hold garbage that is never read back)
            xq, xs = xp if fp8_in else ops.quant_fp8_group128(xp)
            I = cfg.moe_intermediate_size
            E = self.e_end - self.e_begin
            bn = 0
            if expected_rows > 0:
                bn = 32 if expected_rows <= 32 else (64 if expected_rows <= 64 else 128)
            gu = torch.empty(n, 2 * I, dtype=torch.bfloat16, device=dev)
            L.grouped_gemm_fp8(xq, xs, self.w_gate_up.q, self.w_gate_up.scale, gu, offsets, max_rows or n, bn)
            # SwiGLU and the quantisation of its result in one pass over the rows that exist
            aq = torch.empty(n, I, dtype=torch.float8_e4m3fn, device=dev)
            a_s = torch.empty(I // 128, n, dtype=torch.float32, device=dev)
            L.silu_mul_quant_fp8(gu, aq, a_s, offsets[E:E + 1])
            L.grouped_gemm_fp8(aq, a_s, self.w_down.q, self.w_down.scale, out, offsets, max_rows or n, bn)
            return out
        if fp8_in:
            raise ValueError("quantised rows need fp8 expert weights")
        if act is None:
            act = torch.empty(n, cfg.moe_intermediate_size, dtype=xp.dtype, device=dev)
        L.grouped_gemm_bf16(xp, self.w_gate_up, act, offsets, n, True, 0)
        L.grouped_gemm_bf16(act, self.w_down, out, offsets, n, False, 0)
        return out

    def _experts_ref(self, x, ids, w, shared_out=None):
        cfg = self.cfg
        y = torch.zeros(x.shape[0], cfg.hidden_size, dtype=torch.float32, device=x.device)
        if shared_out is not None:
            y += shared_out.float()
        I = cfg.moe_intermediate_size
        for e in range(self.e_begin, self.e_end):
            tok, slot = torch.nonzero(ids == e, as_tuple=True)
            if tok.numel() == 0:
                continue
            xe = x[tok]
            gu = self.w_gate_up[e - self.e_begin]
            h = ops.reference.linear_swiglu(xe, gu)
            o = ops.reference.linear(h, self.w_down[e - self.e_begin])
            y.index_add_(0, tok, o.float() * w[tok, slot].unsqueeze(1))
        return y.to(x.dtype)

    def forward(self, x):
        ids, w = route(self.router_logits(x), self.bias, self.cfg)
        return self.experts_forward(x, ids, w, self.shared_forward(x))

    __call__ = forward
