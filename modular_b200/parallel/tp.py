"""Tensor parallelism: one process per GPU, symmetric buffers, weight sharding.

``TPContext`` wraps the process group and allocates *symmetric* device buffers (same size on
every rank, every rank knows every peer's address) through ``torch.distributed``'s symmetric
memory, which only does the plumbing (allocation + handle exchange over the NCCL/TCP store);
all traffic is issued by this package's own kernels in ``csrc/kernels/comm.cu``.

Sharding follows the reference's strategies (max/python/max/nn/linear.py rowwise / columnwise,
nn/attention/attention_with_rope.py:972 heads split across devices,
nn/transformer/distributed_transformer.py:283-290 MLP gate/up column-split and down row-split):

    wqkv   rows of this rank's query and KV heads        (column parallel)
    wo     columns of this rank's query heads            (row parallel  -> partial sums)
    wgu    rows [gate_shard; up_shard]                   (column parallel)
    wd     columns of the shard                          (row parallel  -> partial sums)
    lm_head rows of the vocabulary shard                 (column parallel -> gathered logits)
    embedding and norms are replicated.

The residual stream is kept sharded by rows between layers (sequence-parallel layout,
reference: architectures/deepseekV3/deepseekV3.py:583-649 ``TP_EP`` mode), so the only data
crossing NVLink per half-layer is one pull of the partial sums a rank owns and one push of
its normalised rows.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class SymmetricBuffer:
    tensor: torch.Tensor          # this rank's buffer
    peer_ptrs: list               # device address of the buffer on every rank (index = rank)
    handle: object = None


class TPContext:
    def __init__(self, group=None, device: Optional[torch.device] = None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised (one process per GPU)")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self._keep = []

    def alloc_symmetric(self, numel: int, dtype: torch.dtype, zero: bool = False) -> SymmetricBuffer:
        import torch.distributed._symmetric_memory as symm_mem

        t = symm_mem.empty(numel, dtype=dtype, device=self.device)
        if zero:
            t.zero_()
        try:
            hdl = symm_mem.rendezvous(t, self.group)
        except TypeError:
            hdl = symm_mem.rendezvous(t, self.group.group_name)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        sb = SymmetricBuffer(t, ptrs, hdl)
        self._keep.append(sb)
        return sb

    def barrier(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def collectives(self, max_bytes: int = 64 << 20) -> "Collectives":
        """Stand-alone collectives on this context (lazily built, one staging area per context)."""
        if getattr(self, "_coll", None) is None or self._coll.max_bytes < max_bytes:
            self._coll = Collectives(self, max_bytes)
        return self._coll


class Collectives:
    """All-reduce / all-gather / broadcast over peer memory with this package's kernels.

    Inputs are staged into a symmetric buffer (one device-to-device copy) unless they already live
    in one. Results are bit-identical on every rank (fixed summation order). Reference:
    max/kernels/src/comm/allreduce.mojo:257-468 (1-stage / 2-stage dispatch by size),
    comm/allgather.mojo:167, comm/broadcast.mojo:173; nn/comm/allreduce.py:40 (``Allreduce`` layer).
    """

    # messages up to this size take the barrier-free path under ``auto`` (the reference selects its sentinel
    # kernel for <= 1 MB on 2/4/8 B200, comm/allreduce.mojo:320-372)
    LAMPORT_MAX_BYTES = 1 << 20

    def __init__(self, ctx: TPContext, max_bytes: int = 64 << 20):
        from .._native import lib

        self.ctx, self.max_bytes, self.L = ctx, max_bytes, lib()
        self.inp = ctx.alloc_symmetric(max_bytes // 2, torch.bfloat16)
        self.out = ctx.alloc_symmetric(max_bytes // 2, torch.bfloat16)
        self.flags = ctx.alloc_symmetric(self.L.tp_flag_ints(), torch.int32, zero=True)
        self.multicast_ptr = int(getattr(self.inp.handle, "multicast_ptr", 0) or 0)
        # barrier-free small-message path: receive buffers [3 generations][world][cap] of bf16 -0.0 sentinels
        self.lam_cap = min(self.LAMPORT_MAX_BYTES, max_bytes) // 2
        self.lam = ctx.alloc_symmetric(3 * ctx.world * self.lam_cap, torch.bfloat16)
        self.lam.tensor.view(torch.int16).fill_(-32768)
        self.lam_state = torch.zeros(8, dtype=torch.int32, device=ctx.device)
        ctx.barrier()

    def all_reduce(self, x: torch.Tensor, algo: str = "auto") -> torch.Tensor:
        """Sum of ``x`` (bf16, numel % 8 == 0) over all ranks.
        algo: auto | lamport (barrier-free, sentinel-polled; small messages) | one_shot | two_shot | multimem."""
        n = x.numel()
        if x.dtype != torch.bfloat16 or n % 8 or n * 2 > self.max_bytes:
            raise ValueError("all_reduce: bf16 tensors with numel % 8 == 0 up to the staging size")
        if algo == "lamport" or (algo == "auto" and n <= self.lam_cap):
            if n > self.lam_cap:
                raise ValueError(f"lamport all-reduce takes at most {self.lam_cap} elements")
            c = self.ctx
            res = torch.empty_like(x)
            self.L.tp_allreduce_lamport(c.world, c.rank, self.lam.peer_ptrs, x.contiguous(), res, self.lam_cap,
                                        self.lam_state, None, None, 0.0)
            return res
        code = {"auto": 0, "one_shot": 1, "two_shot": 2, "multimem": 3}[algo]
        if code == 3 and not self.multicast_ptr:
            raise RuntimeError("this symmetric allocation has no NVLink multicast mapping")
        c = self.ctx
        self.inp.tensor[:n].copy_(x.reshape(-1))
        res = torch.empty_like(x)
        two_shot = code == 2 or (code == 0 and n * 2 > (512 << 10))
        self.L.tp_allreduce(c.world, c.rank, self.inp.peer_ptrs, self.out.peer_ptrs, res, self.multicast_ptr,
                            self.flags.peer_ptrs, n, 2 if two_shot else (code or 1))
        if two_shot:
            res.copy_(self.out.tensor[:n].view_as(x))
        return res

    def all_reduce_add_rms_norm(self, x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float):
        """``residual += all_reduce(x)`` (in place) and ``rms_norm(residual) * gamma`` in one barrier-free kernel.
        x, residual: [rows, cols] bf16. Returns (normalised rows, residual)."""
        if x.numel() > self.lam_cap or x.shape != residual.shape or x.shape[-1] % 8:
            raise ValueError("all_reduce_add_rms_norm: rows of a multiple of 8 elements, within the receive buffer")
        c = self.ctx
        out = torch.empty_like(x)
        self.L.tp_allreduce_lamport(c.world, c.rank, self.lam.peer_ptrs, x.contiguous(), out, self.lam_cap,
                                    self.lam_state, residual, gamma, eps)
        return out, residual

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """Concatenation of every rank's ``x`` along dim 0 (bf16 or fp32 rows of 16-byte multiples)."""
        c = self.ctx
        x2 = x.reshape(x.shape[0], -1).contiguous()
        rows, row_bytes = x2.shape[0], x2.shape[1] * x2.element_size()
        if row_bytes % 16 or c.world * rows * row_bytes > self.max_bytes:
            raise ValueError("all_gather: rows must be multiples of 16 bytes and fit the staging size")
        # every rank's block lands at row offset rank * rows of every rank's `out` buffer
        dst = [p + c.rank * rows * row_bytes for p in self.out.peer_ptrs]
        self.L.tp_allgather(c.world, c.rank, dst, self.flags.peer_ptrs, x2, rows, row_bytes, row_bytes,
                            row_bytes, 0)
        n = c.world * rows * x2.shape[1]
        return self.out.tensor.view(x.dtype)[:n].view(c.world * x.shape[0], *x.shape[1:]).clone()

    def scatter(self, x: Optional[torch.Tensor], like: torch.Tensor, root: int = 0) -> torch.Tensor:
        """Rank r receives ``x[r]`` of the root's ``x`` ([world, ...]); ``like`` gives the chunk's shape and dtype on
        every rank (``x`` is only read on the root)."""
        c = self.ctx
        nbytes = like.numel() * like.element_size()
        if nbytes % 16 or nbytes * c.world > self.max_bytes // 2:
            raise ValueError("scatter: chunks must be multiples of 16 bytes and fit the staging size")
        if c.rank == root:
            if x is None or x.shape[0] != c.world or x[0].numel() != like.numel():
                raise ValueError("scatter: the root passes a tensor of world chunks")
            self.inp.tensor.view(torch.uint8)[: nbytes * c.world].copy_(x.contiguous().reshape(-1).view(torch.uint8))
        res = torch.empty_like(like)
        self.L.tp_scatter(c.world, c.rank, root, self.inp.peer_ptrs, res, self.flags.peer_ptrs, nbytes)
        return res

    def broadcast(self, x: torch.Tensor, root: int = 0) -> torch.Tensor:
        c = self.ctx
        nbytes = x.numel() * x.element_size()
        if nbytes % 16 or nbytes > self.max_bytes // 2:
            raise ValueError("broadcast: size must be a multiple of 16 bytes and fit the staging size")
        if c.rank == root:
            self.inp.tensor.view(torch.uint8)[:nbytes].copy_(x.reshape(-1).view(torch.uint8))
        res = torch.empty_like(x)
        self.L.tp_broadcast(c.world, c.rank, root, self.inp.peer_ptrs, res, self.flags.peer_ptrs, nbytes)
        return res


def shard_llama_config(cfg, world: int):
    if cfg.num_attention_heads % world or cfg.num_key_value_heads % world:
        raise ValueError(f"TP degree {world} must divide the query heads ({cfg.num_attention_heads}) and "
                         f"KV heads ({cfg.num_key_value_heads})")
    if cfg.intermediate_size % (world * 8) or cfg.vocab_size % (world * 8):
        raise ValueError("TP degree must divide the FFN and vocabulary sizes (in units of 8)")
    local = copy.copy(cfg)
    local.num_attention_heads = cfg.num_attention_heads // world
    local.num_key_value_heads = cfg.num_key_value_heads // world
    local.intermediate_size = cfg.intermediate_size // world
    return local


def _shard_fp8_layer(cfg, l, rank: int, world: int):
    """Shard of a block-scaled fp8 layer: weights are cut on 128-element boundaries so that every scale block
    stays whole (the shard sizes of the supported models are multiples of 128)."""
    from ..models.llama3 import LayerWeights

    hd = cfg.head_dim
    nq, nkv = cfg.num_attention_heads // world, cfg.num_key_value_heads // world
    qd, kd, I = cfg.q_dim, cfg.kv_dim, cfg.intermediate_size
    Il = I // world
    if (nq * hd) % 128 or (nkv * hd) % 128 or Il % 128:
        raise ValueError("fp8 tensor parallelism needs per-rank head and FFN sizes that are multiples of 128")
    u8 = lambda w: w.view(torch.uint8)
    f8 = lambda w: w.contiguous().view(torch.float8_e4m3fn)

    def rows(w, s, a, n):          # rows [a, a + n) of weight and scales
        return u8(w)[a:a + n], s[a // 128:(a + n) // 128]

    def cols(w, s, a, n):
        return u8(w)[:, a:a + n], s[:, a // 128:(a + n) // 128]

    parts = [rows(l.wqkv, l.wqkv_s, rank * nq * hd, nq * hd), rows(l.wqkv, l.wqkv_s, qd + rank * nkv * hd, nkv * hd),
             rows(l.wqkv, l.wqkv_s, qd + kd + rank * nkv * hd, nkv * hd)]
    wqkv = f8(torch.cat([p[0] for p in parts], 0))
    wqkv_s = torch.cat([p[1] for p in parts], 0).contiguous()
    wo, wo_s = cols(l.wo, l.wo_s, rank * nq * hd, nq * hd)
    gu = [rows(l.wgu, l.wgu_s, rank * Il, Il), rows(l.wgu, l.wgu_s, I + rank * Il, Il)]
    wgu = f8(torch.cat([p[0] for p in gu], 0))
    wgu_s = torch.cat([p[1] for p in gu], 0).contiguous()
    wd, wd_s = cols(l.wd, l.wd_s, rank * Il, Il)
    return LayerWeights(l.attn_norm, wqkv, f8(wo), l.mlp_norm, wgu, f8(wd), wqkv_s, wo_s.contiguous(), wgu_s,
                        wd_s.contiguous(), _shard_qkv_bias(cfg, l.qkv_bias, rank, world), l.q_norm, l.k_norm)


def _shard_qkv_bias(cfg, bias, rank: int, world: int):
    """This rank's entries of a [q; k; v] projection bias: the rows of its query and KV heads."""
    if bias is None:
        return None
    hd = cfg.head_dim
    nq, nkv = cfg.num_attention_heads // world, cfg.num_key_value_heads // world
    q, k, v = torch.split(bias, [cfg.q_dim, cfg.kv_dim, cfg.kv_dim])
    q0, k0 = rank * nq * hd, rank * nkv * hd
    return torch.cat([q[q0:q0 + nq * hd], k[k0:k0 + nkv * hd], v[k0:k0 + nkv * hd]]).contiguous()


def shard_llama_weights(cfg, weights, rank: int, world: int):
    """Slice full weights into this rank's shard (see the module docstring for the layout)."""
    from ..models.llama3 import LayerWeights, Llama3Weights

    hd = cfg.head_dim
    nq, nkv = cfg.num_attention_heads // world, cfg.num_key_value_heads // world
    q0, k0 = rank * nq * hd, rank * nkv * hd
    I = cfg.intermediate_size
    Il = I // world
    layers = []
    for l in weights.layers:
        if l.is_fp8:
            layers.append(_shard_fp8_layer(cfg, l, rank, world))
            continue
        q, k, v = torch.split(l.wqkv, [cfg.q_dim, cfg.kv_dim, cfg.kv_dim], dim=0)
        wqkv = torch.cat([q[q0:q0 + nq * hd], k[k0:k0 + nkv * hd], v[k0:k0 + nkv * hd]], dim=0).contiguous()
        wo = l.wo[:, q0:q0 + nq * hd].contiguous()
        g, u = l.wgu[:I], l.wgu[I:]
        wgu = torch.cat([g[rank * Il:(rank + 1) * Il], u[rank * Il:(rank + 1) * Il]], dim=0).contiguous()
        wd = l.wd[:, rank * Il:(rank + 1) * Il].contiguous()
        layers.append(LayerWeights(l.attn_norm, wqkv, wo, l.mlp_norm, wgu, wd,
                                   qkv_bias=_shard_qkv_bias(cfg, l.qkv_bias, rank, world), q_norm=l.q_norm,
                                   k_norm=l.k_norm))
    Vl = cfg.vocab_size // world
    lm_head = weights.lm_head[rank * Vl:(rank + 1) * Vl].contiguous()
    return Llama3Weights(weights.embed, layers, weights.final_norm, lm_head)
