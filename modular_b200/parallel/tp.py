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
        q, k, v = torch.split(l.wqkv, [cfg.q_dim, cfg.kv_dim, cfg.kv_dim], dim=0)
        wqkv = torch.cat([q[q0:q0 + nq * hd], k[k0:k0 + nkv * hd], v[k0:k0 + nkv * hd]], dim=0).contiguous()
        wo = l.wo[:, q0:q0 + nq * hd].contiguous()
        g, u = l.wgu[:I], l.wgu[I:]
        wgu = torch.cat([g[rank * Il:(rank + 1) * Il], u[rank * Il:(rank + 1) * Il]], dim=0).contiguous()
        wd = l.wd[:, rank * Il:(rank + 1) * Il].contiguous()
        layers.append(LayerWeights(l.attn_norm, wqkv, wo, l.mlp_norm, wgu, wd))
    Vl = cfg.vocab_size // world
    lm_head = weights.lm_head[rank * Vl:(rank + 1) * Vl].contiguous()
    return Llama3Weights(weights.embed, layers, weights.final_norm, lm_head)
