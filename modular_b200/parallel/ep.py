"""Expert parallelism: token dispatch to the ranks that own the experts, and the combine back.

Each rank holds ``E / W`` routed experts (a contiguous slice) and its own batch of tokens
(data-parallel attention, expert-parallel MoE — the reference's ``TP_EP`` / ``DP_EP`` modes,
architectures/deepseekV3/deepseekV3.py:583-649, nn/moe/expert_parallel.py). One MoE layer is

    route -> dispatch (push rows into the owner's receive buffer over NVLink)
          -> sort received rows by local expert -> grouped gate/up(SwiGLU) and down GEMMs
          -> combine_send (push results back to the token's rank) -> weighted reduce.

On CUDA the exchange is done by this package's own kernels in ``csrc/kernels/comm_ep.cu`` over
symmetric peer memory (no NCCL call on the data path; reference counterpart
max/kernels/src/shmem/ep_comm.mojo). On CPU (``gloo``) the same exchange is expressed with
``all_to_all`` so the host-side logic is testable without GPUs.

Buffers are sized for ``cap`` rows per (source, owner) pair; a pair that would overflow the
capacity is dropped and counted (``EPMoE.dropped``). ``cap = max_tokens * top_k`` can never overflow.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .._native import lib as _lib
from ..nn.moe import Fp8ExpertWeights, MoE, MoEConfig, route
from .tp import TPContext


class EPContext:
    """Symmetric receive / return buffers for one MoE shape, shared by all layers."""

    def __init__(self, ctx: TPContext, hidden: int, n_experts: int, top_k: int, max_tokens: int,
                 cap: Optional[int] = None, fp8_dispatch: bool = False):
        if n_experts % ctx.world:
            raise ValueError(f"{n_experts} experts cannot be split over {ctx.world} ranks")
        if hidden % 128:
            raise ValueError("hidden size must be a multiple of 128")
        self.ctx, self.world, self.rank = ctx, ctx.world, ctx.rank
        self.hidden, self.top_k = hidden, top_k
        self.e_local = n_experts // ctx.world
        self.cap = cap if cap is not None else max_tokens * top_k
        self.max_tokens = max_tokens
        self.fp8 = fp8_dispatch
        self.row_bytes = hidden + hidden // 128 * 4 if fp8_dispatch else hidden * 2
        W, L = self.world, _lib()
        self.recv_x = ctx.alloc_symmetric(W * self.cap * self.row_bytes, torch.uint8)
        self.recv_meta = ctx.alloc_symmetric(W * self.cap * 2, torch.int32, zero=True)
        self.ret_x = ctx.alloc_symmetric(W * self.cap * hidden, torch.bfloat16)
        self.flags = ctx.alloc_symmetric(L.ep_flag_ints(), torch.int32, zero=True)
        dev = ctx.device
        n = W * self.cap
        self.ids_recv = torch.empty(n, dtype=torch.int32, device=dev)
        self.order = torch.empty(n, dtype=torch.int32, device=dev)
        self.inverse = torch.empty(n, dtype=torch.int32, device=dev)
        self.scratch = torch.zeros(2 * self.e_local, dtype=torch.int32, device=dev)
        self.offsets = torch.empty(self.e_local + 1, dtype=torch.int32, device=dev)
        self.xp = torch.empty(n, hidden, dtype=torch.bfloat16, device=dev)
        self.xq = torch.empty(n, self.row_bytes, dtype=torch.uint8, device=dev) if fp8_dispatch else None
        self.send_pos = torch.zeros(max_tokens * top_k, dtype=torch.int32, device=dev)
        self.last_pairs = 0
        ctx.barrier()   # flags are zero everywhere before the first kernel signals a peer

    # ------------------------------------------------------------------ stages
    def dispatch(self, x: torch.Tensor, ids: torch.Tensor, keep_fp8: bool = False):
        """Push rows to their owners. Returns (rows in local-expert order, offsets [E_local+1], send_pos).
        With fp8 dispatch and ``keep_fp8`` the rows stay quantised: ``(xq e4m3 [n, H] strided, xs fp32
        [H/128, n])``, the operand form of the block-scaled grouped GEMM."""
        L, W = _lib(), self.world
        T = x.shape[0]
        assert T <= self.max_tokens and ids.shape[1] == self.top_k
        send_pos = self.send_pos[: T * self.top_k]
        self.last_pairs = T * self.top_k
        L.ep_dispatch(W, self.rank, self.recv_x.peer_ptrs, self.recv_meta.peer_ptrs, self.flags.peer_ptrs,
                      x, ids, send_pos, self.e_local, self.cap, self.fp8)
        L.ep_gather_ids(self.recv_meta.tensor, self.flags.tensor, self.ids_recv, W, self.cap)
        L.moe_create_indices(self.ids_recv.view(-1, 1), 0, self.e_local, self.scratch, self.offsets,
                             self.order, self.inverse)
        n_rows = self.offsets[self.e_local:self.e_local + 1]
        if self.fp8:
            L.moe_permute_rows(self.recv_x.tensor.view(W * self.cap, self.row_bytes), self.order, n_rows,
                               self.xq, 1)
            if keep_fp8:
                xq = self.xq[:, : self.hidden].view(torch.float8_e4m3fn)
                xs = self.xq[:, self.hidden:].view(torch.float32).t().contiguous()
                return (xq, xs), self.offsets, send_pos
            L.ep_dequant_rows(self.xq, self.xp, W * self.cap, n_rows)
        else:
            L.moe_permute_rows(self.recv_x.tensor.view(torch.bfloat16).view(W * self.cap, self.hidden),
                               self.order, n_rows, self.xp, 1)
        return self.xp, self.offsets, send_pos

    def combine(self, out_sorted: torch.Tensor, ids: torch.Tensor, send_pos: torch.Tensor, w: torch.Tensor,
                shared: Optional[torch.Tensor]) -> torch.Tensor:
        L, W = _lib(), self.world
        n_rows = self.offsets[self.e_local:self.e_local + 1]
        L.ep_combine_send(W, self.rank, self.ret_x.peer_ptrs, self.flags.peer_ptrs, out_sorted, self.order,
                          n_rows, self.cap)
        y = torch.empty(ids.shape[0], self.hidden, dtype=torch.bfloat16, device=out_sorted.device)
        L.ep_combine_reduce(self.ret_x.tensor, ids, send_pos, w, shared, y, self.e_local, self.cap)
        return y


class EPMoE:
    """A MoE layer whose routed experts are split across the ranks of ``ctx``."""

    def __init__(self, moe: MoE, ep: Optional[EPContext] = None, group=None):
        self.moe, self.ep = moe, ep
        self.group = group
        self.world = ep.world if ep is not None else dist.get_world_size(group)
        self.rank = ep.rank if ep is not None else dist.get_rank(group)
        self.e_local = moe.cfg.n_routed_experts // self.world
        assert moe.e_begin == self.rank * self.e_local and moe.e_end == moe.e_begin + self.e_local, \
            "the MoE must hold exactly this rank's expert slice"
        self._act = self._out = None

    @property
    def dropped(self) -> int:
        """Pairs of the last forward that exceeded the receive capacity of their owner."""
        if self.ep is None:
            return 0
        return int((self.ep.send_pos[: self.ep.last_pairs] < 0).sum().item())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        moe, cfg = self.moe, self.moe.cfg
        logits = x.float() @ moe.gate.float().t()
        ids, w = route(logits, moe.bias, cfg)
        shared = moe.shared_forward(x)
        if not x.is_cuda:
            return self._forward_host(x, ids, w, shared)
        ep, L = self.ep, _lib()
        fp8_experts = isinstance(moe.w_gate_up, Fp8ExpertWeights)
        xp, offsets, send_pos = ep.dispatch(x, ids, keep_fp8=fp8_experts)
        n = (xp[0] if isinstance(xp, tuple) else xp).shape[0]
        if self._out is None:
            self._act = (None if fp8_experts else
                         torch.empty(n, cfg.moe_intermediate_size, dtype=x.dtype, device=x.device))
            self._out = torch.empty(n, cfg.hidden_size, dtype=x.dtype, device=x.device)
        moe.local_gemms(xp, offsets, self._act, self._out)
        return ep.combine(self._out, ids, send_pos, w.contiguous(), shared)

    __call__ = forward

    # ------------------------------------------------------------------ host path (gloo)
    def _forward_host(self, x, ids, w, shared):
        """Same exchange with all_to_all: the reference semantics the kernels are tested against."""
        W, El, k = self.world, self.e_local, ids.shape[1]
        T, H = x.shape
        owner = (ids // El).flatten()                                   # [T*k]
        pair = torch.arange(T * k)
        send_rows, send_meta, send_pairs = [], [], []
        for r in range(W):
            sel = pair[owner == r]
            send_pairs.append(sel)
            send_rows.append(x[sel // k].contiguous())
            send_meta.append((ids.flatten()[sel] - r * El).to(torch.int64))
        counts = torch.tensor([len(s) for s in send_pairs], dtype=torch.int64)
        rcounts = torch.empty_like(counts)
        dist.all_to_all_single(rcounts, counts, group=self.group)
        sc, rc = [int(c) for c in counts], [int(c) for c in rcounts]
        rows = torch.empty(sum(rc), H, dtype=x.dtype)
        meta = torch.empty(sum(rc), dtype=torch.int64)
        # gloo implements only the single-tensor form of all-to-all
        dist.all_to_all_single(rows, torch.cat(send_rows), rc, sc, group=self.group)
        dist.all_to_all_single(meta, torch.cat(send_meta), rc, sc, group=self.group)
        out = torch.zeros(rows.shape[0], H, dtype=x.dtype)
        from ..ops import reference as R
        for e in range(El):
            sel = torch.nonzero(meta == e).flatten()
            if sel.numel():
                h = R.linear_swiglu(rows[sel], self.moe.w_gate_up[e])
                out[sel] = R.linear(h, self.moe.w_down[e]).to(x.dtype)
        back_all = torch.empty(sum(sc), H, dtype=x.dtype)
        dist.all_to_all_single(back_all, out, sc, rc, group=self.group)
        back = list(back_all.split(sc))
        y = torch.zeros(T, H, dtype=torch.float32)
        if shared is not None:
            y += shared.float()
        wf = w.flatten().float()
        for r in range(W):
            sel = send_pairs[r]
            if sel.numel():
                y.index_add_(0, sel // k, back[r].float() * wf[sel].unsqueeze(1))
        return y.to(x.dtype)


def shard_moe(full: MoE, rank: int, world: int) -> MoE:
    """The slice of a fully-populated MoE that ``rank`` owns (gate, bias and shared experts replicated)."""
    El = full.cfg.n_routed_experts // world
    e0 = rank * El
    return MoE(full.cfg, full.gate, full.w_gate_up[e0:e0 + El].contiguous(), full.w_down[e0:e0 + El].contiguous(),
               full.bias, full.shared_gate_up, full.shared_down, e_begin=e0, e_end=e0 + El)
