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
    """Symmetric receive / return buffers for one MoE shape, shared by all layers.

    Buffers are allocated for ``max_tokens`` tokens per rank; a step that is known to be smaller (every rank
    calls :meth:`set_step_tokens` with the same bound) addresses them with a smaller per-pair capacity, so the
    index kernels, the row moves and the GEMM grids of a decode step are sized for the decode step."""

    def __init__(self, ctx: TPContext, hidden: int, n_experts: int, top_k: int, max_tokens: int,
                 cap: Optional[int] = None, fp8_dispatch: bool = False, host_group=None, collect_load: bool = False):
        if n_experts % ctx.world:
            raise ValueError(f"{n_experts} experts cannot be split over {ctx.world} ranks")
        if hidden % 128:
            raise ValueError("hidden size must be a multiple of 128")
        self.ctx, self.world, self.rank = ctx, ctx.world, ctx.rank
        self.hidden, self.top_k = hidden, top_k
        self.e_local = n_experts // ctx.world
        if self.e_local > 128:
            raise ValueError("at most 128 experts per rank")
        self.cap = cap if cap is not None else max_tokens * top_k
        self.step_cap = self.cap
        self.step_tokens = max_tokens
        self.max_tokens = max_tokens
        self.fp8 = fp8_dispatch
        self.host_group = host_group        # a gloo group of the same ranks: per-step agreement on the bound
        self.collect_load = collect_load    # every layer adds its received rows per expert to EPMoE.load (EPLB input)
        self.row_bytes = hidden + hidden // 128 * 4 if fp8_dispatch else hidden * 2
        if self.row_bytes % 16:
            raise ValueError("fp8 dispatch needs a hidden size that is a multiple of 512 (rows move as 16-byte vectors)")
        W, L = self.world, _lib()
        self.recv_x = ctx.alloc_symmetric(W * self.cap * self.row_bytes, torch.uint8)
        self.recv_meta = ctx.alloc_symmetric(W * self.cap * 2, torch.int32, zero=True)
        self.ret_x = ctx.alloc_symmetric(W * self.cap * hidden, torch.bfloat16)
        self.flags = ctx.alloc_symmetric(L.ep_flag_ints(), torch.int32, zero=True)
        dev = ctx.device
        n = W * self.cap
        self.order = torch.empty(n, dtype=torch.int32, device=dev)
        self.offsets = torch.zeros(self.e_local + 1, dtype=torch.int32, device=dev)
        self.n_rows = self.offsets[self.e_local:self.e_local + 1]
        # rows in expert order: bf16 [n, H], or e4m3 [n, H] with group-major scales [H / 128, n]
        self.xrows = torch.empty(n * hidden * (1 if fp8_dispatch else 2), dtype=torch.uint8, device=dev)
        self.xs = torch.empty(hidden // 128 * n, dtype=torch.float32, device=dev) if fp8_dispatch else None
        self.xdq = None                      # bf16 rows for bf16 experts behind an fp8 dispatch (lazily)
        self.out = torch.empty(n, hidden, dtype=torch.bfloat16, device=dev)    # expert outputs, all layers
        self.send_pos = torch.zeros(max_tokens * top_k, dtype=torch.int32, device=dev)
        self.side = torch.cuda.Stream(device=dev)       # the shared experts run beside the exchange
        self.last_pairs = 0
        ctx.barrier()   # flags are zero everywhere before the first kernel signals a peer

    # ------------------------------------------------------------------ per-step bound
    def set_step_tokens(self, tokens: int) -> int:
        """Bound of the tokens any rank brings to the MoE layers of the coming step. Must be the same on every
        rank: with a host group the ranks agree on the maximum here, else the caller guarantees it."""
        if self.host_group is not None:
            t = torch.tensor([tokens], dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.host_group)
            tokens = int(t)
        return self.set_step_tokens_local(tokens)

    def set_step_tokens_local(self, tokens: int) -> int:
        """The same without the exchange: the caller already holds a bound that every rank shares."""
        tokens = max(1, min(int(tokens), self.max_tokens))
        self.step_tokens = tokens
        self.step_cap = min(self.cap, tokens * self.top_k)
        return tokens

    @property
    def step_rows(self) -> int:
        """Upper bound of the rows this rank can receive in a step."""
        return self.world * self.step_cap

    # ------------------------------------------------------------------ stages
    def dispatch(self, x: torch.Tensor, ids: torch.Tensor, keep_fp8: bool = False):
        """Push rows to their owners. Returns (rows in local-expert order, offsets [E_local+1], send_pos).
        With fp8 dispatch and ``keep_fp8`` the rows stay quantised: ``(xq e4m3 [n, H], xs fp32 [H/128, n])``,
        the operand form of the block-scaled grouped GEMM."""
        L, W, cap, H = _lib(), self.world, self.step_cap, self.hidden
        T = x.shape[0]
        assert T <= self.step_tokens and ids.shape[1] == self.top_k
        send_pos = self.send_pos[: T * self.top_k]
        self.last_pairs = T * self.top_k
        L.ep_dispatch(W, self.rank, self.recv_x.peer_ptrs, self.recv_meta.peer_ptrs, self.flags.peer_ptrs,
                      x, ids, send_pos, self.e_local, cap, self.fp8)
        n = W * cap
        if self.fp8:
            xq = self.xrows[: n * H].view(n, H)
            xs = self.xs[: H // 128 * n].view(H // 128, n)
            L.ep_recv_compact(self.recv_x.tensor, self.recv_meta.tensor, self.flags.tensor, W, cap, self.e_local, H,
                              True, n, self.offsets, self.order, xq, xs)
            if keep_fp8:
                return (xq.view(torch.float8_e4m3fn), xs), self.offsets, send_pos
            if self.xdq is None:
                self.xdq = torch.empty(W * self.cap, H, dtype=torch.bfloat16, device=x.device)
            xp = self.xdq[:n]
            L.dequant_fp8_group128(xq, xs, xp, self.n_rows)
            return xp, self.offsets, send_pos
        xp = self.xrows[: n * H * 2].view(torch.bfloat16).view(n, H)
        L.ep_recv_compact(self.recv_x.tensor, self.recv_meta.tensor, self.flags.tensor, W, cap, self.e_local, H,
                          False, n, self.offsets, self.order, xp, None)
        return xp, self.offsets, send_pos

    def combine(self, out_sorted: torch.Tensor, ids: torch.Tensor, send_pos: torch.Tensor, w: torch.Tensor,
                shared: Optional[torch.Tensor], residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Expert outputs back to their tokens and the weighted sum (+ shared experts, + ``residual``, which is
        then also the output: the layer's residual add happens here)."""
        L, W = _lib(), self.world
        L.ep_combine_send(W, self.rank, self.ret_x.peer_ptrs, self.flags.peer_ptrs, out_sorted, self.order,
                          self.n_rows, self.step_cap)
        y = residual if residual is not None else torch.empty(ids.shape[0], self.hidden, dtype=torch.bfloat16,
                                                              device=out_sorted.device)
        L.ep_combine_reduce(self.ret_x.tensor, ids, send_pos, w, shared, y, self.e_local, self.step_cap, residual)
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
        # rows received per local expert since the start (all ranks' tokens): the load statistic of the balancer
        self.load = (torch.zeros(self.e_local, dtype=torch.int64, device=ep.ctx.device)
                     if ep is not None and ep.collect_load else None)

    @property
    def dropped(self) -> int:
        """Pairs of the last forward that exceeded the receive capacity of their owner."""
        if self.ep is None:
            return 0
        return int((self.ep.send_pos[: self.ep.last_pairs] < 0).sum().item())

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``moe(x)``, or ``residual + moe(x)`` written into ``residual`` when one is given."""
        moe, cfg = self.moe, self.moe.cfg
        ids, w = route(moe.router_logits(x), moe.bias, cfg)
        if not x.is_cuda:
            y = self._forward_host(x, ids, w, moe.shared_forward(x))
            if residual is None:
                return y
            residual.copy_((residual.float() + y.float()).to(residual.dtype))
            return residual
        ep = self.ep
        # the shared experts need no exchange: they run on a side stream while the rows travel (reference:
        # nn/moe/expert_parallel.py:247-300 issues the shared expert between dispatch and its wait)
        shared = None
        if moe.shared_gate_up is not None:
            main = torch.cuda.current_stream()
            ep.side.wait_stream(main)
            with torch.cuda.stream(ep.side):
                shared = moe.shared_forward(x)
            shared.record_stream(main)
        fp8_experts = isinstance(moe.w_gate_up, Fp8ExpertWeights)
        xp, offsets, send_pos = ep.dispatch(x, ids, keep_fp8=fp8_experts)
        if self.load is not None:
            self.load.add_(offsets[1:self.e_local + 1] - offsets[: self.e_local])
        n = ep.step_rows
        out = ep.out[:n]
        # rows per expert: no more than one per token of any rank; a balanced router gives pairs / experts
        moe.local_gemms(xp, offsets, None, out, max_rows=min(n, self.world * ep.step_tokens),
                        expected_rows=ep.step_tokens * cfg.num_experts_per_tok // self.e_local + 1)
        if shared is not None:
            torch.cuda.current_stream().wait_stream(ep.side)
        return ep.combine(out, ids, send_pos, w.contiguous(), shared, residual)

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
