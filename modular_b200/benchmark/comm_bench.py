"""Microbenchmarks of the kernels fused with a collective, against NCCL + separate kernels.

Run one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m modular_b200.benchmark.comm_bench [--what tp|ep|all] [--iters 20]

``tp``: one tensor-parallel half-layer of Llama-3.1-8B / 70B shapes
    fused     row-parallel GEMM with reduce-scatter pushes -> reduce+residual+RMSNorm with ready
              flags -> flag-gated column-parallel GEMM                      (3 launches, 0 barriers)
    baseline  the same tcgen05 GEMMs, NCCL reduce_scatter_tensor, add+RMSNorm kernel, NCCL
              all_gather_into_tensor                                       (5 launches)
``sweep``: N = K = 8192 sharded over the ranks, M in {1 ... 8192}: GEMM -> reduce (one fused kernel up to 256
    rows) and all-gather -> GEMM, each against NCCL + separate kernels (see ``bench_sweep``)
``ep``: MoE dispatch + combine of DeepSeek-V3 shapes (hidden 7168, top-8, 256 experts)
    fused     peer-memory dispatch / combine kernels (bf16 and fp8 payload)
    baseline  NCCL all_to_all_single of the same rows, both directions

Timing: each chain is captured into a CUDA graph (so small cases measure GPU time, not Python
launch overhead); CUDA events on the launching stream around each replay, an L2-sized buffer is
overwritten between iterations, median over iterations, max over ranks. Roofline per case:
max(FLOPs / measured bf16 peak, NVLink bytes per GPU / 770 GB/s).

Reference harness: max/kernels/benchmarks/gpu (bench_allreduce / bench_ep_*), driven by kbench.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters, flush, warmup=3, graph=True):
    """Median device time of `fn` in microseconds, max over ranks. The launches are replayed as one
    CUDA graph so that at small sizes the figure is GPU time and not Python launch overhead."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        fn = g.replay
        fn()
        torch.cuda.synchronize()
        dist.barrier()
    ts = []
    for _ in range(iters):
        flush.zero_()
        dist.barrier()          # ranks enter each iteration together, as layers of a model do
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bench_tp(args, ctx, L, peaks, flush, out):
    from .. import ops
    world, rank, dev = ctx.world, ctx.rank, ctx.device
    shapes = {"llama8b": (4096, 4096, 14336, 6144), "llama70b": (8192, 8192, 28672, 10240)}
    T_max = 2048
    for name, (H, q_dim, inter, qkv) in shapes.items():
        if q_dim % world or inter % world:
            continue
        partial_rows = T_max + world
        sym_partial = ctx.alloc_symmetric(partial_rows * H, torch.bfloat16)
        sym_xn = ctx.alloc_symmetric(T_max * H, torch.bfloat16)
        sym_flags = ctx.alloc_symmetric(L.tp_flag_ints(), torch.int32, zero=True)
        ctx.barrier()
        g = torch.Generator().manual_seed(1)
        mk = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        gamma = torch.ones(H, dtype=torch.bfloat16, device=dev)
        for case, K_local, N2, dual in (("o_proj->gate_up", q_dim // world, inter // world, True),
                                        ("down->qkv", inter // world, qkv // world, False)):
            w1 = mk(H, K_local)
            w2 = mk(N2 * (2 if dual else 1), H)
            for T in args.tokens:
                rpr = (T + world - 1) // world
                x = mk(T, K_local)
                h_local = mk(rpr, H)
                y = torch.empty(T, N2, dtype=torch.bfloat16, device=dev)
                xn_view = sym_xn.tensor[: T * H].view(T, H)
                max_slots = partial_rows // rpr

                def fused():
                    e, s = L.gemm_bf16_comm(x, w1, None, T, False, False, True, 0, 0, world, rank, rpr,
                                            sym_flags.peer_ptrs, sym_partial.peer_ptrs, max_slots)
                    L.tp_rs_norm_ag_ex(world, rank, sym_partial.peer_ptrs, sym_xn.peer_ptrs,
                                       sym_flags.peer_ptrs, h_local, gamma, T, rpr, 1e-5, True, 3, world * s, e)
                    L.gemm_bf16_comm(xn_view, w2, y, T, dual, True, False, 0, 1, world, rank, rpr,
                                     sym_flags.peer_ptrs, [], 0)

                Tp = rpr * world
                part = torch.zeros(Tp, H, dtype=torch.bfloat16, device=dev)
                mine = torch.empty(rpr, H, dtype=torch.bfloat16, device=dev)
                xn_loc = torch.empty(rpr, H, dtype=torch.bfloat16, device=dev)
                xn_all = torch.empty(Tp, H, dtype=torch.bfloat16, device=dev)
                ws = ops.gemm_workspace(dev)

                def baseline():
                    L.gemm_bf16(x, w1, part[:T], None, False, ws, 0, 0, 0)
                    dist.reduce_scatter_tensor(mine, part)
                    L.add_rmsnorm(mine, h_local, gamma, xn_loc, 1e-5, 0.0, False)
                    dist.all_gather_into_tensor(xn_all, xn_loc)
                    L.gemm_bf16(xn_all[:T], w2, y, None, dual, None, 0, 1, 0)

                t_f = _time(fused, args.iters, flush)
                t_b = _time(baseline, args.iters, flush)
                flops = 2.0 * T * H * K_local + 2.0 * T * H * N2 * (2 if dual else 1)
                link = (world - 1) / world * T * H * 2 * 2        # RS + AG bytes leaving one GPU
                bound = max(flops / (peaks["bf16_tflops"] * 1e12), link / 770e9) * 1e6
                rec = dict(kind="tp", model=name, case=case, world=world, tokens=T, fused_us=round(t_f, 1),
                           nccl_us=round(t_b, 1), speedup=round(t_b / t_f, 2), roofline_us=round(bound, 1),
                           frac_of_measured_roofline=round(bound / t_f, 3))
                out.append(rec)
                if rank == 0:
                    print(json.dumps(rec), flush=True)
            del w1, w2
        ops.check_device_error()


def bench_sweep(args, ctx, L, peaks, flush, out):
    """Square sweep N = K = 8192 (K or N sharded over the ranks), M in --sweep-tokens:

    gemm_reduce   row-parallel GEMM whose partial sums are reduced over the ranks.
                  M <= 256: ONE kernel, the decode-step GEMM with sentinel-polled all-reduce + residual + RMSNorm
                  (every rank ends with all rows); baseline: GEMM, NCCL all_reduce, add+RMSNorm kernel.
                  M > 256: GEMM with reduce-scatter pushes, then reduce + residual + RMSNorm + all-gather pushes;
                  baseline: GEMM, NCCL reduce_scatter, add+RMSNorm kernel, NCCL all_gather.
    ag_gemm       rows sharded over the ranks -> all-gather -> column-parallel GEMM: norm + pushes with ready
                  flags, GEMM tiles gated on the flags; baseline: RMSNorm kernel, NCCL all_gather, GEMM.
    """
    from .. import ops
    world, rank, dev = ctx.world, ctx.rank, ctx.device
    N = K = 8192
    if K % world:
        return
    T_max = max(args.sweep_tokens)
    partial_rows = T_max + world
    sym_partial = ctx.alloc_symmetric(partial_rows * N, torch.bfloat16)
    sym_xn = ctx.alloc_symmetric(T_max * N, torch.bfloat16)
    sym_flags = ctx.alloc_symmetric(L.tp_flag_ints(), torch.int32, zero=True)
    dec_rows = L.gemm_dec_sizes()[2]
    sym_lam = ctx.alloc_symmetric(L.gemm_dec_lamport_elems(world, dec_rows, N), torch.bfloat16)
    sym_lam.tensor.view(torch.int16).fill_(-32768)
    _, dec_state = ops.decode_gemm_workspace(dev)
    tp = dict(world=world, rank=rank, lam=sym_lam.peer_ptrs, lam_rows=dec_rows, state=dec_state)
    ctx.barrier()
    g = torch.Generator().manual_seed(2)
    mk = lambda *s_, std=0.02: (torch.randn(*s_, generator=g) * std).to(torch.bfloat16).to(dev)
    gamma = torch.ones(N, dtype=torch.bfloat16, device=dev)
    w_row = mk(N, K // world)              # row-parallel weight shard
    w_col = mk(N // world, K)              # column-parallel weight shard
    ws = ops.gemm_workspace(dev)
    for T in args.sweep_tokens:
        rpr = (T + world - 1) // world
        Tp = rpr * world
        x = mk(T, K // world, std=1.0)
        link_rs_ag = (world - 1) / world * T * N * 2 * 2
        # ---------------- GEMM -> reduce
        if T <= dec_rows:
            h = mk(T, N, std=1.0)
            xn = torch.empty(T, N, dtype=torch.bfloat16, device=dev)

            def fused():
                ops.linear_decode(x, w_row, mode="add_norm", h=h, gamma=gamma, xn=xn, tp=tp)

            part = torch.empty(T, N, dtype=torch.bfloat16, device=dev)

            def baseline():
                L.gemm_bf16(x, w_row, part, None, False, ws, 0, 0, 0)
                dist.all_reduce(part)
                L.add_rmsnorm(part, h, gamma, xn, 1e-5, 0.0, False)

            link = (world - 1) * T * N * 2           # one-shot: every rank sends its partial to every peer
            variant = "one kernel: GEMM + all-reduce + residual + RMSNorm"
        else:
            h_local = mk(rpr, N, std=1.0)
            max_slots = partial_rows // rpr

            def fused():
                e, s_ = L.gemm_bf16_comm(x, w_row, None, T, False, False, True, 0, 0, world, rank, rpr,
                                         sym_flags.peer_ptrs, sym_partial.peer_ptrs, max_slots)
                L.tp_rs_norm_ag_ex(world, rank, sym_partial.peer_ptrs, sym_xn.peer_ptrs, sym_flags.peer_ptrs,
                                   h_local, gamma, T, rpr, 1e-5, True, 1, world * s_, e)

            part = torch.zeros(Tp, N, dtype=torch.bfloat16, device=dev)
            mine = torch.empty(rpr, N, dtype=torch.bfloat16, device=dev)
            xn_loc = torch.empty(rpr, N, dtype=torch.bfloat16, device=dev)
            xn_all = torch.empty(Tp, N, dtype=torch.bfloat16, device=dev)

            def baseline():
                L.gemm_bf16(x, w_row, part[:T], None, False, ws, 0, 0, 0)
                dist.reduce_scatter_tensor(mine, part)
                L.add_rmsnorm(mine, h_local, gamma, xn_loc, 1e-5, 0.0, False)
                dist.all_gather_into_tensor(xn_all, xn_loc)

            link = link_rs_ag
            variant = "GEMM with reduce-scatter pushes + reduce/norm/all-gather kernel"
        t_f = _time(fused, args.iters, flush)
        t_b = _time(baseline, args.iters, flush)
        flops = 2.0 * T * N * (K // world)
        bound = max(flops / (peaks["bf16_tflops"] * 1e12), link / 770e9, (N * (K // world) * 2) / (peaks["hbm_gbs"] * 1e9)) * 1e6
        rec = dict(kind="sweep", case="gemm_reduce", variant=variant, world=world, M=T, N=N, K=K, fused_us=round(t_f, 1),
                   nccl_us=round(t_b, 1), speedup=round(t_b / t_f, 2), roofline_us=round(bound, 1),
                   frac_of_measured_roofline=round(bound / t_f, 3))
        out.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)
        # ---------------- all-gather -> GEMM
        h_rows = mk(rpr, N, std=1.0)
        y = torch.empty(T, N // world, dtype=torch.bfloat16, device=dev)
        xn_view = sym_xn.tensor[: T * N].view(T, N)

        def fused_ag():
            # has_partials = 0: normalise this rank's rows, push them to every rank, raise the ready flags
            L.tp_rs_norm_ag_ex(world, rank, sym_partial.peer_ptrs, sym_xn.peer_ptrs, sym_flags.peer_ptrs,
                               h_rows, gamma, T, rpr, 1e-5, False, 2, 0, 0)
            L.gemm_bf16_comm(xn_view, w_col, y, T, False, True, False, 0, 1, world, rank, rpr,
                             sym_flags.peer_ptrs, [], 0)

        xl = torch.empty(rpr, N, dtype=torch.bfloat16, device=dev)
        xa = torch.empty(Tp, N, dtype=torch.bfloat16, device=dev)

        def baseline_ag():
            L.rmsnorm(h_rows, gamma, xl, 1e-5, 0.0, False)
            dist.all_gather_into_tensor(xa, xl)
            L.gemm_bf16(xa[:T], w_col, y, None, False, ws, 0, 0, 0)

        t_f = _time(fused_ag, args.iters, flush)
        t_b = _time(baseline_ag, args.iters, flush)
        flops = 2.0 * T * (N // world) * K
        link = (world - 1) / world * T * K * 2
        bound = max(flops / (peaks["bf16_tflops"] * 1e12), link / 770e9, ((N // world) * K * 2) / (peaks["hbm_gbs"] * 1e9)) * 1e6
        rec = dict(kind="sweep", case="ag_gemm", world=world, M=T, N=N, K=K, fused_us=round(t_f, 1),
                   nccl_us=round(t_b, 1), speedup=round(t_b / t_f, 2), roofline_us=round(bound, 1),
                   frac_of_measured_roofline=round(bound / t_f, 3))
        out.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)
    ops.check_device_error()


def bench_ep(args, ctx, L, peaks, flush, out):
    from .. import ops
    from ..parallel.ep import EPContext
    world, rank, dev = ctx.world, ctx.rank, ctx.device
    H, E, k = 7168, 256, 8
    if E % world:
        return
    T_max = max(args.ep_tokens)
    for fp8 in (False, True):
        ep = EPContext(ctx, H, E, k, T_max, cap=T_max * k, fp8_dispatch=fp8)
        for T in args.ep_tokens:
            g = torch.Generator().manual_seed(10 + rank)
            x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
            ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).int().to(dev)
            w = torch.full((T, k), 1.0 / k, device=dev)

            ep.set_step_tokens_local(T)          # every rank brings T tokens: buffers addressed for T * k pairs

            def fused():
                # dispatch + receive compaction (the grouped GEMM's operands), then the combine; a bf16 buffer of
                # the same shape stands in for the expert outputs: same bytes on the wire
                xp, offsets, send_pos = ep.dispatch(x, ids, keep_fp8=fp8)
                rows = ep.out[: ep.step_rows] if fp8 else xp
                ep.combine(rows, ids, send_pos, w, None)

            # NCCL baseline: the same rows as all_to_all_single with precomputed splits
            owner = (ids // (E // world)).flatten().cpu()
            counts = torch.bincount(owner, minlength=world)
            sc = counts.tolist()
            rc_t = torch.empty(world, dtype=torch.int64, device=dev)
            dist.all_to_all_single(rc_t, counts.to(dev))
            rc = rc_t.tolist()
            order = torch.argsort(owner.to(dev), stable=True)
            send = torch.empty(sum(sc), H, dtype=torch.bfloat16, device=dev)
            recv = torch.empty(sum(rc), H, dtype=torch.bfloat16, device=dev)
            back = torch.empty(sum(sc), H, dtype=torch.bfloat16, device=dev)

            def baseline():
                torch.index_select(x, 0, order // k, out=send)
                dist.all_to_all_single(recv, send, rc, sc)
                dist.all_to_all_single(back, recv, sc, rc)

            t_f = _time(fused, args.iters, flush)
            t_b = _time(baseline, args.iters, flush) if not fp8 else float("nan")
            remote = T * k * (world - 1) / world
            link = remote * (ep.row_bytes + H * 2)                # dispatch + combine bytes leaving one GPU
            bound = link / 770e9 * 1e6
            rec = dict(kind="ep", world=world, tokens=T, fp8_dispatch=fp8, fused_us=round(t_f, 1),
                       nccl_us=None if fp8 else round(t_b, 1), roofline_us=round(bound, 1),
                       frac_of_measured_roofline=round(bound / t_f, 3))
            out.append(rec)
            if rank == 0:
                print(json.dumps(rec), flush=True)
        ops.check_device_error()
        del ep


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="all", choices=["tp", "ep", "sweep", "all"])
    ap.add_argument("--sweep-tokens", type=int, nargs="+", default=[1, 16, 64, 256, 1024, 4096, 8192])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", type=int, nargs="+", default=[64, 256, 1024, 2048])
    ap.add_argument("--ep-tokens", type=int, nargs="+", default=[64, 512])
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from .._native import lib
    from ..parallel.tp import TPContext
    from ..utils.peaks import measured_peaks

    ctx = TPContext(device=dev)
    L = lib()
    peaks = measured_peaks()
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    out = []
    if args.what in ("tp", "all"):
        bench_tp(args, ctx, L, peaks, flush, out)
    if args.what == "sweep":
        bench_sweep(args, ctx, L, peaks, flush, out)
    if args.what in ("ep", "all"):
        bench_ep(args, ctx, L, peaks, flush, out)
    if ctx.rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(out, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
