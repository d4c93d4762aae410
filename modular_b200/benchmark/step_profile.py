"""Time one scheduler step of a Llama-shaped model in isolation.

    python -m modular_b200.benchmark.step_profile --layers 32 --decode 64 --ctx 1152 \
        --prefill 256 --prefill-offset 512 --iters 20

Builds the model with random weights, fabricates a batch in a given state (``--decode``
single-token sequences with ``--ctx`` tokens of context plus one prefill chunk of
``--prefill`` tokens that already has ``--prefill-offset`` tokens cached) and replays that
exact step, so kernel work can be timed (CUDA events) or listed (ncu with
``--metrics gpu__time_duration.sum``) without a serving loop around it. KV contents are
whatever the allocator left - only the shapes matter here.
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys

import numpy as np
import torch

from ..kv_cache import KVCacheParams, PagedKVCacheManager
from ..models.llama3 import Llama3Config, Llama3Model, Llama3Weights
from ..pipelines.batch import BatchPacker
from ..pipelines.context import TextContext
from .. import ops


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=0, help="0 = the model's own count")
    ap.add_argument("--model", default="llama8b", choices=["llama8b", "llama70b"])
    ap.add_argument("--fp8", action="store_true", help="block-scaled fp8 projection weights (shard-size random init)")
    ap.add_argument("--decode", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1152)
    ap.add_argument("--prefill", type=int, default=256)
    ap.add_argument("--prefill-offset", type=int, default=512)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--graph", action="store_true", help="replay the step as a CUDA graph")
    ap.add_argument("--out", default=None)
    ap.add_argument("--breakdown", action="store_true",
                    help="also time every kernel group of the step with events (eager launches)")
    args = ap.parse_args(argv)

    import os
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = Llama3Config.llama33_70b() if args.model == "llama70b" else Llama3Config.llama31_8b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    shard_init = args.fp8 or args.model == "llama70b"      # too large (or fp8): created at shard size
    if not shard_init:
        w = Llama3Weights.random_init(cfg, dev, torch.bfloat16, seed=0)
    tp = None
    if world > 1:
        # launched with torch.distributed.run: one tensor-parallel rank per process
        import torch.distributed as dist
        from ..parallel.tp import TPContext, shard_llama_config, shard_llama_weights
        dist.init_process_group("nccl", device_id=dev)
        tp = TPContext(device=dev)
    if shard_init:
        w = Llama3Weights.random_init_shard(cfg, rank, world, dev, torch.bfloat16, seed=0, fp8=args.fp8)
    if world > 1:
        full_cfg = cfg
        if not shard_init:
            w = shard_llama_weights(full_cfg, w, rank, world)
        cfg = shard_llama_config(full_cfg, world)
        torch.cuda.empty_cache()
    page = 128
    n_seq = args.decode + (1 if args.prefill else 0)
    pages_per_seq = (max(args.ctx, args.prefill_offset + args.prefill) + page) // page + 1
    kvp = KVCacheParams(cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.head_dim, page,
                        torch.bfloat16, False, False)
    kv = PagedKVCacheManager(kvp, n_seq * pages_per_seq + 2, dev, max_seq_len=pages_per_seq * page)
    T = args.decode + args.prefill
    model = Llama3Model(cfg, w, kv.kv, max_tokens=max(T, 2176), max_seqs=max(n_seq, 1),
                        max_position=pages_per_seq * page, tp=tp)
    packer = BatchPacker(cfg.num_attention_heads, cfg.num_key_value_heads, page, max(T, 16),
                         max(n_seq, 1), kv.max_pages_per_seq, device=dev)
    rng = np.random.default_rng(0)
    ctxs = []
    for i in range(args.decode):
        c = TextContext.from_prompt(rng.integers(0, cfg.vocab_size, size=args.ctx), 1 << 20, f"d{i}")
        kv.claim(c)
        kv.alloc(c)
        c.tokens.processed = args.ctx - 1
        ctxs.append(c)
    if args.prefill:
        n = args.prefill_offset + args.prefill
        c = TextContext.from_prompt(rng.integers(0, cfg.vocab_size, size=n + 1), 1 << 20, "p0")
        kv.claim(c)
        kv.alloc(c)
        c.tokens.processed = args.prefill_offset
        c.tokens.active_end = n
        ctxs.append(c)
    sb = packer.pack(ctxs, kv)
    meta = packer.upload(sb)
    call = lambda: model.forward_packed(meta, sb.offsets, sb.T, sb.B, sb.bt_stride, sb.n_tiles,
                                        sb.n_decode, sb.n_logits, False, True, 1)
    for _ in range(args.warmup):
        call()
    torch.cuda.synchronize()
    if args.graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            call()
        run = g.replay
    else:
        run = call
    times = []
    n0 = model.executor.launches()
    for _ in range(args.iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        run()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    ops.check_device_error()
    if tp is not None:
        # a multi-GPU step lasts as long as its slowest rank
        import torch.distributed as dist
        tt = torch.tensor(times, dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        times = tt.tolist()
    breakdown = None
    if args.breakdown:
        model.executor.set_profiling(True)
        for _ in range(3):
            if tp is not None:
                tp.barrier()
            call()
        torch.cuda.synchronize()
        breakdown = {name: dict(calls_per_step=n // 3, us_per_call=round(ms * 1e3 / n, 2),
                                ms_per_step=round(ms / 3, 3))
                     for name, n, ms in model.executor.profile()}
        model.executor.set_profiling(False)
    rec = dict(world=world, rank=rank, breakdown=breakdown, layers=args.layers, decode=args.decode, ctx=args.ctx, prefill=args.prefill,
               tokens=sb.T, graph=args.graph, ms_median=statistics.median(times), ms_min=min(times),
               launches_per_step=(model.executor.launches() - n0) // max(1, args.iters) if not args.graph else None,
               gemm_impl=ops.GEMM_IMPL)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if tp is not None:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if args.out and rank == 0:
        with open(args.out, "a") as f:
            f.write(json.dumps(rec) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
