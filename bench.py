#!/usr/bin/env python
"""Headline serving benchmark: output tokens/s at fixed concurrency, with p50 TTFT / TPOT.

Workload (the reference's serving benchmark shape): Llama-3.1-8B architecture, bf16,
random-init weights, synthetic uniform-random prompts of 1024 tokens, 256 forced output
tokens (EOS ignored, greedy), closed-loop concurrency 64, 128-token KV pages.

A *step* is one concurrency-width of requests (64) served to completion, so the default
``--steps 16`` is the full 1024-request run. ``--warmup W`` first serves W x 64 requests
untimed (this also captures the CUDA graphs). The timed region is bracketed by a barrier
and ``torch.cuda.synchronize()`` on both sides.

Two numbers come out:
* ``value``  - output tokens / GPU-busy time, from CUDA events recorded around every
  scheduler step's device work (max over ranks);
* ``e2e``    - output tokens / wall time of the same run through ``LLM.generate`` (the public
  API): every step copies its packed inputs from pinned host memory (H2D) and reads the
  sampled tokens back (D2H); byte counts are taken from those copies.

Launch for N > 1: ``python -m torch.distributed.run --nnodes=1 --nproc-per-node N
--master-addr 127.0.0.1 --master-port P bench.py --gpus N ...`` (tensor parallel over NCCL
bootstrap; one rank per GPU).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def _reference_arm(args) -> int:
    """The reference (modular/modular) needs Bazel, a Mojo toolchain and a prebuilt engine
    wheel fetched from the network; none can be installed offline, so there is nothing to run."""
    marker = os.path.join(REPO, "baseline", "reference_install.json")
    why = "reference needs bazel + mojo toolchain + closed engine wheel (network); pip install from source fails offline"
    try:
        with open(marker) as f:
            why = json.load(f).get("unavailable", why)
    except Exception:  # noqa: BLE001
        pass
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def _server_arm(args, world: int, model_name: str) -> dict:
    """The same metric measured at the serving endpoint: starts ``serve`` (HTTP server + model worker, tensor
    parallel over ``world`` GPUs) as a child process and drives it with the serving benchmark client at the same
    concurrency, so HTTP, the ZMQ hop between the API and worker processes, detokenisation and SSE streaming are
    all inside the timed region."""
    import asyncio
    import socket
    import urllib.request

    from modular_b200.benchmark.benchmark_serving import run_benchmark

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s_:
        s_.bind(("127.0.0.1", 0))
        port = s_.getsockname()[1]
    preset = "preset:llama3.3-70b" if args.model == "llama70b-fp8" else "preset:llama3.1-8b"
    cmd = [sys.executable, "-m", "modular_b200.entrypoints", "serve", "--model-path", preset, "--served-model-name", model_name,
           "--devices", "gpu:" + ",".join(str(i) for i in range(world)), "--max-length", str(args.input_len + args.output_len + 8),
           "--max-batch-size", str(args.concurrency), "--max-batch-input-tokens", str(args.max_batch_input_tokens),
           "--enable-in-flight-batching", "--port", str(port), "--host", "127.0.0.1"]
    if args.model == "llama70b-fp8":
        cmd += ["--quantization-encoding", "float8_e4m3fn"]
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "0"))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_RUN_ID", "GROUP_RANK",
              "LOCAL_WORLD_SIZE", "ROLE_RANK", "ROLE_WORLD_SIZE"):
        env.pop(k, None)           # the server starts its own ranks
    import tempfile

    log = tempfile.NamedTemporaryFile("w+", suffix=".log", prefix="bench_server_", delete=False)

    def log_tail() -> str:
        try:
            log.flush()
            with open(log.name) as f:
                return " | ".join(f.read().strip().splitlines()[-3:])[-400:]
        except Exception:  # noqa: BLE001
            return ""

    proc = subprocess.Popen(cmd, cwd=REPO, env=env, stdout=log, stderr=subprocess.STDOUT)
    base = f"http://127.0.0.1:{port}"
    try:
        deadline = time.time() + 420
        while True:
            if proc.poll() is not None:
                return {"unavailable": f"server exited with code {proc.returncode} before it was ready: {log_tail()}"}
            try:
                with urllib.request.urlopen(base + "/health", timeout=2) as r:
                    if r.status == 200:
                        break
            except Exception:  # noqa: BLE001
                pass
            if time.time() > deadline:
                return {"unavailable": "server was not ready within 7 minutes"}
            time.sleep(1.0)
        conc = args.concurrency
        # every client run has a time limit: a stalled endpoint must not take the in-process numbers with it
        run = lambda n, seed: asyncio.run(asyncio.wait_for(
            run_benchmark(base, model_name, n, conc, args.input_len, args.output_len, vocab_size=128256, seed=seed),
            timeout=600))
        try:
            run(args.warmup * conc, 1)
            res = run(args.steps * conc, 2)
        except asyncio.TimeoutError:
            return {"unavailable": f"the endpoint did not finish a client run within 10 minutes: {log_tail()}"}
        if res["failed"]:
            return {"unavailable": f"{res['failed']} requests failed: {res['errors']}"}
        return {"value": res["output_token_throughput"], "unit": "tok/s", "p50_ttft_ms": res["p50_ttft_ms"],
                "p50_tpot_ms": res["p50_tpot_ms"], "p99_ttft_ms": res["p99_ttft_ms"], "p99_tpot_ms": res["p99_tpot_ms"],
                "duration_s": res["duration_s"], "completed": res["completed"],
                "path": "HTTP /v1/completions (SSE) -> API process -> ZMQ -> model worker(s)"}
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=30)
        except Exception:  # noqa: BLE001
            proc.kill()
        log.close()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def _deepseek_arm(args, defaults) -> int:
    """DeepSeek-V3 served expert-parallel: every rank holds E / N routed experts (block-scaled fp8) and a copy of
    the attention, dense and shared-expert weights, and serves its own concurrency / N requests; the ranks meet
    in the dispatch / combine kernels of every MoE layer. Device time is one pair of CUDA events around the
    whole closed-loop run on every rank, maximum over ranks."""
    import numpy as np
    import torch
    import torch.distributed as dist

    if args.warmup < 3:
        args.warmup = 3
    conc_total = 256 if args.concurrency == defaults.concurrency else args.concurrency
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from modular_b200 import _native
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.models.deepseek_v3 import DeepseekV3Config, DeepseekV3Weights
    from modular_b200.pipelines.context import SamplingParams

    _native.count_calls(True)
    cfg = DeepseekV3Config.deepseek_v3()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    conc = conc_total // world
    max_len = args.input_len + args.output_len + 8
    weights = DeepseekV3Weights.random_init_ep(cfg, rank, world, dev, torch.bfloat16, seed=0, fp8_experts=True)
    pages = conc * (-(-max_len // 128) + 1) + 16
    llm = LLM(cfg, weights, device=dev, dtype=torch.bfloat16, max_length=max_len, max_batch_size=conc,
              max_batch_input_tokens=args.max_batch_input_tokens, page_size=128, num_kv_pages=pages,
              enable_prefix_caching=False, enable_chunked_prefill=True, enable_in_flight_batching=False,
              device_graph_capture=True, graph_batch_sizes=[conc], seed=0,
              ep_size=world, ep_rank=rank, ep_fp8_dispatch=True)
    sp = SamplingParams(temperature=0.0, max_new_tokens=args.output_len, ignore_eos=True)
    rng = np.random.default_rng(1234 + rank)

    def prompts(n):
        return [rng.integers(0, cfg.vocab_size, size=args.input_len, dtype=np.int64) for _ in range(n)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # every rank runs the same number of requests of the same lengths: the schedulers take the same steps
    llm.generate(prompts(args.warmup * conc), sp, max_concurrency=conc)
    barrier()
    st = llm.pipeline.stats
    steps0, calls0, rep0 = st.steps, _native.native_calls(), llm.model.replayed_calls
    sampler = ClockSampler(local_rank)
    sampler.start()
    timed = prompts(args.steps * conc)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.perf_counter()
    ev0.record()
    prof = None
    if os.environ.get("MB200_HOST_PROFILE") and rank == 0:      # where the host spends the timed region
        import cProfile

        prof = cProfile.Profile()
        prof.enable()
    recs = llm.generate(timed, sp, max_concurrency=conc)
    if prof is not None:
        import pstats

        prof.disable()
        pstats.Stats(prof, stream=sys.stderr).sort_stats("cumulative").print_stats(45)
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    out_tokens = sum(len(r.tokens) for r in recs)
    assert out_tokens == args.steps * conc * args.output_len, (out_tokens,)
    from modular_b200 import ops

    ops.check_device_error()
    times = torch.tensor([ev0.elapsed_time(ev1) / 1e3, wall], dtype=torch.float64, device="cuda")
    total = torch.tensor([out_tokens], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(total)
    dev_s, wall = times.tolist()
    total_out = float(total)
    launches = (_native.native_calls() - calls0) + (llm.model.replayed_calls - rep0)
    if rank == 0:
        ttft = sorted(r.ttft for r in recs)
        tpot = sorted(r.tpot for r in recs)
        p = lambda a, q: a[min(len(a) - 1, int(q * len(a)))]
        full = not args.layers
        line = {
            "metric": f"output_tokens_per_s_at_concurrency_{conc_total}", "value": total_out / dev_s, "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_s / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8 e4m3 routed experts (128x128 block scales) with fp8 dispatch, bf16 elsewhere",
            "data": "synthetic uniform-random token ids; random-init N(0,0.02) weights", "impl": "ours",
            "config": {"model": "DeepSeek-V3 architecture (61L, h7168, MLA 128 heads, 256 routed experts top-8 + 1 shared, "
                                "vocab 129280)" + ("" if full else f" REDUCED TO {args.layers} LAYERS (not the named config)"),
                       "global_batch": conc_total, "seq_len": args.input_len + args.output_len,
                       "input_len": args.input_len, "output_len": args.output_len,
                       "num_requests": args.steps * conc_total, "concurrency": conc_total,
                       "parallelism": f"ep{world} + data-parallel attention ({conc} requests per rank)",
                       "kv_page_tokens": 128, "max_batch_input_tokens": args.max_batch_input_tokens,
                       "step_definition": f"{conc_total} requests served to completion (closed loop)",
                       "l2_policy": "inputs larger than L2 (each rank streams GBs of weights every iteration)"},
            "p50_ttft_ms": p(ttft, 0.5) * 1e3, "p99_ttft_ms": p(ttft, 0.99) * 1e3,
            "p50_tpot_ms": p(tpot, 0.5) * 1e3, "p99_tpot_ms": p(tpot, 0.99) * 1e3,
            "scheduler_iterations": st.steps - steps0, "graph_replays": llm.model.graph_replays,
            "clocks": clocks,
            # the device interval already contains the per-step uploads and token read-backs of the engine
            "e2e": {"value": total_out / wall, "unit": "tok/s", "wall_s": wall,
                    "note": "inputs are uploaded from host memory and sampled tokens read back every iteration"},
            "gpu_launches": launches,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--concurrency", type=int, default=64)
    ap.add_argument("--max-batch-input-tokens", type=int, default=2176)
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (marks the run invalid)")
    ap.add_argument("--no-server", action="store_true",
                    help="skip the second measurement through the HTTP serving endpoint")
    ap.add_argument("--server", action="store_true",
                    help="measure through the HTTP serving endpoint on more than one GPU too (by default only "
                         "one-GPU runs do: on N GPUs the endpoint needs a second bring-up of all ranks)")
    ap.add_argument("--model", default="llama8b", choices=["llama8b", "llama70b-fp8", "deepseek-v3"],
                    help="llama8b: the headline config (bf16, any --gpus); llama70b-fp8: Llama-3.3-70B shapes with "
                         "block-scaled fp8 weights, tensor parallel over --gpus (input 2048 / output 512 / "
                         "concurrency 128 unless given); deepseek-v3: DeepSeek-V3 shapes, fp8 routed experts, "
                         "expert parallel over --gpus with data-parallel attention (concurrency 256 over all ranks)")
    args = ap.parse_args()
    if args.model == "deepseek-v3":
        if args.impl == "reference":
            return _reference_arm(args)
        return _deepseek_arm(args, ap.parse_args([]))
    if args.model == "llama70b-fp8":
        defaults = ap.parse_args([])
        if args.input_len == defaults.input_len:
            args.input_len = 2048
        if args.output_len == defaults.output_len:
            args.output_len = 512
        if args.concurrency == defaults.concurrency:
            args.concurrency = 128
        if args.max_batch_input_tokens == defaults.max_batch_input_tokens:
            args.max_batch_input_tokens = 4224
    if args.impl == "reference":
        return _reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.models.llama3 import Llama3Config
    from modular_b200.pipelines.context import SamplingParams

    fp8 = args.model == "llama70b-fp8"
    cfg = Llama3Config.llama33_70b() if fp8 else Llama3Config.llama31_8b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    conc = args.concurrency
    max_len = args.input_len + args.output_len + 8
    weights, sharded = None, False
    if fp8:
        # 70 GB of e4m3 weights: every rank creates its own shard, quantised layer by layer
        from modular_b200.models.llama3 import Llama3Weights
        weights = Llama3Weights.random_init_shard(cfg, rank, world, f"cuda:{local_rank}", torch.bfloat16, seed=0, fp8=True)
        sharded = world > 1
    llm = LLM(cfg, weights, device=f"cuda:{local_rank}", dtype=torch.bfloat16, max_length=max_len,
              max_batch_size=conc, max_batch_input_tokens=args.max_batch_input_tokens, page_size=128,
              enable_prefix_caching=True, enable_chunked_prefill=True, enable_in_flight_batching=True,
              enable_overlap_scheduler=True, device_graph_capture=True, graph_batch_sizes=[conc],
              tp_size=world, tp_rank=rank, seed=0, weights_are_sharded=sharded)
    sp = SamplingParams(temperature=0.0, max_new_tokens=args.output_len, ignore_eos=True)
    rng = np.random.default_rng(1234)

    def prompts(n):
        return [rng.integers(0, cfg.vocab_size, size=args.input_len, dtype=np.int64) for _ in range(n)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up: W steps of `conc` requests (graph capture happened in the constructor)
    llm.generate(prompts(args.warmup * conc), sp, max_concurrency=conc)
    barrier()
    st = llm.pipeline.stats
    st0 = (st.steps, st.h2d_bytes, st.d2h_bytes, st.tokens_out, llm.pipeline.gpu_launches())
    llm.pipeline.reset_gpu_time()
    sampler = ClockSampler(local_rank)
    sampler.start()
    timed_prompts = prompts(args.steps * conc)
    barrier()
    t0 = time.perf_counter()
    recs = llm.generate(timed_prompts, sp, max_concurrency=conc)
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    gpu_busy = llm.pipeline.gpu_time_s()
    out_tokens = sum(len(r.tokens) for r in recs)
    assert out_tokens == args.steps * conc * args.output_len, (out_tokens,)
    times = torch.tensor([gpu_busy, wall], dtype=torch.float64, device="cuda")
    ranks_agree = True
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        # every rank samples from the same gathered logits: the generated ids must be identical everywhere
        import hashlib

        h = hashlib.sha256()
        for r in recs:
            h.update(np.asarray(r.tokens, dtype=np.int64).tobytes())
        digests = [None] * world
        dist.all_gather_object(digests, h.hexdigest())
        ranks_agree = all(d == digests[0] for d in digests)
        assert ranks_agree, f"tensor-parallel ranks generated different tokens: {digests}"
    gpu_busy, wall = times.tolist()
    n_sched_steps = st.steps - st0[0]
    counters = dict(h2d=st.h2d_bytes - st0[1], d2h=st.d2h_bytes - st0[2], graph_replays=st.graph_replays,
                    launches=llm.pipeline.gpu_launches() - st0[4])
    # the serving-endpoint measurement needs the GPUs: leave the process group, drop the engine, then rank 0
    # alone starts the server (which brings up its own ranks)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    server = None
    if world > 1 and not args.server and not args.no_server:
        server = {"skipped": "multi-GPU runs measure the endpoint only with --server"}
    elif not args.no_server:
        import gc

        del llm
        gc.collect()
        torch.cuda.empty_cache()
        if rank == 0:
            if world > 1:
                time.sleep(5.0)      # the other ranks' processes are exiting and returning their memory
            try:
                server = _server_arm(args, world, "bench-model")
            except Exception as e:  # noqa: BLE001
                server = {"unavailable": f"{type(e).__name__}: {e}"}
    if rank == 0:
        ttft = sorted(r.ttft for r in recs)
        tpot = sorted(r.tpot for r in recs)
        p = lambda a, q: a[min(len(a) - 1, int(q * len(a)))]
        n_sched = n_sched_steps
        value = out_tokens / gpu_busy
        e2e = out_tokens / wall
        line = {
            "metric": f"output_tokens_per_s_at_concurrency_{conc}", "value": value, "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": gpu_busy / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8 e4m3 weights (128x128 block scales) + per-token-group fp8 activations, bf16 elsewhere" if fp8 else "bf16",
            "data": "synthetic uniform-random token ids; random-init N(0,0.02) weights",
            "impl": "ours",
            "config": {"model": ("Llama-3.3-70B architecture (80L, h8192, 64q/8kv, ffn 28672, vocab 128256), fp8 block-scaled"
                                 if fp8 else "Llama-3.1-8B architecture (32L, h4096, 32q/8kv, ffn 14336, vocab 128256)")
                       + (f" DEBUG {args.layers} layers" if args.layers else ""),
                       "global_batch": conc, "seq_len": args.input_len + args.output_len,
                       "input_len": args.input_len, "output_len": args.output_len,
                       "num_requests": args.steps * conc, "concurrency": conc,
                       "parallelism": f"tp{world}", "kv_page_tokens": 128,
                       "max_batch_input_tokens": args.max_batch_input_tokens,
                       "step_definition": f"{conc} requests served to completion (closed loop)",
                       "l2_policy": "inputs larger than L2 (the rank's whole weight shard, GBs, is streamed every scheduler iteration)"},
            "p50_ttft_ms": p(ttft, 0.5) * 1e3, "p99_ttft_ms": p(ttft, 0.99) * 1e3,
            "p50_tpot_ms": p(tpot, 0.5) * 1e3, "p99_tpot_ms": p(tpot, 0.99) * 1e3,
            "total_tokens_per_s": (out_tokens + args.steps * conc * args.input_len) / wall,
            "scheduler_iterations": n_sched, "graph_replays": counters["graph_replays"],
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tok/s", "wall_s": wall,
                    "h2d_bytes_per_step": counters["h2d"] / args.steps,
                    "d2h_bytes_per_step": counters["d2h"] / args.steps},
            "server": server,
            "gpu_launches": counters["launches"],
            "ranks_agree": ranks_agree,
        }
        print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
