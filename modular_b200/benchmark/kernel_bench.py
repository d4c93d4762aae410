"""Kernel micro-benchmarks: each hand-written kernel against its library baseline and roofline.

    python -m modular_b200.benchmark.kernel_bench --what gemm,attn --out results.json

Timing follows the usual hygiene: >= 3 warm-up runs, CUDA events on the launching stream,
an L2 flush (a write larger than the 126 MB L2) between timed runs, median of N.
The reference keeps the same kind of harness under max/kernels/benchmarks/gpu
(bench_matmul.mojo and the YAML shape lists).
"""

from __future__ import annotations

import argparse
import json
import math
import statistics
import sys

import torch

from .. import ops
from ..utils.peaks import measured_peaks


def _flush_l2(buf):
    buf.zero_()


def time_fn(fn, iters=10, warmup=3, flush=True):
    flush_buf = torch.empty(192 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            _flush_l2(flush_buf)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) * 1e-3)
    return statistics.median(times)


def bench_gemm(shapes, results, configs=None):
    peaks = measured_peaks()
    for name, M, N, K, mode in shapes:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        rows = 2 * N if mode == "swiglu" else N
        w = (torch.randn(rows, K, device="cuda") * 0.02).to(torch.bfloat16)
        flops = 2.0 * M * rows * K
        bytes_ = 2.0 * (M * K + rows * K + M * N)
        if mode == "swiglu":
            ours = lambda: ops.linear_swiglu(x, w)
            lib = lambda: ops.reference.silu_mul(x @ w.t())
        else:
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            ours = lambda: ops.linear(x, w, out=out)
            lib = lambda: torch.matmul(x, w.t(), out=out)
        t_ours = time_fn(ours)
        t_lib = time_fn(lib)
        if mode == "swiglu":
            t_tiled = time_fn(lambda: ops.linear_swiglu(x, w, impl="tiled"))
        else:
            t_tiled = time_fn(lambda: ops.linear(x, w, out=out, impl="tiled"))
        t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), bytes_ / (peaks["hbm_gbs"] * 1e9))
        rec = dict(kernel="gemm_bf16", name=name, M=M, N=N, K=K, mode=mode,
                   plan=list(ops._lib().gemm_plan(M, N, K, mode == "swiglu")),
                   us=t_ours * 1e6, lib_us=t_lib * 1e6, tiled_us=t_tiled * 1e6, tflops=flops / t_ours / 1e12,
                   gbs=bytes_ / t_ours / 1e9, frac_of_measured_roofline=t_roof / t_ours,
                   speedup_vs_lib=t_lib / t_ours)
        if configs:
            best = None
            for bn, st, sp in configs:
                if mode == "swiglu" and (sp > 1 or bn > 128):
                    continue
                try:
                    if mode == "swiglu":
                        t = time_fn(lambda: ops.linear_swiglu(x, w, bn=bn, stages=st), iters=5)
                    else:
                        t = time_fn(lambda: ops.linear(x, w, out=out, bn=bn, stages=st, splits=sp), iters=5)
                except Exception:  # noqa: BLE001
                    continue
                if best is None or t < best[0]:
                    best = (t, bn, st, sp)
            rec["best_cfg"] = dict(us=best[0] * 1e6, bn=best[1], stages=best[2], splits=best[3])
        results.append(rec)
        print(json.dumps(rec), flush=True)
    torch.cuda.synchronize()
    ops.check_device_error()


def bench_attention(results):
    peaks = measured_peaks()
    n_q, n_kv, hd, ps = 32, 8, 128, 128
    for name, q_lens, kv_lens in [
        ("decode_b64_ctx1152", [1] * 64, [1152] * 64),
        ("decode_b256_ctx1152", [1] * 256, [1152] * 256),
        ("prefill_1x1024", [1024], [1024]),
        ("prefill_8x1024", [1024] * 8, [1024] * 8),
        ("mixed_64dec_256pf", [1] * 64 + [256], [1152] * 64 + [768]),
    ]:
        B = len(q_lens)
        max_pages = max((k + ps - 1) // ps for k in kv_lens)
        n_pages = B * max_pages
        kv = (torch.randn(n_pages, 2, 1, n_kv, ps, hd, device="cuda") * 0.5).to(torch.bfloat16)
        bt = torch.randperm(n_pages, device="cuda").int().view(B, max_pages)
        T = sum(q_lens)
        q = torch.randn(T, (n_q + 2 * n_kv) * hd, device="cuda", dtype=torch.bfloat16)
        qs = torch.tensor([sum(q_lens[:i]) for i in range(B)], device="cuda", dtype=torch.int32)
        ql = torch.tensor(q_lens, device="cuda", dtype=torch.int32)
        kl = torch.tensor(kv_lens, device="cuda", dtype=torch.int32)
        ts, t0, ds = ops.build_attention_plan(q_lens, n_q, n_kv)
        plan = tuple(torch.from_numpy(a).cuda() if a.size else None for a in (ts, t0, ds))
        out = torch.empty(T, n_q * hd, device="cuda", dtype=torch.bfloat16)
        fn = lambda: ops.paged_attention(q, kv[:, 0, 0], kv[:, 1, 0], bt, qs, ql, kl, n_q, n_kv,
                                         hd, 1 / math.sqrt(hd), plan=plan, out=out, kv=kv, layer=0)
        fn_old = lambda: ops.paged_attention(q, kv[:, 0, 0], kv[:, 1, 0], bt, qs, ql, kl, n_q, n_kv,
                                             hd, 1 / math.sqrt(hd), plan=plan, out=out)
        t = time_fn(fn)
        t_old = time_fn(fn_old)
        kv_bytes = sum(kv_lens) * n_kv * hd * 2 * 2
        flops = sum(4.0 * n_q * hd * q_ * (k_ - q_ / 2) for q_, k_ in zip(q_lens, kv_lens))
        t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), kv_bytes / (peaks["hbm_gbs"] * 1e9))
        rec = dict(kernel="paged_attention", name=name, us=t * 1e6, cp_async_us=t_old * 1e6, kv_gbs=kv_bytes / t / 1e9,
                   tflops=flops / t / 1e12, frac_of_measured_roofline=t_roof / t)
        results.append(rec)
        print(json.dumps(rec), flush=True)


LLAMA8B_SHAPES = []
for _m in (16, 64, 128, 320, 512, 1024, 4096):
    LLAMA8B_SHAPES += [
        (f"qkv_m{_m}", _m, 6144, 4096, "plain"),
        (f"o_m{_m}", _m, 4096, 4096, "plain"),
        (f"gate_up_m{_m}", _m, 14336, 4096, "swiglu"),
        (f"down_m{_m}", _m, 4096, 14336, "plain"),
    ]
LLAMA8B_SHAPES += [("lm_head_m64", 64, 128256, 4096, "plain"), ("square_8192", 8192, 8192, 8192, "plain")]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,attn")
    ap.add_argument("--out", default=None)
    ap.add_argument("--sweep", action="store_true", help="also sweep tile configs per shape")
    ap.add_argument("--only", default=None, help="comma-separated GEMM shape names to run")
    args = ap.parse_args(argv)
    results = []
    what = set(args.what.split(","))
    if "gemm" in what:
        cfgs = None
        if args.sweep:
            cfgs = [(bn, st, sp) for bn in (16, 32, 64, 96, 128, 160, 192, 256) for st in (3, 4, 6, 8)
                    for sp in (1, 2, 4)]
        shapes = LLAMA8B_SHAPES
        if args.only:
            keep = set(args.only.split(","))
            shapes = [s for s in shapes if s[0] in keep]
        bench_gemm(shapes, results, cfgs)
    if "attn" in what:
        bench_attention(results)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
