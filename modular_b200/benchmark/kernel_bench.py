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


def bench_decode_gemm(results, tp_degrees=(1, 8), only=None):
    """Decode-step GEMMs (gemm_decode.cu) against the tiled kernels + stand-alone RMSNorm and against cuBLAS, per
    shape (L2 flushed) and as the GEMM chain of a run of layers with distinct weights (weights cold, launches
    back to back, which is what a decode step does). Shapes: Llama-3.1-8B, whole and the shard of each TP degree.
    ``only``: case names (``down_m64_tp1``; a ``_w8`` suffix runs the block-scaled fp8 weight form against the
    activation quantiser + fp8 GEMM) to run alone, a few launches each, without the chains: what a profiler is
    pointed at."""
    peaks = measured_peaks()
    bw = peaks["hbm_gbs"] * 1e9
    H, I, QKV, QD = 4096, 14336, 6144, 4096
    dev = "cuda"
    for tp in tp_degrees:
        shapes = [("qkv", QKV // tp, H, "plain"), ("o", H, QD // tp, "add_norm"),
                  ("gate_up", I // tp, H, "swiglu"), ("down", H, I // tp, "add_norm")]
        for M in (1, 16, 64, 128, 256):
            for name, N, K, mode in shapes:
                case = f"{name}_m{M}_tp{tp}"
                if only is not None and case not in only and case + "_w8" not in only:
                    continue
                rows = 2 * N if mode == "swiglu" else N
                if only is not None and case + "_w8" in only:
                    if rows % 128 or K % 128:
                        continue
                    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
                    wq, wsc = ops.reference.quant_fp8_weight_block128((torch.randn(rows, K, device=dev) * 0.02).to(torch.bfloat16))
                    h = torch.randn(M, H, device=dev, dtype=torch.bfloat16)
                    g = torch.ones(H, device=dev, dtype=torch.bfloat16)
                    xn = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
                    kw = dict(h=h, gamma=g, xn=xn) if mode == "add_norm" else {}
                    new = lambda: ops.linear_decode(x, wq, mode=mode, w_scale=wsc, **kw)
                    old = lambda: ops.linear_fp8(x, wq, wsc)
                    t_new, t_old = time_fn(new), time_fn(old)
                    nbytes = rows * K + 2.0 * (M * K + M * N)
                    rec = dict(kernel="gemm_decode_w8", name=case + "_w8", M=M, N=N, K=K, mode=mode, us=t_new * 1e6,
                               quant_plus_fp8_gemm_us=t_old * 1e6, gbs=nbytes / t_new / 1e9,
                               frac_of_measured_roofline=nbytes / bw / t_new)
                    results.append(rec)
                    print(json.dumps(rec), flush=True)
                    continue
                x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
                w = (torch.randn(rows, K, device=dev) * 0.02).to(torch.bfloat16)
                h = torch.randn(M, H, device=dev, dtype=torch.bfloat16)
                g = torch.ones(H, device=dev, dtype=torch.bfloat16)
                out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
                xn = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
                if mode == "plain":
                    new = lambda: ops.linear_decode(x, w, out=out)
                    old = lambda: ops.linear(x, w, out=out)
                    lib = lambda: torch.matmul(x, w.t(), out=out)
                elif mode == "swiglu":
                    new = lambda: ops.linear_decode(x, w, mode="swiglu", out=out)
                    old = lambda: ops.linear_swiglu(x, w, out=out)
                    lib = lambda: ops.reference.silu_mul(x @ w.t())
                else:
                    new = lambda: ops.linear_decode(x, w, mode="add_norm", h=h, gamma=g, xn=xn)
                    old = lambda: (ops.linear(x, w, residual=h, out=h), ops.rms_norm(h, g, 1e-5, out=xn))
                    lib = lambda: (torch.addmm(h, x, w.t(), out=h), ops.rms_norm(h, g, 1e-5, out=xn))
                t_new, t_old, t_lib = time_fn(new), time_fn(old), time_fn(lib)
                nbytes = 2.0 * (rows * K + M * K + M * N)
                rec = dict(kernel="gemm_decode", name=f"{name}_m{M}_tp{tp}", M=M, N=N, K=K, mode=mode, us=t_new * 1e6,
                           tiled_us=t_old * 1e6, lib_us=t_lib * 1e6, gbs=nbytes / t_new / 1e9,
                           frac_of_measured_roofline=nbytes / bw / t_new, speedup_vs_tiled=t_old / t_new,
                           speedup_vs_lib=t_lib / t_new)
                results.append(rec)
                print(json.dumps(rec), flush=True)
        if only is not None:
            continue
        # chain of 8 layers' GEMMs (no attention): us per layer
        n_layers = 8
        ws = [[(torch.randn(r, k, device=dev) * 0.02).to(torch.bfloat16)
               for (r, k) in ((QKV // tp, H), (H, QD // tp), (2 * I // tp, H), (H, I // tp))] for _ in range(n_layers)]
        g = torch.ones(H, device=dev, dtype=torch.bfloat16)
        for M in (16, 64, 128):
            h = torch.randn(M, H, device=dev, dtype=torch.bfloat16) * 0.1
            xn = torch.randn(M, H, device=dev, dtype=torch.bfloat16)
            qkv = torch.empty(M, QKV // tp, device=dev, dtype=torch.bfloat16)
            act = torch.empty(M, I // tp, device=dev, dtype=torch.bfloat16)

            def chain_new():
                for wq, wo, wg, wd in ws:
                    ops.linear_decode(xn, wq, out=qkv)
                    ops.linear_decode(qkv[:, :QD // tp], wo, mode="add_norm", h=h, gamma=g, xn=xn)
                    ops.linear_decode(xn, wg, mode="swiglu", out=act)
                    ops.linear_decode(act, wd, mode="add_norm", h=h, gamma=g, xn=xn)

            def chain_old():
                for wq, wo, wg, wd in ws:
                    ops.rms_norm(h, g, 1e-5, out=xn)
                    ops.linear(xn, wq, out=qkv)
                    ops.linear(qkv[:, :QD // tp], wo, residual=h, out=h)
                    ops.rms_norm(h, g, 1e-5, out=xn)
                    ops.linear_swiglu(xn, wg, out=act)
                    ops.linear(act, wd, residual=h, out=h)

            res = {}
            for label, fn in (("decode", chain_new), ("tiled", chain_old)):
                gr = torch.cuda.CUDAGraph()
                fn()
                torch.cuda.synchronize()
                with torch.cuda.graph(gr):
                    fn()
                res[label] = time_fn(gr.replay, flush=False) / n_layers
            wbytes = sum(w.numel() * 2 for w in ws[0])
            rec = dict(kernel="gemm_decode_chain", name=f"layer_gemms_m{M}_tp{tp}", M=M, us_per_layer=res["decode"] * 1e6,
                       tiled_us_per_layer=res["tiled"] * 1e6, weight_mb=wbytes / 1e6,
                       frac_of_measured_roofline=wbytes / bw / res["decode"], speedup_vs_tiled=res["tiled"] / res["decode"])
            results.append(rec)
            print(json.dumps(rec), flush=True)
        del ws
    torch.cuda.synchronize()
    ops.check_device_error()


def bench_attention(results, only=None):
    peaks = measured_peaks()
    hd, ps = 128, 128
    ops.ensure_attention_split_workspace("cuda")
    for name, q_lens, kv_lens, n_q, n_kv in [
        ("decode_b64_ctx1152", [1] * 64, [1152] * 64, 32, 8),
        ("decode_b64_ctx1152_tp8shard", [1] * 64, [1152] * 64, 4, 1),
        ("decode_b256_ctx1152", [1] * 256, [1152] * 256, 32, 8),
        ("decode_b16_ctx8192", [1] * 16, [8192] * 16, 32, 8),
        ("prefill_1x1024", [1024], [1024], 32, 8),
        ("prefill_8x1024", [1024] * 8, [1024] * 8, 32, 8),
        ("mixed_64dec_256pf", [1] * 64 + [256], [1152] * 64 + [768], 32, 8),
    ]:
        if only and name not in only:
            continue
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
        t_nosplit = None
        if name.startswith("decode"):
            ops._lib().set_attn_split(0)
            t_nosplit = time_fn(fn)
            ops._lib().set_attn_split(2)
            t = time_fn(fn)
            ops._lib().set_attn_split(1)
        kv_bytes = sum(kv_lens) * n_kv * hd * 2 * 2
        flops = sum(4.0 * n_q * hd * q_ * (k_ - q_ / 2) for q_, k_ in zip(q_lens, kv_lens))
        t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), kv_bytes / (peaks["hbm_gbs"] * 1e9))
        rec = dict(kernel="paged_attention", name=name, us=t * 1e6, cp_async_us=t_old * 1e6, kv_gbs=kv_bytes / t / 1e9,
                   tflops=flops / t / 1e12, frac_of_measured_roofline=t_roof / t)
        if t_nosplit is not None:
            rec["one_cta_per_seq_us"] = t_nosplit * 1e6   # `us` is the split-KV kernel for the decode rows
        results.append(rec)
        print(json.dumps(rec), flush=True)


def bench_misc(results):
    """The remaining hot kernels on DeepSeek-V3 / Llama shapes: block-scaled fp8 GEMM, grouped (MoE) GEMM,
    MLA decode attention, router, RMSNorm, RoPE + KV store, SwiGLU, sampling. Roofline = bytes (or FLOPs)
    over the measured peaks."""
    from ..nn.moe import MoEConfig, route
    peaks = measured_peaks()
    dev = "cuda"
    bw, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12

    def rec(name, t, nbytes, flops=0.0, **kw):
        roof = max(nbytes / bw, flops / tf)
        r = dict(kernel=name, us=t * 1e6, gbs=nbytes / t / 1e9, tflops=flops / t / 1e12,
                 frac_of_measured_roofline=roof / t, **kw)
        results.append(r)
        print(json.dumps(r), flush=True)

    # block-scaled fp8 GEMM (DeepSeek-V3 o_proj-like: K = 7168, N = 7168)
    for M in (64, 512):
        N, K = 7168, 7168
        w = torch.randn(N, K, device=dev) * 0.02
        wq, ws = ops.reference.quant_fp8_weight_block128(w)
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        xq, xs = ops.quant_fp8_group128(x)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        t = time_fn(lambda: ops.linear_fp8_blockscaled(xq, xs, wq, ws, out=out))
        # compute roofline uses the bf16 peak measured here (fp8 peak is not in the measured file)
        rec("gemm_fp8_blockscaled", t, N * K + M * K + 2 * M * N, 2.0 * M * N * K, M=M, N=N, K=K)
        tq = time_fn(lambda: ops.quant_fp8_group128(x))
        rec("quant_fp8_group128", tq, M * K * 3, M=M, K=K)
    # grouped GEMM: 32 local experts (EP8 of 256), moe_inter 2048, hidden 7168, 512 tokens x top-8 / 8 ranks
    E, H, I, rows = 32, 7168, 2048, 512
    offs = (torch.arange(E + 1, dtype=torch.int32) * (rows // E)).to(dev)
    xg = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
    wgu = (torch.randn(E, 2 * I, H, device=dev) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=dev) * 0.02).to(torch.bfloat16)
    act = torch.empty(rows, I, device=dev, dtype=torch.bfloat16)
    yo = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)
    L = ops._lib()
    t = time_fn(lambda: L.grouped_gemm_bf16(xg, wgu, act, offs, rows // E, True, 0))
    rec("grouped_gemm_gate_up_swiglu", t, wgu.numel() * 2 + xg.numel() * 2, 2.0 * rows * 2 * I * H, experts=E, rows=rows)
    t = time_fn(lambda: L.grouped_gemm_bf16(act, wd, yo, offs, rows // E, False, 0))
    rec("grouped_gemm_down", t, wd.numel() * 2 + act.numel() * 2, 2.0 * rows * I * H, experts=E, rows=rows)
    del wgu, wd
    # MLA decode attention: 64 sequences x 1152 tokens of latent cache, 128 heads, kv_lora 512 + rope 64
    B, ctx, h, R, page = 64, 1152, 128, 512, 128
    ppseq = ctx // page
    cache = (torch.randn(B * ppseq + 1, page, R + 64, device=dev) * 0.3).to(torch.bfloat16)
    bt = (torch.randperm(B * ppseq, device=dev) + 1).int().view(B, ppseq)
    q_lat = (torch.randn(B, h, R, device=dev) * 0.2).to(torch.bfloat16)
    q_rope = (torch.randn(B, h, 64, device=dev) * 0.2).to(torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    qs, ql, kl = i32(list(range(B))), i32([1] * B), i32([ctx] * B)
    t = time_fn(lambda: ops.mla_paged_attention(q_lat, q_rope, cache, bt, qs, ql, kl, 0.1))
    rec("mla_decode", t, B * ctx * (R + 64) * 2, 2.0 * B * h * ctx * (2 * R + 64), batch=B, ctx=ctx, heads=h)
    t = time_fn(lambda: ops.mla_paged_attention(q_lat, q_rope, cache, bt, qs, ql, kl, 0.1, decode_only=False))
    rec("mla_decode_mma_sync", t, B * ctx * (R + 64) * 2, 2.0 * B * h * ctx * (2 * R + 64), batch=B, ctx=ctx,
        heads=h)
    # router (DeepSeek-V3: 256 experts, 8 groups, top-4 groups, top-8 experts)
    cfg = MoEConfig(7168, 2048, 256, 8, 1, 8, 4, True, 2.5, "sigmoid")
    logits = torch.randn(512, 256, device=dev)
    bias = torch.randn(256, device=dev) * 0.1
    t = time_fn(lambda: route(logits, bias, cfg))
    rec("moe_router_group_limited", t, logits.numel() * 4, tokens=512)
    # elementwise kernels at a mixed-step size (320 tokens of Llama-3.1-8B)
    T, Hd = 320, 4096
    xe = torch.randn(T, Hd, device=dev, dtype=torch.bfloat16)
    g = torch.ones(Hd, device=dev, dtype=torch.bfloat16)
    oe = torch.empty_like(xe)
    t = time_fn(lambda: ops.rms_norm(xe, g, 1e-5, out=oe))
    rec("rmsnorm", t, 2 * xe.numel() * 2, rows=T, cols=Hd)
    gu = torch.randn(T, 2 * 14336, device=dev, dtype=torch.bfloat16)
    t = time_fn(lambda: ops.silu_mul(gu))
    rec("silu_mul", t, gu.numel() * 2 * 1.5, rows=T)
    n_q, n_kv, hd, ps = 32, 8, 128, 128
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, device=dev, dtype=torch.bfloat16)
    kvc = torch.zeros(8, 2, 1, n_kv, ps, hd, device=dev, dtype=torch.bfloat16)
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    slots = torch.arange(T, device=dev, dtype=torch.long) + ps
    inv = 1.0 / (500000.0 ** (torch.arange(0, hd, 2, device=dev).float() / hd))
    ang = torch.arange(4096, device=dev).float()[:, None] * inv[None]
    cs = torch.cat([ang.cos(), ang.sin()], dim=1).contiguous()
    t = time_fn(lambda: ops.rope_kv_store(qkv, pos, slots, cs, kvc[:, 0, 0], kvc[:, 1, 0], n_q, n_kv, hd, False))
    rec("rope_kv_store", t, qkv.numel() * 2 * 2, tokens=T)
    lg = torch.randn(64, 128256, device=dev)
    temp = torch.full((64,), 0.8, device=dev)
    tk = torch.full((64,), 50, device=dev, dtype=torch.int32)
    tp_ = torch.full((64,), 0.9, device=dev)
    mp = torch.zeros(64, device=dev)
    seeds = torch.arange(64, device=dev, dtype=torch.int64)
    t = time_fn(lambda: ops.sample(lg, temp, tk, tp_, mp, seeds, 1))
    rec("sample_topk_topp", t, lg.numel() * 4, rows=64, vocab=128256)
    ops.set_sample_cluster(False)
    t = time_fn(lambda: ops.sample(lg, temp, tk, tp_, mp, seeds, 1))
    rec("sample_topk_topp_one_cta_per_row", t, lg.numel() * 4, rows=64, vocab=128256)
    ops.set_sample_cluster(True)
    t = time_fn(lambda: ops.sample(lg, temp, None, tp_, None, seeds, 1))
    rec("sample_topp_only", t, lg.numel() * 4, rows=64, vocab=128256)
    t = time_fn(lambda: ops.argmax(lg))
    rec("argmax", t, lg.numel() * 4, rows=64, vocab=128256)
    torch.cuda.synchronize()
    ops.check_device_error()


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
    if "dec" in what:
        bench_decode_gemm(results, only=set(args.only.split(",")) if args.only else None)
    if "attn" in what:
        bench_attention(results, set(args.only.split(",")) if args.only else None)
    if "misc" in what:
        bench_misc(results)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
