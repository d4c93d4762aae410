"""Numerics of every CUDA kernel against the fp32 PyTorch reference of the same op."""

import math

import pytest
import torch

from modular_b200 import ops
from modular_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-6)).item()


@pytest.fixture(autouse=True)
def _no_device_error():
    yield
    torch.cuda.synchronize()
    ops.check_device_error()


@pytest.mark.parametrize(
    "M,N,K",
    [(1, 128, 64), (16, 256, 128), (64, 4096, 4096), (100, 384, 520), (320, 6144, 4096),
     (257, 1000, 1024), (1024, 4096, 14336), (2048, 2048, 512)],
)
@pytest.mark.parametrize("impl", ["tiled", "persistent", "pair"])
def test_gemm_bf16(M, N, K, impl):
    torch.manual_seed(0)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    y = ops.linear(x, w, impl=impl)
    yr = ref.linear(x, w)
    assert _rel_err(y, yr) < 1e-2
    assert (y.float() - yr.float()).abs().max() <= 0.02 * yr.float().abs().max() + 1e-2


@pytest.mark.parametrize("M,N,K", [(2176, 6144, 1024), (1280, 3840, 512), (1000, 5000, 520), (4096, 4096, 256)])
def test_gemm_pair_persistent(M, N, K):
    # more tiles than pairs of SMs: the pair kernel walks over tiles with two accumulator stages
    torch.manual_seed(5)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    r = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    ops.set_gemm_pair_token_major(0)               # the weight-major kernels are the ones under test here
    try:
        for _ in range(2):
            y = ops.linear(x, w, impl="pair")
            yr = ops.linear(x, w, residual=r, impl="pair")
        ops.set_gemm_pair_persistent(False)
        y0 = ops.linear(x, w, impl="pair")
    finally:
        ops.set_gemm_pair_persistent(True)
        ops.set_gemm_pair_token_major(3)
    assert _rel_err(y, ref.linear(x, w)) < 1e-2
    assert _rel_err(yr, ref.linear(x, w, r)) < 1e-2
    assert torch.equal(y, y0)          # same tiles, same K order: bit-identical to one launch per tile
    ops.check_device_error()


@pytest.mark.parametrize("M,N,K", [(2176, 6144, 1024), (1000, 5000, 520), (4100, 4096, 256), (700, 28672, 128)])
def test_gemm_pair_token_major(M, N, K):
    # tokens on the MMA's M side: plain, residual (also in place) and fused SwiGLU, against fp32 references
    torch.manual_seed(7)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    r = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    ops.set_gemm_pair_token_major(3)
    try:
        for _ in range(2):
            y = ops.linear(x, w, impl="pair")
            yr = ops.linear(x, w, residual=r, impl="pair")
        h = r.clone()
        ops.linear(x, w, residual=h, out=h, impl="pair")
        ys = ops.linear_swiglu(x, w[: N // 256 * 256], impl="pair")
    finally:
        ops.set_gemm_pair_token_major(0)
    try:
        y_wm = ops.linear(x, w, impl="pair")           # weight-major kernels: same K order, same rounding
    finally:
        ops.set_gemm_pair_token_major(3)
    assert torch.equal(y, y_wm)
    assert _rel_err(y, ref.linear(x, w)) < 1e-2
    assert (y.float() - ref.linear(x, w).float()).abs().max() <= 0.02 * ref.linear(x, w).float().abs().max() + 1e-2
    assert _rel_err(yr, ref.linear(x, w, r)) < 1e-2
    assert torch.equal(h, yr)
    assert _rel_err(ys, ref.linear_swiglu(x, w[: N // 256 * 256])) < 1.5e-2
    ops.check_device_error()


def test_gemm_pair_persistent_swiglu():
    torch.manual_seed(6)
    M, K, I = 2176, 1024, 1536                    # 17 token tiles x 6 row pairs: more tiles than pairs of SMs
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(2 * I, K, device=DEV) * 0.05).to(torch.bfloat16)
    ops.set_gemm_pair_token_major(0)
    try:
        y = ops.linear_swiglu(x, w, impl="pair")
        ops.set_gemm_pair_persistent(False)
        y0 = ops.linear_swiglu(x, w, impl="pair", bn=128)
    finally:
        ops.set_gemm_pair_persistent(True)
        ops.set_gemm_pair_token_major(3)
    assert _rel_err(y, ref.linear_swiglu(x, w)) < 1.5e-2
    assert torch.equal(y, y0)
    ops.check_device_error()


@pytest.mark.parametrize("bn,stages,splits", [(16, 2, 1), (32, 4, 1), (64, 8, 1), (128, 4, 2), (256, 3, 4), (160, 4, 1)])
def test_gemm_tile_configs(bn, stages, splits):
    torch.manual_seed(1)
    M, N, K = 300, 512, 2048
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    y = ops.linear(x, w, bn=bn, stages=stages, splits=splits, impl="tiled")
    assert _rel_err(y, ref.linear(x, w)) < 1e-2


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("M,N,K,bn,stages", [(300, 512, 2048, 160, 4), (64, 4096, 4096, 64, 8),
                                              (1, 256, 8192, 16, 3), (700, 1024, 1024, 256, 4),
                                              (320, 6144, 4096, 0, 0), (48, 128, 16384, 48, 6),
                                              (1500, 19200, 256, 0, 0), (130, 18944, 512, 0, 0)])
def test_gemm_persistent_modes(M, N, K, bn, stages, mode):
    torch.manual_seed(11)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    r = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(3):  # repeated launches reuse the counters the kernel resets itself
        y = ops.linear(x, w, residual=r, bn=bn, stages=stages, impl="persistent", mode=mode)
    assert _rel_err(y, ref.linear(x, w, r)) < 1e-2
    y2 = ops.linear(x, w, residual=r, bn=bn, stages=stages, impl="persistent", mode=mode)
    assert torch.equal(y, y2)  # deterministic reduction order


def test_gemm_residual_and_fp32_out():
    torch.manual_seed(2)
    M, N, K = 200, 4096, 1024
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    r = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    for impl in ("tiled", "persistent", "pair"):
        y = ops.linear(x, w, residual=r, impl=impl)
        assert _rel_err(y, ref.linear(x, w, r)) < 1e-2
        # in-place residual (output aliases the residual)
        h = r.clone()
        ops.linear(x, w, residual=h, out=h, impl=impl)
        assert _rel_err(h, ref.linear(x, w, r)) < 1e-2
        yf = ops.linear(x, w, out_dtype=torch.float32, impl=impl)
        assert yf.dtype == torch.float32
        assert _rel_err(yf, x.float() @ w.float().t()) < 2e-3
    # split-K with residual
    y2 = ops.linear(x, w, residual=r, splits=4, bn=64, impl="tiled")
    assert _rel_err(y2, ref.linear(x, w, r)) < 1e-2


@pytest.mark.parametrize("impl,mode", [("tiled", -1), ("persistent", 0), ("persistent", 1), ("persistent", 2),
                                       ("pair", -1)])
@pytest.mark.parametrize("M", [1, 48, 130, 320, 512])
def test_gemm_swiglu(M, impl, mode):
    torch.manual_seed(3)
    K, I = 1024, 1408
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(2 * I, K, device=DEV) * 0.05).to(torch.bfloat16)
    y = ops.linear_swiglu(x, w, impl=impl, mode=mode)
    assert _rel_err(y, ref.linear_swiglu(x, w)) < 1.5e-2


@pytest.mark.parametrize("mbc", [False, True])
def test_rmsnorm(mbc):
    torch.manual_seed(4)
    x = torch.randn(77, 4096, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(4096, device=DEV, dtype=torch.bfloat16)
    y = ops.rms_norm(x, w, 1e-5, 0.0, mbc)
    assert _rel_err(y, ref.rms_norm(x, w, 1e-5, 0.0, mbc)) < 4e-3
    r = torch.randn_like(x)
    r2 = r.clone()
    y2, h = ops.add_rms_norm(x, r2, w, 1e-5, 0.0, mbc)
    yr, hr = ref.add_rms_norm(x, r, w, 1e-5, 0.0, mbc)
    assert torch.equal(h, hr)
    assert _rel_err(y2, yr) < 4e-3


def test_silu_mul_and_embedding():
    torch.manual_seed(5)
    gu = torch.randn(33, 2 * 1408, device=DEV, dtype=torch.bfloat16)
    assert _rel_err(ops.silu_mul(gu), ref.silu_mul(gu)) < 4e-3
    table = torch.randn(1000, 256, device=DEV, dtype=torch.bfloat16)
    ids = torch.randint(0, 1200, (50,), device=DEV)
    assert torch.equal(ops.embedding(ids, table, 100), ref.embedding(ids, table, 100))


def _make_cache(pages, n_layers, n_kv, page_size, hd):
    return torch.zeros(pages, 2, n_layers, n_kv, page_size, hd, device=DEV, dtype=torch.bfloat16)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("hd", [64, 128])
def test_rope_kv_store(interleaved, hd):
    torch.manual_seed(6)
    n_q, n_kv, T, ps = 8, 2, 37, 16
    kv = _make_cache(12, 2, n_kv, ps, hd)
    kv_ref = kv.clone()
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, device=DEV, dtype=torch.bfloat16)
    qkv_ref = qkv.clone()
    pos = torch.randint(0, 500, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(12 * ps, device=DEV)[:T].long()
    slots[3] = -1
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device=DEV).float() / hd))
    ang = torch.arange(512, device=DEV).float()[:, None] * inv[None]
    cos_sin = torch.cat([ang.cos(), ang.sin()], dim=1).contiguous()
    ops.rope_kv_store(qkv, pos, slots, cos_sin, kv[:, 0, 1], kv[:, 1, 1], n_q, n_kv, hd, interleaved)
    ref.rope_kv_store(qkv_ref, pos, slots, cos_sin, kv_ref[:, 0, 1], kv_ref[:, 1, 1], n_q, n_kv, hd, interleaved)
    assert _rel_err(qkv[:, : n_q * hd], qkv_ref[:, : n_q * hd]) < 4e-3
    assert _rel_err(kv, kv_ref) < 4e-3
    assert torch.equal(kv[:, :, 0], kv_ref[:, :, 0])


@pytest.mark.parametrize("tma", [False, True, "tc"])
@pytest.mark.parametrize("n_q,n_kv,hd,ps", [(32, 8, 128, 128), (4, 2, 64, 16), (8, 8, 128, 64), (16, 1, 64, 32),
                                            (16, 2, 64, 128), (8, 1, 128, 64), (16, 1, 128, 128), (4, 2, 128, 64)])
def test_paged_attention_mixed_batch(n_q, n_kv, hd, ps, tma):
    if tma and ps % 64:
        pytest.skip("the TMA kernel needs pages that are multiples of 64 tokens")
    if tma == "tc" and hd != 128:
        pytest.skip("the tcgen05 prefill kernel is built for head_dim 128")
    torch.manual_seed(7)
    q_lens = [1, 70, 1, 200, 33, 1]
    kv_lens = [513, 70, 64, 456, 161, 1]
    B = len(q_lens)
    max_pages = max((k + ps - 1) // ps for k in kv_lens)
    n_pages = B * max_pages + 3
    n_layers, layer = 3, 1
    kv = (torch.randn(n_pages, 2, n_layers, n_kv, ps, hd, device=DEV) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(n_pages, device=DEV)[: B * max_pages].int().view(B, max_pages)
    T = sum(q_lens)
    ld = (n_q + 2 * n_kv) * hd
    # large queries for the tcgen05 path: scores spread over many powers of two, which exercises the
    # lazy rescaling of the accumulator
    q = (torch.randn(T, ld, device=DEV) * (6.0 if tma == "tc" and n_kv == 8 else 1.0)).to(torch.bfloat16)
    qs = torch.tensor([sum(q_lens[:i]) for i in range(B)], device=DEV, dtype=torch.int32)
    ql = torch.tensor(q_lens, device=DEV, dtype=torch.int32)
    kl = torch.tensor(kv_lens, device=DEV, dtype=torch.int32)
    scale = 1.0 / math.sqrt(hd)
    from modular_b200._native import lib
    was = lib().get_attn_tc()
    lib().set_attn_tc(1 if tma == "tc" else 0)   # prefill tiles on the tcgen05 kernel, decode rows on the mma.sync kernel
    try:
        o = ops.paged_attention(q, kv[:, 0, layer], kv[:, 1, layer], perm, qs, ql, kl, n_q, n_kv, hd, scale,
                                kv=kv if tma else None, layer=layer)
        torch.cuda.synchronize()
    finally:
        lib().set_attn_tc(was)
    ops.check_device_error()
    o_ref = ref.paged_attention(q, kv[:, 0, layer], kv[:, 1, layer], perm, qs, ql, kl, n_q, n_kv, hd, scale)
    assert torch.isfinite(o.float()).all()
    assert _rel_err(o, o_ref) < 1e-2
    assert (o.float() - o_ref.float()).abs().max() < 3e-2


def test_argmax_and_sampling():
    torch.manual_seed(8)
    logits = torch.randn(9, 128256, device=DEV)
    assert torch.equal(ops.argmax(logits), logits.argmax(-1))
    # greedy through the sampler
    t0 = torch.zeros(9, device=DEV)
    assert torch.equal(ops.sample(logits, temperature=t0), logits.argmax(-1))
    # distribution check on a small vocab
    V = 50
    lg = torch.randn(1, V, device=DEV) * 2
    rows = lg.repeat(4096, 1).contiguous()
    seeds = torch.arange(4096, device=DEV, dtype=torch.int64) * 7919 + 11
    for kw in (dict(), dict(top_k=5), dict(top_p=0.7), dict(top_k=20, top_p=0.9, min_p=0.02)):
        temperature = torch.full((4096,), 0.8, device=DEV)
        args = dict(temperature=temperature, seeds=seeds, step=3)
        if "top_k" in kw:
            args["top_k"] = torch.full((4096,), kw["top_k"], device=DEV, dtype=torch.int32)
        if "top_p" in kw:
            args["top_p"] = torch.full((4096,), kw["top_p"], device=DEV)
        if "min_p" in kw:
            args["min_p"] = torch.full((4096,), kw["min_p"], device=DEV)
        s = ops.sample(rows, **args)
        emp = torch.bincount(s, minlength=V).float() / 4096
        p = ref.filtered_probs(lg[0], 0.8, kw.get("top_k", 0), kw.get("top_p", 1.0), kw.get("min_p", 0.0))
        assert (emp[p == 0] == 0).all(), kw
        assert (emp - p).abs().max() < 0.04, kw
    # full-size vocabulary: the samples stay inside the filtered support
    big = (torch.randn(1, 128256, device=DEV) * 3).repeat(512, 1).contiguous()
    sd = torch.arange(512, device=DEV, dtype=torch.int64) * 104729 + 5
    t1 = torch.ones(512, device=DEV)
    for kw in (dict(top_k=50), dict(top_p=0.6), dict(top_k=1000, top_p=0.95)):
        args = dict(temperature=t1, seeds=sd, step=1)
        if "top_k" in kw:
            args["top_k"] = torch.full((512,), kw["top_k"], device=DEV, dtype=torch.int32)
        if "top_p" in kw:
            args["top_p"] = torch.full((512,), kw["top_p"], device=DEV)
        s = ops.sample(big, **args)
        p = ref.filtered_probs(big[0], 1.0, kw.get("top_k", 0), kw.get("top_p", 1.0), 0.0)
        assert (p[s] > 0).all(), kw
        assert s.unique().numel() > 8, kw


def test_cluster_sampler_matches_one_cta_sampler():
    # the same seeds give the same uniform draw, and both kernels walk the kept set in index order: apart
    # from rounding at a bucket edge the two pick the same token
    torch.manual_seed(81)
    R, V = 96, 128256
    logits = torch.randn(R, V, device=DEV) * 2
    hot = torch.randint(0, V, (R, 40), device=DEV)
    logits.scatter_add_(1, hot, torch.rand(R, 40, device=DEV) * 9)      # a peaked head like a language model's
    seeds = torch.arange(R, device=DEV, dtype=torch.int64) * 31 + 7
    temp = torch.full((R,), 0.9, device=DEV)
    temp[::7] = 0.0                                                      # greedy rows pass through
    cases = [dict(top_k=torch.full((R,), 40, device=DEV, dtype=torch.int32)),
             dict(top_p=torch.full((R,), 0.85, device=DEV)),
             dict(min_p=torch.full((R,), 0.05, device=DEV)),
             dict(top_k=torch.randint(0, 300, (R,), device=DEV, dtype=torch.int32),
                  top_p=torch.rand(R, device=DEV) * 0.6 + 0.4, min_p=torch.rand(R, device=DEV) * 0.02),
             dict(top_k=torch.full((R,), 20000, device=DEV, dtype=torch.int32))]   # too wide: left to the other kernel
    for kw in cases:
        for lg in (logits, logits[:, :50001]):                           # second view: rows off a 16-byte boundary
            ops.set_sample_cluster(True)
            a = ops.sample(lg, temperature=temp, seeds=seeds, step=5, **kw)
            ops.set_sample_cluster(False)
            b = ops.sample(lg, temperature=temp, seeds=seeds, step=5, **kw)
            ops.set_sample_cluster(True)
            assert (a >= 0).all() and (a < lg.shape[1]).all()
            assert (a == b).float().mean() >= 0.97, (list(kw), (a != b).sum().item())
            assert torch.equal(a[::7], lg[::7].argmax(-1))
    ops.check_device_error()


def test_penalties():
    torch.manual_seed(9)
    logits = torch.randn(3, 1000, device=DEV)
    lr = logits.clone()
    tok = torch.tensor([1, 5, 9, 2, 7], device=DEV, dtype=torch.int32)
    cnt = torch.tensor([2, 0, 1, 3, 0], device=DEV, dtype=torch.int32)
    off = torch.tensor([0, 3, 3, 5], device=DEV, dtype=torch.int32)
    f = torch.tensor([0.5, 0.1, 0.2], device=DEV)
    p = torch.tensor([0.3, 0.0, 0.1], device=DEV)
    r = torch.tensor([1.2, 1.0, 1.5], device=DEV)
    ops.apply_penalties(logits, tok, cnt, off, f, p, r)
    ref.apply_penalties(lr, tok, cnt, off, f, p, r)
    assert torch.allclose(logits, lr, atol=1e-5)


def test_quant_fp8_group128():
    torch.manual_seed(20)
    x = (torch.randn(70, 1000, device=DEV) * 3).to(torch.bfloat16)
    q, s = ops.quant_fp8_group128(x)
    qr, sr = ref.quant_fp8_group128(x)
    assert torch.allclose(s, sr, rtol=1e-6, atol=0)
    # same scale -> identical codes except where the division rounds differently at a tie
    assert (q.float() != qr.float()).float().mean() < 1e-3
    deq = q.float().view(70, -1) * s.t().repeat_interleave(128, 1)[:, :1000]
    assert _rel_err(deq, x) < 0.04


@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (64, 4096, 4096), (130, 1024, 7168), (400, 2048, 1536),
                                   (96, 512, 2000)])
def test_gemm_fp8_blockscaled(M, N, K):
    torch.manual_seed(21)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    wq, ws = ref.quant_fp8_weight_block128(w)
    xq, xs = ops.quant_fp8_group128(x)
    r = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    y = ops.linear_fp8_blockscaled(xq, xs, wq, ws)
    y_ref = ref.linear_fp8_blockscaled(xq, xs, wq, ws)
    assert _rel_err(y, y_ref) < 5e-3          # same quantised operands: only summation order differs
    assert _rel_err(y, ref.linear(x, w)) < 0.06   # against the unquantised product
    y2 = ops.linear_fp8_blockscaled(xq, xs, wq, ws, residual=r)
    assert _rel_err(y2, ref.linear_fp8_blockscaled(xq, xs, wq, ws, r)) < 5e-3


def test_gemm_fp8_blockscaled_split_k_matches_single_pass():
    torch.manual_seed(22)
    M, N, K = 70, 1024, 3712          # 29 K groups: uneven splits
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    wq, ws = ref.quant_fp8_weight_block128(w)
    xq, xs = ops.quant_fp8_group128(x)
    r = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    y1 = ops.linear_fp8_blockscaled(xq, xs, wq, ws, residual=r, splits=1)
    for splits in (2, 3, 8):
        ys = ops.linear_fp8_blockscaled(xq, xs, wq, ws, residual=r, splits=splits)
        assert _rel_err(ys, y1) < 3e-3, splits
    assert _rel_err(y1, ref.linear_fp8_blockscaled(xq, xs, wq, ws, r)) < 5e-3


def test_grouped_gemm_fp8_and_fp8_experts():
    """Grouped block-scaled fp8 GEMM against per-expert references, and a MoE layer with fp8 expert weights
    against the same layer with those weights dequantised to bf16."""
    from modular_b200._native import lib
    from modular_b200.nn.moe import Fp8ExpertWeights, MoE, MoEConfig

    torch.manual_seed(23)
    E, N, K = 5, 256, 512
    counts = [40, 0, 130, 1, 64]
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    rows = sum(counts)
    x = torch.randn(rows + 7, K, device=DEV, dtype=torch.bfloat16)        # trailing rows belong to no expert
    w = (torch.randn(E, N, K, device=DEV) * 0.05).to(torch.bfloat16)
    fw = Fp8ExpertWeights.quantize(w)
    xq, xs = ops.quant_fp8_group128(x)
    y = torch.zeros(rows + 7, N, device=DEV, dtype=torch.bfloat16)
    lib().grouped_gemm_fp8(xq, xs, fw.q, fw.scale, y, offsets, rows + 7, 0)
    for e in range(E):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            # same quantised operands: xs is K-group-major over all rows
            yr = ref.linear_fp8_blockscaled(xq[a:b], xs[:, a:b].contiguous(), fw.q[e], fw.scale[e])
            assert _rel_err(y[a:b], yr) < 5e-3, e
    assert torch.all(y[rows:] == 0)

    cfg = MoEConfig(hidden_size=512, moe_intermediate_size=256, n_routed_experts=8, num_experts_per_tok=2,
                    n_shared_experts=1, n_group=4, topk_group=2, routed_scaling_factor=2.5)
    moe = MoE.random_init(cfg, DEV, torch.bfloat16, seed=5, std=0.05)
    gu8, dn8 = Fp8ExpertWeights.quantize(moe.w_gate_up), Fp8ExpertWeights.quantize(moe.w_down)
    deq = lambda f: torch.stack([f[e] for e in range(f.shape[0])]).to(torch.bfloat16)
    moe_bf16 = MoE(cfg, moe.gate, deq(gu8), deq(dn8), moe.bias, moe.shared_gate_up, moe.shared_down)
    moe_fp8 = MoE(cfg, moe.gate, gu8, dn8, moe.bias, moe.shared_gate_up, moe.shared_down)
    xt = torch.randn(77, 512, device=DEV, dtype=torch.bfloat16)
    assert _rel_err(moe_fp8(xt), moe_bf16(xt)) < 4e-2      # activations are quantised to fp8 on the fp8 path


def test_grouped_gemm_fp8_many_experts_with_row_bound():
    """The tile list of the grouped GEMM: more experts than one round of the in-kernel prefix sum covers, empty
    experts, a row count that is only an upper bound, and every token tile size."""
    from modular_b200._native import lib
    from modular_b200.nn.moe import Fp8ExpertWeights

    torch.manual_seed(24)
    E, N, K = 40, 128, 256
    g = torch.Generator().manual_seed(1)
    counts = torch.randint(0, 150, (E,), generator=g)
    counts[[3, 17, 39]] = 0
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]).to(torch.int32).to(DEV)
    rows, bound = int(counts.sum()), int(counts.sum()) + 300
    x = torch.randn(bound, K, device=DEV, dtype=torch.bfloat16)
    fw = Fp8ExpertWeights.quantize((torch.randn(E, N, K, device=DEV) * 0.05).to(torch.bfloat16))
    xq, xs = ops.quant_fp8_group128(x)
    for bn in (0, 32, 64, 128):
        y = torch.zeros(bound, N, device=DEV, dtype=torch.bfloat16)
        lib().grouped_gemm_fp8(xq, xs, fw.q, fw.scale, y, offsets, 150, bn)
        for e in range(E):
            a, b = int(offsets[e]), int(offsets[e + 1])
            if b > a:
                yr = ref.linear_fp8_blockscaled(xq[a:b], xs[:, a:b].contiguous(), fw.q[e], fw.scale[e])
                assert _rel_err(y[a:b], yr) < 5e-3, (bn, e)
        assert torch.all(y[rows:] == 0)


def test_silu_mul_quant_fp8_equals_two_passes_and_respects_row_count():
    from modular_b200._native import lib

    torch.manual_seed(25)
    M, I = 300, 512
    gu = (torch.randn(M, 2 * I, device=DEV) * 2).to(torch.bfloat16)
    q2, s2 = ops.quant_fp8_group128(ops.silu_mul(gu))
    q = torch.zeros(M, I, dtype=torch.float8_e4m3fn, device=DEV)
    s = torch.zeros(I // 128, M + 20, dtype=torch.float32, device=DEV)
    lib().silu_mul_quant_fp8(gu, q, s, None)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s[:, :M], s2)
    n_rows = torch.tensor([77], dtype=torch.int32, device=DEV)
    q.view(torch.uint8).zero_()
    s.zero_()
    lib().silu_mul_quant_fp8(gu, q, s, n_rows)
    assert torch.equal(q.view(torch.uint8)[:77], q2.view(torch.uint8)[:77]) and torch.all(q.view(torch.uint8)[77:] == 0)
    assert torch.equal(s[:, :77], s2[:, :77]) and torch.all(s[:, 77:] == 0)
    # and back: the dequantised rows are the bf16 activations to fp8 precision
    out = torch.zeros(M, I, dtype=torch.bfloat16, device=DEV)
    lib().dequant_fp8_group128(q2, s2, out, n_rows)
    assert _rel_err(out[:77], ops.silu_mul(gu)[:77]) < 0.04 and torch.all(out[77:] == 0)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("world,cap,E,counts", [(4, 64, 8, [64, 0, 17, 33]), (2, 300, 32, [299, 150]),
                                                (8, 16, 128, [1, 0, 0, 16, 5, 0, 9, 2]), (1, 2000, 5, [1777])])
def test_ep_recv_compact_sorts_received_rows_by_expert(fp8, world, cap, E, counts):
    """The receive side of the expert-parallel dispatch in one launch, checked against a stable sort of the same
    receive buffers: offsets, the order array, the rows, and (fp8) the payload / scale split."""
    from modular_b200._native import lib

    torch.manual_seed(26)
    H = 512            # fp8 rows carry H / 128 fp32 scales behind the payload and must stay 16-byte aligned
    row_bytes = H + H // 128 * 4 if fp8 else 2 * H
    recv_x = torch.randint(0, 255, (world * cap, row_bytes), dtype=torch.uint8, device=DEV)
    meta = torch.zeros(world * cap, 2, dtype=torch.int32, device=DEV)
    meta[:, 0] = torch.randint(0, E, (world * cap,), device=DEV).int()
    flags = torch.zeros(lib().ep_flag_ints(), dtype=torch.int32, device=DEV)
    flags[16:16 + world] = torch.tensor(counts, dtype=torch.int32, device=DEV)
    n = world * cap
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=DEV)
    order = torch.full((n,), -1, dtype=torch.int32, device=DEV)
    if fp8:
        xq = torch.zeros(n, H, dtype=torch.uint8, device=DEV)
        xs = torch.zeros(H // 128, n, dtype=torch.float32, device=DEV)
    else:
        xq, xs = torch.zeros(n, H, dtype=torch.bfloat16, device=DEV), None
    lib().ep_recv_compact(recv_x, meta, flags, world, cap, E, H, fp8, n, offsets, order, xq, xs)
    torch.cuda.synchronize()
    flat = torch.cat([torch.arange(c) + s * cap for s, c in enumerate(counts)]).to(DEV)
    ids = meta[flat, 0].long()
    perm = torch.sort(ids, stable=True).indices
    want_order = flat[perm].int()
    total = len(flat)
    want_off = torch.cat([torch.zeros(1, dtype=torch.long, device=DEV), torch.bincount(ids, minlength=E).cumsum(0)]).int()
    assert torch.equal(offsets, want_off)
    assert torch.equal(order[:total], want_order)
    rows = recv_x[want_order.long()]
    if fp8:
        assert torch.equal(xq[:total], rows[:, :H])
        want_s = rows[:, H:].contiguous().view(torch.float32)           # [total, H / 128]
        assert torch.equal(xs[:, :total].view(torch.int32), want_s.t().contiguous().view(torch.int32))
    else:
        assert torch.equal(xq[:total].view(torch.uint8).view(total, -1), rows)


@pytest.mark.parametrize("T,B,N,K,x_off,y_off", [(40, 8, 512, 128, 192, 512), (300, 16, 128, 512, 512, 128),
                                                 (1, 4, 64, 64, 64, 64), (2176, 4, 256, 128, 192, 300 - 300 % 8),
                                                 (32, 128, 512, 128, 192, 512), (32, 128, 128, 512, 512, 128),
                                                 (256, 16, 128, 64, 64, 136), (300, 128, 512, 128, 192, 512)])
def test_batched_gemm_addresses_heads_in_place(T, B, N, K, x_off, y_off):
    from modular_b200._native import lib

    torch.manual_seed(27)
    x = torch.randn(T, B * x_off + 8, device=DEV, dtype=torch.bfloat16)[:, : B * x_off]      # a strided view
    w = (torch.randn(B, N, K, device=DEV) * 0.1).to(torch.bfloat16)
    y = torch.full((T, B * y_off), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.batched_linear_heads(x, w, y, x_off, y_off)
    xs = torch.stack([x[:, b * x_off: b * x_off + K] for b in range(B)]).float()              # [B, T, K]
    want = torch.einsum("btk,bnk->tbn", xs, w.float())
    got = y.view(T, B, y_off)
    assert _rel_err(got[:, :, :N], want) < 1e-2
    if y_off > N:
        assert torch.all(got[:, :, N:] == 7.0)            # columns between the heads' blocks are not touched
    if T <= 256 and N % 128 == 0 and K % 64 == 0:
        # the same product as one persistent launch of the decode-step GEMM
        y2 = torch.full_like(y, 7.0)
        ops.HEADS_ON_DECODE_GEMM = True
        try:
            ops.batched_linear_heads(x, w, y2, x_off, y_off)
        finally:
            ops.HEADS_ON_DECODE_GEMM = False
        assert _rel_err(y2.view(T, B, y_off)[:, :, :N], want) < 1e-2


@pytest.mark.parametrize("T,QL", [(37, 1536), (300, 0), (1, 256)])
def test_mla_post_down_matches_composed_ops(T, QL):
    """Norms of both down-projections, key rotation and the latent-cache store in one launch."""
    from modular_b200._native import lib
    from modular_b200.nn.rotary_embedding import cos_sin_table

    torch.manual_seed(28)
    R, page, pages = 512, 16, 40
    qkv = torch.randn(T, QL + R + 64 + 8, device=DEV, dtype=torch.bfloat16)[:, : QL + R + 64]
    gq = (1 + 0.1 * torch.randn(max(QL, 8), device=DEV)).to(torch.bfloat16)
    gkv = (1 + 0.1 * torch.randn(R, device=DEV)).to(torch.bfloat16)
    cs = cos_sin_table(64, 4096, 10000.0, None, DEV)
    pos = torch.randint(0, 4096, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(page * pages, device=DEV)[:T].long()
    slots[T // 2] = -1
    cache = torch.zeros(pages, page, R + 64, device=DEV, dtype=torch.bfloat16)
    q_a = torch.zeros(T, QL, device=DEV, dtype=torch.bfloat16) if QL else None
    lib().mla_post_down(qkv, QL, gq[:QL] if QL else None, gkv, 1e-6, pos, cs, slots, q_a, cache)
    want = torch.zeros_like(cache)
    c_kv = ops.rms_norm(qkv[:, QL:QL + R].contiguous(), gkv, 1e-6)
    csp = cs[pos.long()]
    k_rope = ref.apply_rope(qkv[:, QL + R:].unsqueeze(1), csp[:, :32], csp[:, 32:], True).squeeze(1)
    ops.mla_kv_store(c_kv, k_rope, slots, want)
    assert torch.equal(cache[..., :R], want[..., :R])
    # the rotation contracts its multiply-adds differently from the op-by-op form: one bf16 ulp at most
    assert torch.allclose(cache[..., R:].float(), want[..., R:].float(), rtol=8e-3, atol=1e-3)
    if QL:
        assert torch.equal(q_a, ops.rms_norm(qkv[:, :QL].contiguous(), gq[:QL], 1e-6))
    # the query side: rotate the trailing 64 values of every head into a contiguous tensor
    h, nope = 8, 128
    q = torch.randn(T, h, nope + 64, device=DEV, dtype=torch.bfloat16)
    q_rope = torch.zeros(T, h, 64, device=DEV, dtype=torch.bfloat16)
    lib().mla_q_rope(q, h, nope, pos, cs, q_rope)
    assert torch.allclose(q_rope.float(), ref.apply_rope(q[..., nope:], csp[:, :32], csp[:, 32:], True).float(),
                          rtol=8e-3, atol=1e-3)


# ---------------------------------------------------------------------------- decode-step GEMM
@pytest.mark.parametrize("M,N,K", [(64, 1280, 8192), (128, 8192, 1024), (1, 256, 128), (200, 1024, 3584), (33, 384, 640)])
def test_gemm_decode_fp8_weights_plain_and_add_norm(M, N, K):
    """Decode-step GEMM on block-scaled fp8 weights with bf16 activations: the weight tiles are converted to scaled
    bf16 in shared memory, so the result equals the product with the dequantised weights up to bf16 rounding of the
    scaled weights."""
    torch.manual_seed(41)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    wq, wsc = ref.quant_fp8_weight_block128(w)
    wd = ref.dequant_fp8_weight_block128(wq, wsc).to(torch.bfloat16)
    for _ in range(2):
        y = ops.linear_decode(x, wq, w_scale=wsc)
        assert _rel_err(y, ref.linear(x, wd)) < 1e-2
    assert _rel_err(y, ref.linear(x, w)) < 0.05                 # against the unquantised product
    h = (torch.randn(M, N, device=DEV) * 0.5).to(torch.bfloat16)
    g = (1 + 0.1 * torch.randn(N, device=DEV)).to(torch.bfloat16)
    h2 = h.clone()
    xn, hh = ops.linear_decode(x, wq, mode="add_norm", h=h2, gamma=g, eps=1e-5, w_scale=wsc)
    want_n, want_h = ref.add_rms_norm(ref.linear(x, wd), h, g, 1e-5)
    assert _rel_err(hh, want_h) < 1e-2 and _rel_err(xn, want_n) < 2e-2
    ops.check_device_error()


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("M,N,K", [(64, 1280, 8192), (1, 256, 128), (200, 1024, 3584), (128, 8192, 1024)])
def test_gemm_decode_nvfp4_and_mxfp8_weights(fmt, M, N, K):
    """Weight-only NVFP4 (e2m1 values, e4m3 scale per 16, fp32 scale per tensor) and MXFP8 (e4m3 values, power-of-two
    scale per 32) on the decode-step GEMM: the tiles are dequantised to bf16 in shared memory, so the result equals
    the product with the dequantised weights up to the bf16 rounding of those."""
    torch.manual_seed(43)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    if fmt == "nvfp4":
        wq, bs, gs = ref.quant_nvfp4_weight(w)
        wd = ref.dequant_nvfp4_weight(wq, bs, gs)
        kw = dict(w_format="nvfp4", w_block_scale=bs, w_global_scale=gs)
        tol_q = 0.15           # 4-bit values: about 10 % relative error of the weights
    else:
        wq, bs = ref.quant_mxfp8_weight(w)
        wd = ref.dequant_mxfp8_weight(wq, bs)
        kw = dict(w_format="mxfp8", w_block_scale=bs)
        tol_q = 0.05
    wd = wd.to(torch.bfloat16)
    for _ in range(2):
        y = ops.linear_decode(x, wq, **kw)
        assert _rel_err(y, ref.linear(x, wd)) < 1e-2
    assert _rel_err(y, ref.linear(x, w)) < tol_q
    if N % 256 == 0:
        ys = ops.linear_decode(x, wq, mode="swiglu", **kw)
        assert _rel_err(ys, ref.linear_swiglu(x, wd)) < 2e-2
    h = (torch.randn(M, N, device=DEV) * 0.5).to(torch.bfloat16)
    g = (1 + 0.1 * torch.randn(N, device=DEV)).to(torch.bfloat16)
    h2 = h.clone()
    xn, hh = ops.linear_decode(x, wq, mode="add_norm", h=h2, gamma=g, eps=1e-5, **kw)
    want_n, want_h = ref.add_rms_norm(ref.linear(x, wd), h, g, 1e-5)
    assert _rel_err(hh, want_h) < 1e-2 and _rel_err(xn, want_n) < 2e-2
    ops.check_device_error()


@pytest.mark.parametrize("M,inter,K", [(64, 3584, 8192), (16, 256, 256), (130, 1792, 1024)])
def test_gemm_decode_fp8_weights_swiglu(M, inter, K):
    torch.manual_seed(42)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(2 * inter, K, device=DEV) * 0.03).to(torch.bfloat16)
    wq, wsc = ref.quant_fp8_weight_block128(w)
    wd = ref.dequant_fp8_weight_block128(wq, wsc).to(torch.bfloat16)
    y = ops.linear_decode(x, wq, mode="swiglu", w_scale=wsc)
    assert _rel_err(y, ref.linear_swiglu(x, wd)) < 2e-2
    ops.check_device_error()


@pytest.mark.parametrize("M,n_q,n_kv,K", [(64, 32, 8, 4096), (1, 4, 1, 4096), (37, 8, 2, 1024), (256, 16, 4, 512)])
def test_gemm_decode_qkv_rope_store_equals_the_two_kernels(M, n_q, n_kv, K):
    """QKV projection with rotation and cache store in its tile epilogue against decode GEMM + rope_kv_store."""
    from modular_b200._native import lib
    from modular_b200.nn.rotary_embedding import cos_sin_table

    torch.manual_seed(40)
    page, pages, hd = 16, 40, 128
    N = (n_q + 2 * n_kv) * hd
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    cs = cos_sin_table(hd, 2048, 500000.0, None, DEV)
    pos = torch.randint(0, 2048, (M,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(page * pages, device=DEV)[:M].long()
    if M > 2:
        slots[M // 2] = -1
    mk = lambda: torch.zeros(pages, 2, n_kv, page, hd, device=DEV, dtype=torch.bfloat16)
    kv_a, kv_b = mk(), mk()
    want = ops.linear_decode(x, w)
    ops.rope_kv_store(want, pos, slots, cs, kv_a[:, 0], kv_a[:, 1], n_q, n_kv, hd)
    got = torch.zeros_like(want)
    ws, state = ops.decode_gemm_workspace(DEV)
    lib().set_gemm_dec_rope(True)          # an option (off by default: it measured slower than the two kernels)
    try:
        for _ in range(2):        # the second call finds the counters cleared
            lib().gemm_dec_qkv_rope(x, w, got, pos, slots, cs, kv_b[:, 0], kv_b[:, 1], n_q, n_kv, ws, state)
    finally:
        lib().set_gemm_dec_rope(False)
    torch.cuda.synchronize()
    ops.check_device_error()
    # rotated queries and the values in the qkv buffer (the stand-alone kernel leaves the keys of that buffer
    # unrotated: attention reads keys from the cache), rotated keys and the values in the cache
    assert torch.allclose(got[:, : n_q * hd].float(), want[:, : n_q * hd].float(), rtol=8e-3, atol=2e-3)
    assert torch.equal(got[:, (n_q + n_kv) * hd:], want[:, (n_q + n_kv) * hd:])
    assert torch.allclose(kv_b.float(), kv_a.float(), rtol=8e-3, atol=2e-3)
    assert torch.equal(kv_b[:, 1], kv_a[:, 1])            # values are copied, not rotated
    # the same through the per-tile epilogue
    lib().set_gemm_dec_tile_epilogue(True)
    lib().set_gemm_dec_rope(True)
    try:
        kv_c, got2 = mk(), torch.zeros_like(want)
        lib().gemm_dec_qkv_rope(x, w, got2, pos, slots, cs, kv_c[:, 0], kv_c[:, 1], n_q, n_kv, ws, state)
        y = ops.linear_decode(x, w)
    finally:
        lib().set_gemm_dec_tile_epilogue(False)
        lib().set_gemm_dec_rope(False)
    assert torch.equal(got2, got) and torch.equal(kv_c, kv_b) and torch.equal(y, ops.linear_decode(x, w))


@pytest.mark.parametrize("M,N,K", [(64, 6144, 4096), (64, 4096, 4096), (64, 4096, 14336), (1, 8192, 8192),
                                   (16, 1024, 1024), (100, 4096, 512), (256, 4096, 1792), (33, 1536, 4160),
                                   (8, 128, 64), (129, 768, 2048)])
def test_gemm_decode_plain(M, N, K):
    torch.manual_seed(3)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    for _ in range(2):   # the second call reuses the counters the first one left behind
        y = ops.linear_decode(x, w)
        yr = ref.linear(x, w)
        assert _rel_err(y, yr) < 1e-2
        assert (y.float() - yr.float()).abs().max() <= 0.02 * yr.float().abs().max() + 1e-2


@pytest.mark.parametrize("M,I,K", [(64, 14336, 4096), (64, 1792, 4096), (17, 688, 256), (200, 3584, 1024)])
def test_gemm_decode_swiglu(M, I, K):
    torch.manual_seed(4)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(2 * I, K, device=DEV) * 0.03).to(torch.bfloat16)
    y = ops.linear_decode(x, w, mode="swiglu")
    yr = ref.linear_swiglu(x, w)
    assert _rel_err(y, yr) < 1.5e-2


@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (64, 4096, 14336), (1, 4096, 512), (130, 8192, 1024),
                                   (256, 1024, 1792), (48, 256, 688)])
@pytest.mark.parametrize("mbc", [False, True])
def test_gemm_decode_add_norm(M, N, K, mbc):
    """One rank: h += x @ w.T, xn = rms_norm(h) * gamma, against the fp32 composition."""
    torch.manual_seed(5)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.03).to(torch.bfloat16)
    h0 = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(N, device=DEV)).to(torch.bfloat16)
    for it in range(2):
        h = h0.clone()
        xn, h = ops.linear_decode(x, w, mode="add_norm", h=h, gamma=gamma, eps=1e-5, multiply_before_cast=mbc)
        hr = (h0.float() + x.float() @ w.float().t()).to(torch.bfloat16)
        xr = ref.rms_norm(hr, gamma, 1e-5, 0.0, mbc)
        assert (h.float() - hr.float()).abs().max() <= 0.02 * hr.float().abs().max() + 1e-2
        assert _rel_err(xn, xr) < 1e-2


def test_gemm_decode_chain_matches_layer_ops():
    """qkv-like, add+norm, SwiGLU, add+norm back to back on one stream (each kernel starts before its
    predecessor has finished when dependent launch is on) against the same chain from the tiled kernels."""
    torch.manual_seed(6)
    T, H, I = 64, 1024, 2816
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    h0 = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    w1 = (torch.randn(H, H, device=DEV) * 0.03).to(torch.bfloat16)
    w2 = (torch.randn(2 * I, H, device=DEV) * 0.03).to(torch.bfloat16)
    w3 = (torch.randn(H, I, device=DEV) * 0.03).to(torch.bfloat16)
    g1 = torch.ones(H, device=DEV, dtype=torch.bfloat16)
    for _ in range(3):
        h = h0.clone()
        a = ops.linear_decode(x, w1)
        xn, h = ops.linear_decode(a, w1, mode="add_norm", h=h, gamma=g1)
        act = ops.linear_decode(xn, w2, mode="swiglu")
        xn2, h = ops.linear_decode(act, w3, mode="add_norm", h=h, gamma=g1)
    hr = h0.clone()
    ar = ops.linear(x, w1)
    hr = ops.linear(ar, w1, residual=hr)
    xr = ops.rms_norm(hr, g1, 1e-5)
    actr = ops.linear_swiglu(xr, w2)
    hr = ops.linear(actr, w3, residual=hr)
    xr2 = ops.rms_norm(hr, g1, 1e-5)
    assert _rel_err(h, hr) < 1e-2 and _rel_err(xn2, xr2) < 1e-2


# ---------------------------------------------------------------------------- split-KV decode attention
@pytest.mark.parametrize("n_q,n_kv,hd,ps", [(32, 8, 128, 128), (4, 1, 128, 128), (8, 8, 128, 64), (16, 2, 64, 64),
                                            (16, 1, 128, 128)])
@pytest.mark.parametrize("case", ["uniform", "ragged", "tiny", "spec"])
@pytest.mark.parametrize("split", [True, False])
def test_paged_attention_decode_split(n_q, n_kv, hd, ps, case, split):
    """Decode-only batches through the split-KV kernel (equal KV shares per CTA, combine by the last
    contributor) and through the one-CTA-per-sequence kernel, against the fp32 reference. Covers sequences
    shorter than one share, one-token contexts, a single sequence spread over every CTA, and (spec) several
    query tokens per sequence, which fill the upper half of the packed query tile."""
    torch.manual_seed(9)
    G = n_q // n_kv
    if case == "uniform":
        kv_lens, q_lens = [1152] * 64, [1] * 64
    elif case == "ragged":
        kv_lens = [1, 63, 64, 65, 513, 2000, 17, 129, 4096, 300, 1, 777]
        q_lens = [1] * len(kv_lens)
    elif case == "tiny":
        kv_lens, q_lens = [700], [1]
    else:
        per = max(1, 16 // G)
        kv_lens = [900, 70, 300, 1500]
        q_lens = [min(per, 3), 1, min(per, 2), min(per, 4)]
    B = len(kv_lens)
    max_pages = max((k + ps - 1) // ps for k in kv_lens)
    n_pages = sum((k + ps - 1) // ps for k in kv_lens) + 3
    kv = (torch.randn(n_pages, 2, 2, n_kv, ps, hd, device=DEV) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(n_pages, device=DEV).int()
    bt = torch.zeros(B, max_pages, dtype=torch.int32, device=DEV)
    nxt = 0
    for i, k in enumerate(kv_lens):
        n = (k + ps - 1) // ps
        bt[i, :n] = perm[nxt:nxt + n]
        nxt += n
    T = sum(q_lens)
    q = torch.randn(T, (n_q + 2 * n_kv) * hd, device=DEV).to(torch.bfloat16)
    qs = torch.tensor([sum(q_lens[:i]) for i in range(B)], device=DEV, dtype=torch.int32)
    ql = torch.tensor(q_lens, device=DEV, dtype=torch.int32)
    kl = torch.tensor(kv_lens, device=DEV, dtype=torch.int32)
    scale = 1.0 / math.sqrt(hd)
    from modular_b200._native import lib
    ops.ensure_attention_split_workspace(q.device)
    lib().set_attn_split(2 if split else 0)
    try:
        outs = [ops.paged_attention(q, kv[:, 0, 1], kv[:, 1, 1], bt, qs, ql, kl, n_q, n_kv, hd, scale, kv=kv, layer=1)
                for _ in range(2)]   # the second launch finds the counters the first one reset
        torch.cuda.synchronize()
    finally:
        lib().set_attn_split(1)
    ops.check_device_error()
    o_ref = ref.paged_attention(q, kv[:, 0, 1], kv[:, 1, 1], bt, qs, ql, kl, n_q, n_kv, hd, scale)
    for o in outs:
        assert torch.isfinite(o.float()).all()
        assert _rel_err(o, o_ref) < 1e-2
        assert (o.float() - o_ref.float()).abs().max() < 3e-2
    assert torch.equal(outs[0], outs[1]), "the combine order must not depend on arrival order"
