"""Plain PyTorch implementations of every op in :mod:`modular_b200.ops`.

They define the semantics the CUDA kernels are tested against (fp32 math, the same
rounding points) and are the execution path on CPU-only machines.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def linear(x, w, residual=None, out_dtype=None):
    y = (x.float() @ w.float().t()).to(out_dtype or x.dtype)
    if residual is not None:
        y = (y.float() + residual.float()).to(y.dtype)
    return y


def linear_swiglu(x, w_gate_up):
    inter = w_gate_up.shape[0] // 2
    g = x.float() @ w_gate_up[:inter].float().t()
    u = x.float() @ w_gate_up[inter:].float().t()
    return (F.silu(g) * u).to(x.dtype)


def rms_norm(x, w, eps, weight_offset=0.0, multiply_before_cast=False):
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    wf = w.float() + weight_offset
    if multiply_before_cast:
        return (n * wf).to(x.dtype)
    return (n.to(x.dtype).float() * wf).to(x.dtype)


def add_rms_norm(x, residual, w, eps, weight_offset=0.0, multiply_before_cast=False):
    h = (x.float() + residual.float()).to(x.dtype)
    return rms_norm(h, w, eps, weight_offset, multiply_before_cast), h


def silu_mul(gate_up):
    inter = gate_up.shape[-1] // 2
    g, u = gate_up[..., :inter].float(), gate_up[..., inter:].float()
    return (F.silu(g) * u).to(gate_up.dtype)


def embedding(ids, table, vocab_start=0):
    local = ids - vocab_start
    ok = (local >= 0) & (local < table.shape[0])
    out = table[local.clamp(0, table.shape[0] - 1)]
    return out * ok.unsqueeze(-1).to(out.dtype)


def apply_rope(x, cos, sin, interleaved=False):
    """x: [T, H, D]; cos/sin: [T, D/2]."""
    xf = x.float()
    c, s = cos.unsqueeze(1).float(), sin.unsqueeze(1).float()
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack((a * c - b * s, b * c + a * s), dim=-1).flatten(-2)
    else:
        half = x.shape[-1] // 2
        a, b = xf[..., :half], xf[..., half:]
        out = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    return out.to(x.dtype)


def rope_kv_store(qkv, positions, slots, cos_sin, k_cache, v_cache, n_q, n_kv, head_dim,
                  interleaved=False):
    """In place: rotates Q (and K) inside ``qkv`` and scatters K/V into the paged cache.

    k_cache / v_cache: [pages, n_kv, page_size, head_dim] views of one layer.
    """
    T = qkv.shape[0]
    half = head_dim // 2
    cs = cos_sin[positions.long()]
    cos, sin = cs[:, :half], cs[:, half:]
    q = qkv[:, : n_q * head_dim].view(T, n_q, head_dim)
    k = qkv[:, n_q * head_dim : (n_q + n_kv) * head_dim].view(T, n_kv, head_dim)
    v = qkv[:, (n_q + n_kv) * head_dim :].view(T, n_kv, head_dim)
    q.copy_(apply_rope(q, cos, sin, interleaved))
    k_rot = apply_rope(k, cos, sin, interleaved)
    page_size = k_cache.shape[2]
    ok = slots >= 0
    pg = torch.div(slots.clamp(min=0), page_size, rounding_mode="floor")
    off = slots.clamp(min=0) % page_size
    k_cache[pg[ok], :, off[ok]] = k_rot[ok].to(k_cache.dtype)
    v_cache[pg[ok], :, off[ok]] = v[ok].to(v_cache.dtype)


def paged_attention(q, k_cache, v_cache, block_table, q_start, q_len, kv_len, n_q, n_kv,
                    head_dim, scale):
    """Ragged causal attention over a paged cache. q: [T, >= n_q*head_dim] (row stride free)."""
    T = q.shape[0]
    out = torch.zeros(T, n_q * head_dim, dtype=q.dtype, device=q.device)
    G = n_q // n_kv
    page_size = k_cache.shape[2]
    for b in range(block_table.shape[0]):
        qs, ql, kl = int(q_start[b]), int(q_len[b]), int(kv_len[b])
        if ql == 0:
            continue
        n_pages = (kl + page_size - 1) // page_size
        pages = block_table[b, :n_pages].long()
        k = k_cache[pages].permute(1, 0, 2, 3).reshape(n_kv, -1, head_dim)[:, :kl].float()
        v = v_cache[pages].permute(1, 0, 2, 3).reshape(n_kv, -1, head_dim)[:, :kl].float()
        qq = q[qs : qs + ql, : n_q * head_dim].view(ql, n_q, head_dim).float()
        k = k.repeat_interleave(G, dim=0)
        v = v.repeat_interleave(G, dim=0)
        s = torch.einsum("qhd,hkd->hqk", qq, k) * scale
        qi = torch.arange(ql, device=q.device).unsqueeze(1) + (kl - ql)
        ki = torch.arange(kl, device=q.device).unsqueeze(0)
        s = s.masked_fill(ki > qi, float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hqk,hkd->qhd", p, v)
        out[qs : qs + ql] = o.reshape(ql, -1).to(q.dtype)
    return out


def argmax(logits):
    return logits.argmax(dim=-1)


def apply_penalties(logits, tok, cnt, offsets, freq=None, pres=None, rep=None):
    for r in range(logits.shape[0]):
        b, e = int(offsets[r]), int(offsets[r + 1])
        if e <= b:
            continue
        t = tok[b:e].long()
        c = cnt[b:e].float()
        x = logits[r, t]
        if rep is not None and float(rep[r]) != 1.0:
            x = torch.where(x > 0, x / rep[r], x * rep[r])
        f = freq[r] if freq is not None else 0.0
        p = pres[r] if pres is not None else 0.0
        x = x - (c > 0).float() * (f * c + p)
        logits[r, t] = x
    return logits


def filtered_probs(logits, temperature, top_k, top_p, min_p):
    """Probability vector the device sampler draws from (used by distribution tests)."""
    x = logits.float() / temperature
    mx = x.max()
    keep = torch.ones_like(x, dtype=torch.bool)
    if top_k and 0 < top_k < x.numel():
        kth = torch.topk(x, top_k).values[-1]
        keep &= x >= kth
    if min_p and min_p > 0:
        keep &= x >= mx + math.log(min_p)
    w = torch.where(keep, torch.exp(x - mx), torch.zeros_like(x))
    if top_p is not None and top_p < 1.0:
        order = torch.argsort(x, descending=True)
        ws = w[order]
        csum = torch.cumsum(ws, 0)
        target = top_p * ws.sum()
        # smallest prefix whose mass reaches the target (ties at the cut stay in)
        n_keep = int((csum < target).sum().item()) + 1
        thr = x[order[min(n_keep, x.numel()) - 1]]
        keep &= x >= thr
        w = torch.where(keep, w, torch.zeros_like(w))
    return w / w.sum()


def sample(logits, temperature=None, top_k=None, top_p=None, min_p=None, generator=None):
    out = torch.empty(logits.shape[0], dtype=torch.long, device=logits.device)
    for r in range(logits.shape[0]):
        T = float(temperature[r]) if temperature is not None else 1.0
        k = int(top_k[r]) if top_k is not None else 0
        if T <= 0 or k == 1:
            out[r] = logits[r].argmax()
            continue
        p = filtered_probs(logits[r], T, k, float(top_p[r]) if top_p is not None else 1.0,
                           float(min_p[r]) if min_p is not None else 0.0)
        out[r] = torch.multinomial(p, 1, generator=generator)[0]
    return out


# ------------------------------------------------------------------ block-scaled fp8
FP8_MAX = 448.0


def quant_fp8_group128(x):
    """Per-token-group (1 x 128) dynamic quantisation. Returns (q float8_e4m3fn [M, K],
    scales fp32 [ceil(K/128), M])."""
    M, K = x.shape
    G = (K + 127) // 128
    xf = torch.zeros(M, G * 128, dtype=torch.float32, device=x.device)
    xf[:, :K] = x.float()
    xg = xf.view(M, G, 128)
    scale = xg.abs().amax(-1).clamp_min(1e-12) / FP8_MAX
    q = (xg / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).view(M, G * 128)[:, :K]
    return q.to(torch.float8_e4m3fn), scale.t().contiguous()


def quant_fp8_weight_block128(w):
    """128x128 block quantisation of a weight [N, K]. Returns (q float8_e4m3fn, scales
    [ceil(N/128), ceil(K/128)]) with scale = amax / 448 (the checkpoint's ``weight_scale_inv``)."""
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    wf = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wf[:N, :K] = w.float()
    blocks = wf.view(nb, 128, kb, 128)
    scale = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12) / FP8_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(nb * 128, kb * 128)[:N, :K]
    return q.to(torch.float8_e4m3fn).contiguous(), scale.contiguous()


def dequant_fp8_weight_block128(q, scale):
    N, K = q.shape
    s = scale.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    return q.float() * s


# ---------------------------------------------------------------------------- nvfp4 (e2m1 values, e4m3 block scales)
_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def quant_nvfp4_weight(w):
    """NVFP4 quantisation of a weight [N, K] (K % 16 == 0): 4-bit e2m1 values, one e4m3 scale per 16 values along K
    and one fp32 scale per tensor. Returns (packed uint8 [N, K / 2] with the even index in the low nibble, block
    scales float8_e4m3fn [N, K / 16], global scale fp32 scalar tensor); ``w ~ e2m1 * block_scale * global_scale``.
    Reference format: the reference's nvfp4 weights (max/python/max/nn/quant_config.py, kernels
    linalg/matmul/gpu/sm100/block_scaled_matmul.mojo)."""
    N, K = w.shape
    assert K % 16 == 0
    wf = w.float()
    amax = wf.abs().amax().clamp_min(1e-12)
    g = amax / (6.0 * FP8_MAX)                                  # block scales then fit e4m3
    blocks = wf.view(N, K // 16, 16)
    bs = (blocks.abs().amax(-1) / 6.0 / g).clamp(max=FP8_MAX).to(torch.float8_e4m3fn)
    denom = (bs.float() * g).clamp_min(1e-30).unsqueeze(-1)
    x = (blocks / denom).clamp(-6.0, 6.0)
    grid = torch.tensor(_E2M1_VALUES, dtype=torch.float32, device=w.device)
    idx = (x.abs().unsqueeze(-1) - grid).abs().argmin(-1)       # nearest representable magnitude
    code = (idx | ((x < 0).long() << 3)).view(N, K).to(torch.uint8)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()
    return packed, bs.contiguous(), g.reshape(()).clone()


def dequant_nvfp4_weight(packed, block_scale, global_scale):
    N, K2 = packed.shape
    grid = torch.tensor(_E2M1_VALUES, dtype=torch.float32, device=packed.device)
    lo, hi = (packed & 0xF).long(), (packed >> 4).long()
    code = torch.stack((lo, hi), dim=-1).view(N, K2 * 2)
    val = grid[code & 7] * torch.where((code & 8) != 0, -1.0, 1.0)
    s = block_scale.float().repeat_interleave(16, 1) * global_scale.float()
    return val * s


def quant_mxfp8_weight(w):
    """MXFP8 quantisation of a weight [N, K] (K % 32 == 0): e4m3 values with one power-of-two scale per 32 values
    along K. Returns (q float8_e4m3fn [N, K], scales uint8 [N, K / 32] in ue8m0: scale = 2^(byte - 127))."""
    N, K = w.shape
    assert K % 32 == 0
    blocks = w.float().view(N, K // 32, 32)
    amax = blocks.abs().amax(-1).clamp_min(2.0 ** -120)
    e = torch.ceil(torch.log2(amax / FP8_MAX)).clamp(-127, 127)
    q = (blocks / torch.exp2(e).unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).view(N, K).to(torch.float8_e4m3fn)
    return q.contiguous(), (e + 127).to(torch.uint8).contiguous()


def dequant_mxfp8_weight(q, scale_bytes):
    s = torch.exp2(scale_bytes.float() - 127.0).repeat_interleave(32, 1)
    return q.float() * s


def linear_fp8_blockscaled(xq, xs, wq, ws, residual=None, out_dtype=torch.bfloat16):
    """fp32 emulation of the block-scaled GEMM: partial sums per 128-wide K group, scaled, added."""
    M, K = xq.shape
    N = wq.shape[0]
    G = (K + 127) // 128
    xf, wf = xq.float(), wq.float()
    y = torch.zeros(M, N, dtype=torch.float32, device=xq.device)
    wsn = ws.repeat_interleave(128, 0)[:N]                      # [N, G]
    for g in range(G):
        k0, k1 = g * 128, min(K, (g + 1) * 128)
        part = xf[:, k0:k1] @ wf[:, k0:k1].t()
        y += part * xs[g].unsqueeze(1) * wsn[:, g].unsqueeze(0)
    y = y.to(out_dtype)
    if residual is not None:
        y = (y.float() + residual.float()).to(out_dtype)
    return y


# ---------------------------------------------------------------------- multi-head latent attention
def mla_kv_store(c_kv, k_rope, slots, cache):
    """Scatter one latent row per token: cache[page, offset] = [c_kv (kv_lora_rank) | k_rope].

    cache: [pages, page_size, kv_lora_rank + rope_dim] view of one layer; slots < 0 are skipped.
    """
    page_size = cache.shape[1]
    ok = slots >= 0
    pg = torch.div(slots.clamp(min=0), page_size, rounding_mode="floor")
    off = slots.clamp(min=0) % page_size
    row = torch.cat((c_kv, k_rope), dim=-1).to(cache.dtype)
    cache[pg[ok], off[ok]] = row[ok]


def mla_paged_attention(q_lat, q_rope, cache, block_table, q_start, q_len, kv_len, scale):
    """Absorbed-form MLA over the latent cache (one shared "KV head" for all query heads).

    q_lat: [T, h, R] queries already multiplied by W_uk; q_rope: [T, h, Dr] rotated;
    cache: [pages, page_size, R + Dr]. Returns the attention output in latent space [T, h, R]
    (the caller multiplies by W_uv).
    """
    T, h, R = q_lat.shape
    out = torch.zeros(T, h, R, dtype=q_lat.dtype, device=q_lat.device)
    page_size = cache.shape[1]
    for b in range(block_table.shape[0]):
        qs, ql, kl = int(q_start[b]), int(q_len[b]), int(kv_len[b])
        if ql == 0:
            continue
        n_pages = (kl + page_size - 1) // page_size
        kv = cache[block_table[b, :n_pages].long()].reshape(-1, cache.shape[-1])[:kl].float()
        c, kr = kv[:, :R], kv[:, R:]
        s = (torch.einsum("qhr,kr->hqk", q_lat[qs:qs + ql].float(), c) +
             torch.einsum("qhd,kd->hqk", q_rope[qs:qs + ql].float(), kr)) * scale
        qi = torch.arange(ql, device=s.device).unsqueeze(1) + (kl - ql)
        ki = torch.arange(kl, device=s.device).unsqueeze(0)
        p = torch.softmax(s.masked_fill(ki > qi, float("-inf")), dim=-1)
        out[qs:qs + ql] = torch.einsum("hqk,kr->qhr", p, c).to(out.dtype)
    return out


def batched_linear(x, w):
    """x: [B, M, K], w: [B, N, K] -> [B, M, N] (per-batch ``x @ w.T``)."""
    return torch.einsum("bmk,bnk->bmn", x.float(), w.float()).to(x.dtype)
