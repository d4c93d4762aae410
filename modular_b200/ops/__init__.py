"""Op layer: one Python function per kernel.

CUDA tensors go to the hand-written sm_100a kernels in ``modular_b200/_C.so``; CPU tensors
go to the PyTorch reference in :mod:`modular_b200.ops.reference`. A CUDA tensor with no
loadable native library raises - there is no eager-PyTorch fallback on a GPU.

The set mirrors the custom-op wrappers the reference's layers call
(max/python/max/nn/kernels.py: fused_qkv_ragged_matmul, rope_split_store_ragged,
flash_attention_ragged, rms_norm, topk_fused_sampling, apply_penalties_to_logits, ...).
"""

from __future__ import annotations

import os

import numpy as np
import torch

from .._native import lib as _lib
from . import reference as ref

__all__ = [
    "linear", "linear_swiglu", "rms_norm", "add_rms_norm", "silu_mul", "embedding",
    "rope_kv_store", "paged_attention", "build_attention_plan", "argmax", "sample",
    "apply_penalties", "gemm_workspace", "check_device_error", "linear_decode", "decode_gemm_workspace",
]

_WORKSPACES: dict[int, torch.Tensor] = {}
_WORKSPACE_BYTES = 64 << 20


def gemm_workspace(device) -> torch.Tensor:
    """Per-device fp32 scratch for split-K partial sums (allocated once, 64 MiB)."""
    idx = torch.device(device).index or 0
    ws = _WORKSPACES.get(idx)
    if ws is None:
        ws = torch.empty(_WORKSPACE_BYTES // 4, dtype=torch.float32, device=device)
        _WORKSPACES[idx] = ws
    return ws


def check_device_error() -> None:
    """Raises if a kernel reported a timed-out wait (reads and clears the error word)."""
    code = _lib().read_error_flag(True)
    if code:
        raise RuntimeError(f"modular_b200 kernel reported a bounded-wait timeout (code {code})")


_PERSISTENT_WS: dict[int, tuple] = {}
# "auto" (default): per-shape choice; "persistent": one CTA per SM with stream-K work split;
# "tiled": one CTA per output tile with optional split-K through a workspace;
# "pair": the tiled kernel on clusters of two CTAs (cta_group::2 MMAs, 256 weight rows per pair).
GEMM_IMPL = os.environ.get("MB200_GEMM", "auto")
PAIR_MIN_TOKENS = 512   # "auto": plain and fused SwiGLU GEMMs of at least this many rows run on CTA pairs


def persistent_gemm_workspace(device):
    """(fp32 partial-tile slots, zeroed int32 tile counters) of the persistent GEMM; one pair
    per device, to be used from one stream at a time."""
    idx = torch.device(device).index or 0
    ws = _PERSISTENT_WS.get(idx)
    if ws is None:
        nbytes, nints = _lib().gemm_persistent_sizes()
        ws = (torch.empty(nbytes // 4, dtype=torch.float32, device=device),
              torch.zeros(nints, dtype=torch.int32, device=device))
        _PERSISTENT_WS[idx] = ws
    return ws


_DEC_WS: dict[int, tuple] = {}


def decode_gemm_workspace(device):
    """(fp32 partial-tile workspace, zeroed int32 state words) of the decode-step GEMM; one pair per
    device, used from one stream at a time. The state words carry the all-reduce generation, so they
    live as long as the receive buffers they are used with."""
    idx = torch.device(device).index or 0
    ws = _DEC_WS.get(idx)
    if ws is None:
        nbytes, nints, _ = _lib().gemm_dec_sizes()
        ws = (torch.empty(nbytes // 4, dtype=torch.float32, device=device),
              torch.zeros(nints, dtype=torch.int32, device=device))
        _DEC_WS[idx] = ws
    return ws


DECODE_GEMM_MAX_TOKENS = 256      # the decode-step GEMM takes at most this many token rows


def linear_decode(x, w, mode="plain", out=None, h=None, gamma=None, eps=1e-5, weight_offset=0.0,
                  multiply_before_cast=False, xn=None, tp=None, w_scale=None, w_format=None, w_block_scale=None,
                  w_global_scale=None):
    """Decode-step GEMM (at most 256 token rows) with its fused tail.

    mode ``plain``: ``x @ w.T``; ``swiglu``: ``silu(x @ wg.T) * (x @ wu.T)`` with ``w = [wg; wu]``;
    ``add_norm``: ``h += x @ w.T`` summed over the tensor-parallel ranks of ``tp`` (a dict with world, rank,
    lam (peer addresses of the receive buffers), lam_rows, state) or this GPU alone, in place, and returns
    ``(rms_norm(h) * gamma, h)``. ``w_scale``: ``w`` is block-scaled fp8 (e4m3 [N, K], fp32 scales
    [N / 128, K / 128]); the kernel converts weight tiles to scaled bf16 in shared memory and the activations stay
    bf16. ``w_format``: ``"nvfp4"`` (``w`` [N, K / 2] bytes of e2m1 pairs, ``w_block_scale`` [N, K / 16] e4m3,
    ``w_global_scale`` fp32 scalar tensor) or ``"mxfp8"`` (``w`` [N, K] e4m3, ``w_block_scale`` [N, K / 32] ue8m0
    bytes): weight-only quantisation, dequantised tile by tile in shared memory. CPU tensors take the PyTorch
    reference."""
    code = {"plain": 0, "swiglu": 1, "add_norm": 2}[mode]
    fmt = {None: 0, "nvfp4": 2, "mxfp8": 3}[w_format]
    if not x.is_cuda:
        if w_scale is not None:
            w = ref.dequant_fp8_weight_block128(w, w_scale).to(x.dtype)
        elif fmt == 2:
            w = ref.dequant_nvfp4_weight(w, w_block_scale, w_global_scale).to(x.dtype)
        elif fmt == 3:
            w = ref.dequant_mxfp8_weight(w, w_block_scale).to(x.dtype)
        if code == 0:
            return ref.linear(x, w)
        if code == 1:
            return ref.linear_swiglu(x, w)
        y, hh = ref.add_rms_norm(ref.linear(x, w), h, gamma, eps, weight_offset, multiply_before_cast)
        h.copy_(hh)
        return y, h
    ws, state = decode_gemm_workspace(x.device)
    if code == 2:
        if xn is None:
            xn = torch.empty_like(h)
        t = tp or {}
        _lib().gemm_dec(x, w, 2, None, h, xn, gamma, eps, weight_offset, multiply_before_cast,
                        t.get("world", 1), t.get("rank", 0), t.get("lam", []), t.get("lam_rows", 0), ws,
                        t.get("state", state), w_scale, fmt, w_block_scale, w_global_scale)
        return xn, h
    if out is None:
        n = w.shape[0] // 2 if code == 1 else w.shape[0]
        out = torch.empty(x.shape[0], n, dtype=x.dtype, device=x.device)
    _lib().gemm_dec(x, w, code, out, None, None, None, 0.0, 0.0, False, 1, 0, [], 0, ws, state, w_scale, fmt,
                    w_block_scale, w_global_scale)
    return out


HEADS_ON_DECODE_GEMM = False


def batched_linear_heads(x, w, out, x_off, y_off):
    """``out[m, b * y_off + n] = sum_k x[m, b * x_off + k] * w[b, n, k]``: per-head products that address the heads
    as column blocks of ``x`` and ``out`` (no transposes). Runs on the tiled GEMM with the head as a grid dimension;
    ``HEADS_ON_DECODE_GEMM`` moves steps of at most 256 rows (N % 128 == 0) to one persistent launch of the
    decode-step GEMM instead (measured slower on B200 inside a CUDA graph: 14.8 vs 10.4 us for 128 heads of
    [32, 128] x [128, 512], 9.8 vs 4.6 us for [32, 512] x [512, 128])."""
    if not x.is_cuda:
        B, N, K = w.shape
        for b in range(B):
            out[:, b * y_off: b * y_off + N] = ref.linear(x[:, b * x_off: b * x_off + K], w[b])
        return out
    if HEADS_ON_DECODE_GEMM and x.shape[0] <= DECODE_GEMM_MAX_TOKENS and w.shape[1] % 128 == 0 and w.shape[2] % 64 == 0:
        ws, state = decode_gemm_workspace(x.device)
        _lib().gemm_dec_batched(x, w, out, x_off, y_off, ws, state)
    else:
        _lib().batched_gemm_bf16(x, w, out, x_off, y_off)
    return out


def linear(x, w, residual=None, out=None, out_dtype=None, bn=0, splits=0, stages=0, impl=None,
           mode=-1, pdl=False):
    """``x @ w.T`` (+ residual). x: [M, K] bf16, w: [N, K] bf16."""
    if not x.is_cuda:
        y = ref.linear(x, w, residual, out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty(x.shape[0], w.shape[0], dtype=out_dtype or x.dtype, device=x.device)
    sel = impl or GEMM_IMPL
    if sel == "auto" and x.shape[0] >= PAIR_MIN_TOKENS and out.dtype == torch.bfloat16 and bn == 0 and splits == 0:
        sel = "pair"        # same choice as the step executor: CTA pairs from 512 tokens up
    if sel == "persistent":
        ws, counters = persistent_gemm_workspace(x.device)
        _lib().gemm_bf16_persistent(x, w, out, residual, False, ws, counters, bn, stages, mode, pdl)
    elif sel == "pair":
        _lib().gemm_bf16(x, w, out, residual, False, gemm_workspace(x.device), bn, splits, stages, False, True)
    else:
        _lib().gemm_bf16(x, w, out, residual, False, gemm_workspace(x.device), bn, splits, stages)
    return out


def linear_swiglu(x, w_gate_up, out=None, bn=0, stages=0, impl=None, mode=-1, pdl=False):
    """``silu(x @ w_gate.T) * (x @ w_up.T)`` with ``w_gate_up = [w_gate; w_up]`` stacked on rows."""
    if not x.is_cuda:
        y = ref.linear_swiglu(x, w_gate_up)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty(x.shape[0], w_gate_up.shape[0] // 2, dtype=x.dtype, device=x.device)
    sel = impl or GEMM_IMPL
    if sel == "auto" and x.shape[0] >= PAIR_MIN_TOKENS and bn == 0 and w_gate_up.shape[0] >= 2 * 128 * 40:
        sel = "pair"        # token-major persistent pairs once there are more tiles than pairs of SMs
    if sel == "pair":
        _lib().gemm_bf16(x, w_gate_up, out, None, True, None, bn, 1, stages, False, True)
    elif sel in ("persistent", "auto"):
        ws, counters = persistent_gemm_workspace(x.device)
        _lib().gemm_bf16_persistent(x, w_gate_up, out, None, True, ws, counters, bn, stages, mode, pdl)
    else:
        _lib().gemm_bf16(x, w_gate_up, out, None, True, None, bn, 1, stages)
    return out


def rms_norm(x, w, eps, weight_offset=0.0, multiply_before_cast=False, out=None):
    if not x.is_cuda or x.dtype != torch.bfloat16:
        y = ref.rms_norm(x, w, eps, weight_offset, multiply_before_cast)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty_like(x)
    _lib().rmsnorm(x, w, out, eps, weight_offset, multiply_before_cast)
    return out


def qk_norm(qkv, q_w, k_w, n_q: int, n_kv: int, head_dim: int, eps: float):
    """RMSNorm over ``head_dim`` of every query and key head of a fused [T, (n_q + 2 n_kv) * head_dim] projection,
    in place (value heads untouched): normalise in fp32, round to the activation dtype, multiply by the weight."""
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16:
        T = qkv.shape[0]
        for w, lo, n in ((q_w, 0, n_q), (k_w, n_q * head_dim, n_kv)):
            part = qkv[:, lo: lo + n * head_dim].reshape(T * n, head_dim)
            qkv[:, lo: lo + n * head_dim] = ref.rms_norm(part, w, eps).reshape(T, n * head_dim)
        return qkv
    _lib().qk_norm(qkv, q_w, k_w, n_q, n_kv, head_dim, float(eps))
    return qkv


def add_rms_norm(x, residual, w, eps, weight_offset=0.0, multiply_before_cast=False, out=None):
    """residual <- x + residual (in place); returns (rms_norm(residual), residual)."""
    if not x.is_cuda or x.dtype != torch.bfloat16:
        y, h = ref.add_rms_norm(x, residual, w, eps, weight_offset, multiply_before_cast)
        residual.copy_(h)
        return y, residual
    if out is None:
        out = torch.empty_like(x)
    _lib().add_rmsnorm(x, residual, w, out, eps, weight_offset, multiply_before_cast)
    return out, residual


def silu_mul(gate_up, out=None):
    if not gate_up.is_cuda or gate_up.dtype != torch.bfloat16:
        return ref.silu_mul(gate_up)
    if out is None:
        out = torch.empty(gate_up.shape[0], gate_up.shape[1] // 2, dtype=gate_up.dtype,
                          device=gate_up.device)
    _lib().silu_mul(gate_up, out)
    return out


def embedding(ids, table, vocab_start=0, out=None):
    if not table.is_cuda or table.dtype != torch.bfloat16:
        return ref.embedding(ids, table, vocab_start)
    if out is None:
        out = torch.empty(ids.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    _lib().embedding(ids, table, out, vocab_start)
    return out


def rope_kv_store(qkv, positions, slots, cos_sin, k_cache, v_cache, n_q, n_kv, head_dim,
                  interleaved=False):
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16:
        return ref.rope_kv_store(qkv, positions, slots, cos_sin, k_cache, v_cache, n_q, n_kv,
                                 head_dim, interleaved)
    _lib().rope_kv_store(qkv, positions, slots, cos_sin, k_cache, v_cache, n_q, n_kv, head_dim,
                         interleaved)


def build_attention_plan(q_lens, n_q: int, n_kv: int):
    """Host-side split of a ragged batch into decode CTAs and prefill tiles.

    Returns (tile_seq, tile_q0, decode_seq) as int32 numpy arrays. A sequence whose new
    tokens times the GQA group size fit one 16-row MMA tile takes the decode kernel.
    """
    G = n_q // n_kv
    tok_per_tile = max(1, 64 // G)
    tile_seq, tile_q0, decode_seq = [], [], []
    for s, ql in enumerate(q_lens):
        ql = int(ql)
        if ql <= 0:
            continue
        if ql * G <= 16:
            decode_seq.append(s)
        else:
            for t0 in range(0, ql, tok_per_tile):
                tile_seq.append(s)
                tile_q0.append(t0)
    return (np.asarray(tile_seq, dtype=np.int32), np.asarray(tile_q0, dtype=np.int32),
            np.asarray(decode_seq, dtype=np.int32))


_ATTN_SPLIT_WS: dict[int, tuple] = {}


def ensure_attention_split_workspace(device) -> None:
    """Registers the workspace of the split-KV decode attention for this process (one GPU per process):
    partial states plus one zeroed counter per (KV head, decode sequence) of up to 1024 sequences x 64 heads.
    ``MB200_ATTN_SPLIT``: 0 keeps decode steps on the one-CTA-per-sequence kernel, 1 (default) splits when
    there are few (sequence, KV head) pairs, 2 always splits."""
    idx = torch.device(device).index or 0
    if idx in _ATTN_SPLIT_WS:
        return
    L = _lib()
    ws = torch.empty(L.attn_split_workspace_bytes() // 4, dtype=torch.float32, device=device)
    counters = torch.zeros(1024 * 64, dtype=torch.int32, device=device)
    _ATTN_SPLIT_WS[idx] = (ws, counters)
    L.set_attn_split_workspace(ws, counters)
    L.set_attn_split(int(os.environ.get("MB200_ATTN_SPLIT", "1")))


def paged_attention(q, k_cache, v_cache, block_table, q_start, q_len, kv_len, n_q, n_kv,
                    head_dim, scale, plan=None, out=None, kv=None, layer=0):
    """Ragged causal attention. q: [T, ld] with the n_q*head_dim query columns first.

    ``k_cache`` / ``v_cache`` are one layer's views ``[pages, n_kv, page, head_dim]``. When the
    whole cache tensor ``kv`` (6-D) and ``layer`` are given and the page size is a multiple of
    64, the TMA-fed single-launch kernel runs; otherwise the cp.async kernels.
    """
    if not q.is_cuda or q.dtype != torch.bfloat16:
        return ref.paged_attention(q, k_cache, v_cache, block_table, q_start, q_len, kv_len,
                                   n_q, n_kv, head_dim, scale)
    if plan is None:
        ts, t0, ds = build_attention_plan(q_len.cpu().numpy(), n_q, n_kv)
        plan = tuple(torch.from_numpy(a).to(q.device) if a.size else None for a in (ts, t0, ds))
    if out is None:
        out = torch.empty(q.shape[0], n_q * head_dim, dtype=q.dtype, device=q.device)
    if kv is not None and kv.shape[4] % 64 == 0 and os.environ.get("MB200_ATTN_TMA", "1") == "1":
        ensure_attention_split_workspace(q.device)
        _lib().paged_attention_tma(q, out, kv, layer, block_table, q_start, q_len, kv_len,
                                   plan[0], plan[1], plan[2], n_q, n_kv, head_dim, scale)
    else:
        _lib().paged_attention(q, out, k_cache, v_cache, block_table, q_start, q_len, kv_len,
                               plan[0], plan[1], plan[2], n_q, n_kv, head_dim, scale)
    return out


def argmax(logits, out=None):
    if not logits.is_cuda:
        return ref.argmax(logits)
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.long, device=logits.device)
    _lib().argmax(logits.float() if logits.dtype != torch.float32 else logits, out)
    return out


def sample(logits, temperature=None, top_k=None, top_p=None, min_p=None, seeds=None, step=0,
           out=None, generator=None):
    if not logits.is_cuda:
        return ref.sample(logits, temperature, top_k, top_p, min_p, generator)
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.long, device=logits.device)
    _lib().sample(logits, out, temperature, top_k, top_p, min_p, seeds, int(step))
    return out


def set_gemm_pair_persistent(on: bool) -> None:
    """Whether the CTA-pair GEMM runs as persistent pairs with two accumulator stages when a problem has more
    tiles than pairs of SMs (default on); off launches one pair per tile."""
    _lib().set_gemm_pair_persistent(bool(on))


def set_gemm_pair_token_major(mask: int) -> None:
    """Which CTA-pair GEMMs with more tiles than SM pairs run the token-major persistent kernel (tokens on the MMA's
    M side, gate and up rows of a fused SwiGLU GEMM in one 256-wide MMA): bit 0 fused SwiGLU, bit 1 plain."""
    _lib().set_gemm_pair_token_major(int(mask))


def set_sample_cluster(on: bool) -> None:
    """Whether rows with a top-k / top-p / min-p filter are first sampled by the kernel that spreads a row
    over a cluster of eight CTAs (default on); off leaves every row to the one-CTA-per-row kernel."""
    _lib().set_sample_cluster(bool(on))


def apply_penalties(logits, tok, cnt, offsets, freq=None, pres=None, rep=None):
    if not logits.is_cuda:
        return ref.apply_penalties(logits, tok, cnt, offsets, freq, pres, rep)
    _lib().apply_penalties(logits, tok, cnt, offsets, freq, pres, rep)
    return logits


# ------------------------------------------------------------------ block-scaled fp8
def quant_fp8_group128(x):
    """Dynamic per-token-group (1 x 128) fp8 quantisation of activations.
    Returns (q [M, K] float8_e4m3fn, scales fp32 [ceil(K/128), M])."""
    if not x.is_cuda:
        return ref.quant_fp8_group128(x)
    M, K = x.shape
    q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((K + 127) // 128, M, dtype=torch.float32, device=x.device)
    _lib().quant_fp8_group128(x, q, s, True)
    return q, s


def linear_fp8_blockscaled(xq, xs, wq, ws, residual=None, out=None, bn=0, stages=0, splits=0):
    """``(xq * xs) @ (wq * ws).T`` with 128x128 weight-block scales and 1x128 activation scales.
    ``splits``: K splits (0 = chosen by the kernel from the tile count and the SM count)."""
    if not xq.is_cuda:
        return ref.linear_fp8_blockscaled(xq, xs, wq, ws, residual)
    if out is None:
        out = torch.empty(xq.shape[0], wq.shape[0], dtype=torch.bfloat16, device=xq.device)
    _lib().gemm_fp8_blockscaled(xq, xs, wq, ws, out, residual, bn, stages, splits, gemm_workspace(xq.device))
    return out


def linear_fp8(x, wq, ws, residual=None, out=None):
    """bf16 activations in: quantise per token group, then the block-scaled fp8 GEMM."""
    xq, xs = quant_fp8_group128(x)
    return linear_fp8_blockscaled(xq, xs, wq, ws, residual, out)


# ---------------------------------------------------------------------- multi-head latent attention
def batched_linear(x, w, out=None):
    """Per-batch ``x[b] @ w[b].T``. x: [B, M, K], w: [B, N, K] -> [B, M, N].

    On CUDA this is the grouped tcgen05 GEMM with one group per batch entry (used for the MLA
    weight absorption, where the batch is the attention head).
    """
    if not x.is_cuda or x.dtype != torch.bfloat16:
        return ref.batched_linear(x, w)
    B, M, K = x.shape
    N = w.shape[1]
    x = x.contiguous()
    if out is None:
        out = torch.empty(B, M, N, dtype=x.dtype, device=x.device)
    key = (x.device.index or 0, B, M)
    offs = _BATCH_OFFSETS.get(key)
    if offs is None:
        offs = (torch.arange(B + 1, dtype=torch.int32) * M).to(x.device)
        _BATCH_OFFSETS[key] = offs
    _lib().grouped_gemm_bf16(x.view(B * M, K), w.contiguous(), out.view(B * M, N), offs, M, False, 0)
    return out


_BATCH_OFFSETS: dict = {}


def mla_kv_store(c_kv, k_rope, slots, cache):
    """cache[slot] = [c_kv | k_rope] for every token with slot >= 0 (one latent row per token)."""
    if c_kv.is_cuda and c_kv.dtype == torch.bfloat16 and hasattr(_lib(), "mla_kv_store"):
        _lib().mla_kv_store(c_kv, k_rope, slots, cache)
        return
    ref.mla_kv_store(c_kv, k_rope, slots, cache)


_MLA_SPLIT_WS: dict = {}


def ensure_mla_split_workspace(device) -> None:
    """Registers the workspace of the KV-split MLA decode path for this process (one GPU per process): partial
    outputs of up to one part per SM and one zeroed counter per (sequence, 128-head block, output half).
    ``MB200_MLA_SPLIT=0`` keeps one CTA pair per sequence."""
    idx = torch.device(device).index or 0
    if idx in _MLA_SPLIT_WS:
        return
    L = _lib()
    ws = torch.empty(L.mla_split_workspace_bytes() // 4, dtype=torch.float32, device=device)
    counters = torch.zeros(4096, dtype=torch.int32, device=device)
    _MLA_SPLIT_WS[idx] = (ws, counters)
    L.set_mla_split_workspace(ws, counters)
    L.set_mla_split(int(os.environ.get("MB200_MLA_SPLIT", "1")))


def mla_paged_attention(q_lat, q_rope, cache, block_table, q_start, q_len, kv_len, scale, plan=None,
                        decode_only=None):
    """Absorbed-form multi-head latent attention over a paged latent cache; returns [T, h, R].

    ``decode_only``: every sequence has exactly one query token (then 512-wide latents with a multiple of 128
    heads run on the tcgen05 kernel). ``None`` infers it from ``T == number of sequences``: schedulers never
    put a sequence without query tokens into a batch."""
    if q_lat.is_cuda and q_lat.dtype == torch.bfloat16 and hasattr(_lib(), "mla_paged_attention"):
        ensure_mla_split_workspace(q_lat.device)
        out = torch.empty_like(q_lat)
        if decode_only is None:
            decode_only = q_lat.shape[0] == block_table.shape[0]
        _lib().mla_paged_attention(q_lat, q_rope, cache, block_table, q_start, q_len, kv_len, out, scale,
                                   bool(decode_only))
        return out
    return ref.mla_paged_attention(q_lat, q_rope, cache, block_table, q_start, q_len, kv_len, scale)


def apply_token_bitmask(logits, bitmask):
    """In place: mask out tokens whose bit is clear in ``bitmask`` (int32 [rows, ceil(vocab/32)])."""
    if logits.is_cuda:
        _lib().apply_token_bitmask(logits, bitmask.to(logits.device, non_blocking=True).contiguous())
    else:
        from ..pipelines.structured_output import apply_token_bitmask_reference
        apply_token_bitmask_reference(logits, bitmask)
    return logits
