"""Rotary position embedding tables.

``cos_sin_table`` returns the fp32 table ``[max_pos, head_dim]`` the RoPE kernels index by
position: the first ``head_dim/2`` columns are cos, the rest sin. Inverse frequencies are
computed in float64 like the reference (max/python/max/nn/rotary_embedding.py:82-125) and
support its scaling families: Llama-3 (:404-441), linear, dynamic-NTK, YaRN / DeepSeek-YaRN
(:582, :907) and LongRoPE (:738).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch


@dataclass
class RopeScaling:
    rope_type: str = "default"       # default | llama3 | linear | dynamic | yarn | deepseek_yarn | longrope
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    short_factor: Optional[Sequence[float]] = None
    long_factor: Optional[Sequence[float]] = None

    @classmethod
    def from_hf(cls, d: Optional[dict]) -> "RopeScaling":
        if not d:
            return cls()
        t = d.get("rope_type", d.get("type", "default"))
        keys = {f for f in cls.__dataclass_fields__}
        kw = {k: v for k, v in d.items() if k in keys}
        kw["rope_type"] = t
        return cls(**kw)


def _yarn_find_dim(n_rot: float, dim: int, base: float, max_pos: int) -> float:
    return (dim * math.log(max_pos / (n_rot * 2 * math.pi))) / (2 * math.log(base))


def _yarn_mscale(scale: float, m: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0


def inverse_frequencies(head_dim: int, theta: float, scaling: RopeScaling,
                        seq_len: Optional[int] = None) -> tuple[np.ndarray, float]:
    """Returns (inv_freq[float64, head_dim/2], attention scale multiplier)."""
    idx = np.arange(0, head_dim, 2, dtype=np.float64)
    inv = 1.0 / (theta ** (idx / head_dim))
    att = 1.0
    t = scaling.rope_type
    if t in ("default", None):
        pass
    elif t == "linear":
        inv = inv / scaling.factor
    elif t == "llama3":
        low_wl = scaling.original_max_position_embeddings / scaling.low_freq_factor
        high_wl = scaling.original_max_position_embeddings / scaling.high_freq_factor
        wl = 2 * math.pi / inv
        smooth = (scaling.original_max_position_embeddings / wl - scaling.low_freq_factor) / (
            scaling.high_freq_factor - scaling.low_freq_factor)
        mid = (1 - smooth) * inv / scaling.factor + smooth * inv
        inv = np.where(wl < high_wl, inv, np.where(wl > low_wl, inv / scaling.factor, mid))
    elif t == "dynamic":
        orig = scaling.original_max_position_embeddings
        if seq_len and seq_len > orig:
            base = theta * ((scaling.factor * seq_len / orig) - (scaling.factor - 1)) ** (
                head_dim / (head_dim - 2))
            inv = 1.0 / (base ** (idx / head_dim))
    elif t in ("yarn", "deepseek_yarn"):
        orig = scaling.original_max_position_embeddings
        lo = max(math.floor(_yarn_find_dim(scaling.beta_fast, head_dim, theta, orig)), 0)
        hi = min(math.ceil(_yarn_find_dim(scaling.beta_slow, head_dim, theta, orig)), head_dim - 1)
        ramp = np.clip((np.arange(head_dim // 2, dtype=np.float64) - lo) / max(hi - lo, 1e-3), 0, 1)
        mask = 1.0 - ramp
        inv = (inv / scaling.factor) * (1 - mask) + inv * mask
        if t == "deepseek_yarn":
            att = _yarn_mscale(scaling.factor, scaling.mscale) / _yarn_mscale(
                scaling.factor, scaling.mscale_all_dim)
        else:
            att = _yarn_mscale(scaling.factor, 1.0)
    elif t == "longrope":
        orig = scaling.original_max_position_embeddings
        use_long = bool(seq_len and seq_len > orig)
        f = scaling.long_factor if use_long else scaling.short_factor
        if f is not None:
            inv = inv / np.asarray(f, dtype=np.float64)
        if scaling.factor > 1:
            att = math.sqrt(1 + math.log(scaling.factor) / math.log(orig))
    else:
        raise ValueError(f"unknown rope scaling type {t!r}")
    return inv, att


def cos_sin_table(head_dim: int, max_pos: int, theta: float = 10000.0,
                  scaling: Optional[RopeScaling] = None, device="cpu") -> torch.Tensor:
    scaling = scaling or RopeScaling()
    inv, att = inverse_frequencies(head_dim, theta, scaling, max_pos)
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * inv[None, :]
    tab = np.concatenate([np.cos(ang) * att, np.sin(ang) * att], axis=1).astype(np.float32)
    return torch.from_numpy(tab).to(device)
