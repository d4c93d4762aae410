"""Loader for the in-tree native library (``modular_b200/_C.so``).

``lib()`` returns the extension module. On a machine with a CUDA device a missing or
unloadable library is an error (ops must never fall back silently to eager PyTorch on a
GPU); on a CPU-only machine ``lib(required=False)`` returns ``None`` and callers use the
PyTorch reference implementations.
"""

from __future__ import annotations

import importlib.util
import os
import threading
from pathlib import Path

_LOCK = threading.Lock()
_MOD = None
_TRIED = False
_ERR: Exception | None = None
SO_PATH = Path(__file__).resolve().parent.parent / "_C.so"


def _load():
    global _MOD, _TRIED, _ERR
    with _LOCK:
        if _TRIED:
            return _MOD
        _TRIED = True
        try:
            if not SO_PATH.exists() and os.environ.get("MB200_NO_BUILD") != "1":
                from .build import build

                build()
            import torch  # noqa: F401  (libtorch must be loaded first)

            spec = importlib.util.spec_from_file_location("modular_b200._C", str(SO_PATH))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            # step kernels launch as programmatic dependents unless MB200_PDL=0 (see csrc/common/launch.h)
            if os.environ.get("MB200_PDL", "1") not in ("", "0") and hasattr(mod, "set_pdl"):
                mod.set_pdl(True)
            # prefill attention on the tcgen05 kernel (head_dim 128) for steps with at least MB200_ATTN_TC
            # 64-row tiles (default 32; 0 turns it off, 1 always uses it)
            if hasattr(mod, "set_attn_tc"):
                mod.set_attn_tc(int(os.environ.get("MB200_ATTN_TC", "32") or 0))
            # GEMMs on CTA pairs (cta_group::2): MB200_GEMM_PAIR="<min tokens, plain>,<min tokens, SwiGLU>",
            # 0 = never for that kind. Measured on B200: plain GEMMs from 512 tokens up are 3-10 % faster on
            # pairs (most with a long K), the fused SwiGLU GEMM is not.
            if hasattr(mod, "set_gemm_pair"):
                plain, _, dual = os.environ.get("MB200_GEMM_PAIR", "512,0").partition(",")
                mod.set_gemm_pair(int(plain or 0), int(dual or 0))
            # MB200_GEMM_PAIR_PERSIST=0: one launch-time pair per tile even when there are more tiles than SM pairs
            # MB200_GEMM_PAIR_TM: which pair GEMMs with many tiles run with the tokens on the MMA's M side (bit 0 fused
            # SwiGLU: gate and up rows in one 256-wide MMA, 1.15-1.35x the one-CTA persistent kernel; bit 1 plain)
            if hasattr(mod, "set_gemm_pair_token_major"):
                mod.set_gemm_pair_token_major(int(os.environ.get("MB200_GEMM_PAIR_TM", "3") or 0))
            if hasattr(mod, "set_gemm_pair_persistent"):
                mod.set_gemm_pair_persistent(os.environ.get("MB200_GEMM_PAIR_PERSIST", "1") not in ("", "0"))
            if hasattr(mod, "set_attn_decode_dense"):
                mod.set_attn_decode_dense(os.environ.get("MB200_ATTN_DECODE_DENSE", "0") not in ("", "0"))
            if hasattr(mod, "set_attn_fork"):
                mod.set_attn_fork(os.environ.get("MB200_ATTN_FORK", "1") not in ("", "0"))
            # MB200_DEC_ROPE=1: rotary embedding + KV store inside the decode-step QKV GEMM. Off by default: measured
            # on B200 under a CUDA graph the decode step is 2.5 % slower with it at TP2 (4.08 vs 3.98 ms) and 9 % at
            # TP1 (the rotation's paired reads slow the GEMM's epilogue by more than the small kernel costs)
            if hasattr(mod, "set_gemm_dec_rope"):
                mod.set_gemm_dec_rope(os.environ.get("MB200_DEC_ROPE", "0") not in ("", "0"))
            if hasattr(mod, "set_mla_tc"):
                mod.set_mla_tc(os.environ.get("MB200_MLA_TC", "1") not in ("", "0"))
            _MOD = mod
        except Exception as e:  # noqa: BLE001
            _ERR = e
            _MOD = None
        return _MOD


class _CountingLib:
    """The extension module with every function call counted (``native_calls()``): a lower bound of the kernels
    launched by paths that are driven op by op from Python (some functions launch two or three kernels)."""

    def __init__(self, mod):
        self._mod, self._cache, self.calls = mod, {}, 0

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            target = getattr(self._mod, name)
            if not callable(target):
                return target

            def fn(*a, __t=target, **k):
                self.calls += 1
                return __t(*a, **k)

            self._cache[name] = fn
        return fn


_COUNTING: _CountingLib | None = None


def count_calls(on: bool = True) -> None:
    """Route ``lib()`` through a call counter (off by default: one Python frame per call)."""
    global _COUNTING
    _COUNTING = _CountingLib(_load()) if on and _load() is not None else None


def native_calls() -> int:
    return _COUNTING.calls if _COUNTING is not None else 0


def lib(required: bool = True):
    mod = _load()
    if _COUNTING is not None:
        return _COUNTING
    if mod is None and required:
        raise RuntimeError(
            f"modular_b200 native library could not be loaded from {SO_PATH}: {_ERR!r}. "
            "Run `python -m modular_b200._native.build`."
        )
    return mod


def available() -> bool:
    return _load() is not None
