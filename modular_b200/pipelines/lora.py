"""LoRA adapters: loading, a slot manager, and batched multi-adapter application.

A batch may mix requests with different adapters (and none). Per linear module the delta is
    y[t] += scale[a(t)] * (x[t] @ A[a(t)].T) @ B[a(t)].T
computed for all tokens at once: tokens are sorted by adapter slot, the "shrink" (to rank r) and
"expand" (back to the output width) products run as grouped tcgen05 GEMMs with one group per adapter,
and the result is scattered back. On CPU the same maths runs per adapter in PyTorch.

Adapters follow the PEFT checkpoint layout (``...layers.N.self_attn.q_proj.lora_A.weight`` [r, in],
``lora_B.weight`` [out, r], ``adapter_config.json`` with ``r`` and ``lora_alpha``).

Reference: max/python/max/pipelines/lora/lora.py (``LoRAManager``: load / unload / LRU slots, batch
sorting by adapter), max/kernels/src/linalg/lora.mojo (SGMV shrink / expand).
"""

from __future__ import annotations

import re
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from .. import ops

MODULES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
_KEY = re.compile(r"layers\.(\d+)\.(?:self_attn|mlp)\.(\w+)\.lora_([AB])(?:\.default)?\.weight$")


@dataclass
class LoRAAdapter:
    name: str
    rank: int
    scale: float
    # (layer, module) -> (A [r, in], B [out, r])
    weights: dict = field(default_factory=dict)

    @classmethod
    def from_state_dict(cls, name: str, sd: dict, rank: Optional[int] = None, alpha: Optional[float] = None,
                        device="cpu", dtype=torch.bfloat16) -> "LoRAAdapter":
        parts: dict = {}
        for k, v in sd.items():
            m = _KEY.search(k)
            if not m:
                continue
            layer, module, ab = int(m.group(1)), m.group(2), m.group(3)
            if module not in MODULES:
                raise ValueError(f"LoRA target module {module!r} is not supported")
            parts.setdefault((layer, module), {})[ab] = v.to(dtype).to(device).contiguous()
        if not parts:
            raise ValueError("no LoRA tensors found in the state dict")
        weights = {}
        for key, ab in parts.items():
            if set(ab) != {"A", "B"}:
                raise ValueError(f"adapter tensor pair incomplete for {key}")
            weights[key] = (ab["A"], ab["B"])
        r = rank or next(iter(weights.values()))[0].shape[0]
        return cls(name, r, (alpha if alpha is not None else r) / r, weights)


def load_peft_adapter_files(path: str) -> tuple:
    """Reads a PEFT adapter from a directory (``adapter_model.safetensors`` + ``adapter_config.json``) or from
    one ``.safetensors`` file. Returns (state dict, lora_alpha or None)."""
    import json
    import os

    from safetensors.torch import load_file

    alpha = None
    if os.path.isdir(path):
        cfg = os.path.join(path, "adapter_config.json")
        if os.path.exists(cfg):
            with open(cfg) as f:
                alpha = json.load(f).get("lora_alpha")
        path = os.path.join(path, "adapter_model.safetensors")
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    return load_file(path), alpha


class LoRAManager:
    """Keeps up to ``max_loras`` adapters resident in slots (LRU eviction of inactive ones)."""

    def __init__(self, max_loras: int = 8, max_rank: int = 64):
        self.max_loras, self.max_rank = max_loras, max_rank
        self._slots: "OrderedDict[str, int]" = OrderedDict()
        self.adapters: dict[int, LoRAAdapter] = {}
        self._pinned: dict[str, int] = {}
        self._generation: dict[str, int] = {}   # how many times a name has been loaded

    def cache_salt(self, name: Optional[str]) -> int:
        """Prefix-cache salt of requests that run on adapter ``name`` (0 for the base model). Adapters change
        the k/v projections, so KV pages written under one adapter must never be reused under another or under
        the base model; the load count makes a re-loaded adapter of the same name miss as well."""
        if not name:
            return 0
        import hashlib
        d = hashlib.blake2b(f"{name}\0{self._generation.get(name, 0)}".encode(), digest_size=8).digest()
        return (int.from_bytes(d, "little") & 0x7FFFFFFFFFFFFFFF) or 1

    def load(self, adapter: LoRAAdapter) -> int:
        if adapter.rank > self.max_rank or adapter.rank % 8:
            raise ValueError(f"LoRA rank {adapter.rank} must be a multiple of 8 and <= {self.max_rank}")
        if adapter.name in self._slots:
            slot = self._slots[adapter.name]
        elif len(self._slots) < self.max_loras:
            slot = next(i for i in range(self.max_loras) if i not in self.adapters)
        else:
            victim = next((n for n in self._slots if self._pinned.get(n, 0) == 0), None)
            if victim is None:
                raise RuntimeError("all LoRA slots are in use by running requests")
            slot = self._slots.pop(victim)
            del self.adapters[slot]
        self._slots[adapter.name] = slot
        self._slots.move_to_end(adapter.name)
        self.adapters[slot] = adapter
        self._generation[adapter.name] = self._generation.get(adapter.name, 0) + 1
        return slot

    def unload(self, name: str) -> bool:
        if self._pinned.get(name, 0) > 0:
            raise RuntimeError(f"adapter {name!r} is in use")
        slot = self._slots.pop(name, None)
        if slot is None:
            return False
        del self.adapters[slot]
        return True

    def slot_of(self, name: Optional[str]) -> int:
        """Slot of a loaded adapter (-1 for the base model); marks it most recently used."""
        if not name:
            return -1
        if name not in self._slots:
            raise KeyError(f"LoRA adapter {name!r} is not loaded (loaded: {list(self._slots)})")
        self._slots.move_to_end(name)
        return self._slots[name]

    def pin(self, name: str) -> None:
        self._pinned[name] = self._pinned.get(name, 0) + 1

    def unpin(self, name: str) -> None:
        self._pinned[name] = max(0, self._pinned.get(name, 0) - 1)

    def names(self) -> list:
        return list(self._slots)


class LoRABatch:
    """Token -> adapter slot map of one step, with the sort by slot done once for all modules."""

    def __init__(self, manager: LoRAManager, token_slots: torch.Tensor):
        self.manager = manager
        ts = token_slots.to(torch.int64)
        self.active = sorted(int(s) for s in torch.unique(ts).tolist() if s >= 0)
        if self.active:
            key = torch.where(ts >= 0, ts, torch.full_like(ts, 1 << 30))
            self.order = torch.argsort(key, stable=True)
            sorted_slots = ts[self.order]
            self.n_lora = int((sorted_slots >= 0).sum())
            counts = [int((sorted_slots == s).sum()) for s in self.active]
            offs = [0]
            for c in counts:
                offs.append(offs[-1] + c)
            self.offsets = torch.tensor(offs, dtype=torch.int32, device=token_slots.device)
            self.max_rows = max(counts)
            self.rows = self.order[: self.n_lora]

    def delta(self, layer: int, module: str, x: torch.Tensor) -> Optional[torch.Tensor]:
        """[T, out] delta for ``module`` of ``layer`` (zeros for tokens without an adapter), or None."""
        if not self.active:
            return None
        ads = [self.manager.adapters[s] for s in self.active]
        ws = [a.weights.get((layer, module)) for a in ads]
        if all(w is None for w in ws):
            return None
        out_dim = next(w for w in ws if w is not None)[1].shape[0]
        xs = x[self.rows].contiguous()
        ys = torch.zeros(self.n_lora, out_dim, dtype=x.dtype, device=x.device)
        uniform = all(w is not None for w in ws) and len({a.rank for a in ads}) == 1
        if x.is_cuda and x.dtype == torch.bfloat16 and uniform and xs.shape[1] % 8 == 0:
            L = ops._lib()
            r = ads[0].rank
            A = torch.stack([w[0] for w in ws]).contiguous()                                  # [n, r, in]
            B = torch.stack([(w[1].float() * a.scale).to(x.dtype) for w, a in zip(ws, ads)]).contiguous()  # [n, out, r]
            mid = torch.empty(self.n_lora, r, dtype=x.dtype, device=x.device)
            L.grouped_gemm_bf16(xs, A, mid, self.offsets, self.max_rows, False, 0)           # shrink
            L.grouped_gemm_bf16(mid, B, ys, self.offsets, self.max_rows, False, 0)           # expand
        else:
            offs = self.offsets.tolist()
            for i, (w, a) in enumerate(zip(ws, ads)):
                if w is None or offs[i] == offs[i + 1]:
                    continue
                seg = xs[offs[i]:offs[i + 1]].float()
                ys[offs[i]:offs[i + 1]] = ((seg @ w[0].float().t()) @ w[1].float().t() * a.scale).to(x.dtype)
        full = torch.zeros(x.shape[0], out_dim, dtype=x.dtype, device=x.device)
        full[self.rows] = ys
        return full


def token_slots_for(manager: LoRAManager, q_lens: Sequence[int], names: Sequence[Optional[str]], device) -> torch.Tensor:
    slots = []
    for n, name in zip(q_lens, names):
        slots.extend([manager.slot_of(name)] * int(n))
    return torch.tensor(slots, dtype=torch.int32, device=device)
