"""Checkpoint IO: HF-layout safetensors directories, config.json, quantisation config.

Reference: max/python/max/graph/weights/load_safetensors.py:34 (lazy multi-file reader),
max/python/max/pipelines/weights/hf_utils.py:390 (repo layout + encoding detection),
max/python/max/pipelines/weights/quant.py:1135 ``parse_quant_config`` (:581 block-scaled fp8).
Loading is zero-copy from the memory-mapped files; large tensors are staged to pinned memory
by the native thread pool and uploaded asynchronously.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Iterator, Optional

import torch


@dataclass
class QuantConfig:
    """Weight/activation quantisation of a checkpoint."""

    format: str = "none"                 # none | blockscaled_fp8 | tensor_fp8 | compressed_tensors_fp8 | nvfp4 | mxfp8
    weight_block_size: tuple = (128, 128)
    activation_scheme: str = "dynamic"   # dynamic per-token-group (1 x 128) | static
    activation_group: int = 128
    weight_dtype: str = "float8_e4m3fn"
    scale_suffix: str = "weight_scale_inv"
    ignored_layers: tuple = ()

    @property
    def is_blockscaled_fp8(self) -> bool:
        return self.format == "blockscaled_fp8"


def parse_quant_config(hf_config: dict) -> Optional[QuantConfig]:
    q = hf_config.get("quantization_config")
    if not q:
        return None
    method = q.get("quant_method", "")
    if method == "fp8":
        wbs = q.get("weight_block_size")
        if wbs:
            if list(wbs) != [128, 128]:
                raise ValueError(f"unsupported fp8 weight_block_size {wbs}; kernels are built for [128, 128]")
            return QuantConfig("blockscaled_fp8", (128, 128), q.get("activation_scheme", "dynamic"), 128,
                               "float8_e4m3fn", "weight_scale_inv",
                               tuple(q.get("modules_to_not_convert") or ()))
        return QuantConfig("tensor_fp8", (0, 0), q.get("activation_scheme", "dynamic"), 0,
                           "float8_e4m3fn", "weight_scale", tuple(q.get("modules_to_not_convert") or ()))
    if method == "compressed-tensors":
        groups = q.get("config_groups", {})
        for g in groups.values():
            w = g.get("weights", {})
            if w.get("type") == "float" and w.get("num_bits") == 8:
                strategy = w.get("strategy", "tensor")
                fmt = "blockscaled_fp8" if strategy == "block" else "compressed_tensors_fp8"
                return QuantConfig(fmt, tuple(w.get("block_structure") or (128, 128)),
                                   "dynamic" if g.get("input_activations", {}).get("dynamic", True) else "static",
                                   128, "float8_e4m3fn", "weight_scale", tuple(q.get("ignore") or ()))
        raise ValueError("compressed-tensors checkpoint without an 8-bit float weight group")
    if method in ("modelopt", "nvfp4"):
        # NVIDIA Model Optimizer checkpoints: NVFP4 = 4-bit e2m1 weights, e4m3 scale per 16 values, fp32 scale per
        # tensor (reference: nn/quant_config.py float4 config, weight adapters of the nvfp4 checkpoints)
        algo = str(q.get("quant_algo") or q.get("quantization", {}).get("quant_algo") or "NVFP4").upper()
        if algo == "NVFP4":
            return QuantConfig("nvfp4", (1, 16), "dynamic", 16, "uint8", "weight_scale",
                               tuple(q.get("exclude_modules") or q.get("ignore") or ()))
        if algo in ("MXFP8", "FP8_MX"):
            return QuantConfig("mxfp8", (1, 32), "dynamic", 32, "float8_e4m3fn", "weight_scale",
                               tuple(q.get("exclude_modules") or q.get("ignore") or ()))
        raise ValueError(f"unsupported modelopt quant_algo {algo!r}")
    if method == "mxfp8":
        return QuantConfig("mxfp8", (1, 32), "dynamic", 32, "float8_e4m3fn", "weight_scale",
                           tuple(q.get("modules_to_not_convert") or ()))
    raise ValueError(f"unsupported quantisation method {method!r}")


def normalize_hf_rope(d: dict) -> dict:
    """``config.json`` written by transformers >= 5 carries the rotary settings as ``rope_parameters``
    (``{"rope_type": ..., "rope_theta": ..., <scaling keys>}``) instead of ``rope_theta`` + ``rope_scaling``: returns
    a copy with the older pair filled in (``rope_scaling`` None for the default type)."""
    rp = d.get("rope_parameters")
    if not isinstance(rp, dict):
        return d
    d = dict(d)
    if "rope_theta" in rp and d.get("rope_theta") is None:
        d["rope_theta"] = rp["rope_theta"]
    if d.get("rope_scaling") is None:
        kind = rp.get("rope_type", rp.get("type", "default"))
        d["rope_scaling"] = None if kind in (None, "default") else {k: v for k, v in rp.items() if k != "rope_theta"}
    return d


def load_hf_config(model_path: str) -> dict:
    g = _gguf_file(model_path)
    if g is not None and not (os.path.isdir(model_path) and (Path(model_path) / "config.json").exists()):
        from .gguf import GGUFReader
        return GGUFReader(g).hf_config()
    return _load_hf_config_json(model_path)


def _load_hf_config_json(model_path: str) -> dict:
    p = Path(model_path) / "config.json"
    if not p.exists():
        raise FileNotFoundError(f"{p} not found: model_path must be a local HF-layout directory "
                                "(there is no hub download here)")
    return json.loads(p.read_text())


def find_weight_files(model_path: str, weight_path=()) -> list[Path]:
    if weight_path:
        return [Path(w) if os.path.isabs(str(w)) else Path(model_path) / w for w in weight_path]
    root = Path(model_path)
    idx = root / "model.safetensors.index.json"
    if idx.exists():
        files = sorted(set(json.loads(idx.read_text())["weight_map"].values()))
        return [root / f for f in files]
    files = sorted(root.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no *.safetensors under {root}")
    return files


class SafetensorWeights:
    """Lazy name -> tensor view over one or more safetensors files."""

    def __init__(self, files):
        from safetensors import safe_open

        self._handles = [safe_open(str(f), framework="pt", device="cpu") for f in files]
        self._where = {}
        for h in self._handles:
            for k in h.keys():
                self._where[k] = h

    def keys(self):
        return self._where.keys()

    def __contains__(self, k):
        return k in self._where

    def __getitem__(self, k) -> torch.Tensor:
        return self._where[k].get_tensor(k)

    def items(self) -> Iterator:
        for k in self._where:
            yield k, self[k]

    def to_dict(self) -> dict:
        return {k: self[k] for k in self._where}


class GGUFWeights:
    """A ``.gguf`` file presented like :class:`SafetensorWeights` (HF names, tensors dequantised on access)."""

    def __init__(self, path: str, dtype: torch.dtype = torch.bfloat16):
        from .gguf import GGUFReader, hf_name

        self.reader, self.dtype = GGUFReader(path), dtype
        self._names = {hf_name(n): n for n in self.reader.tensors if hf_name(n)}

    def keys(self):
        return self._names.keys()

    def __contains__(self, k):
        return k in self._names

    def to_dict(self) -> dict:
        return self.reader.to_hf_state_dict(self.dtype)

    def __getitem__(self, k) -> torch.Tensor:
        return self.to_dict()[k] if ("q_proj" in k or "k_proj" in k) else self.reader.get(self._names[k], self.dtype)


def _gguf_file(model_path: str, weight_path=()) -> Optional[str]:
    cands = [str(w) for w in weight_path if str(w).endswith(".gguf")]
    if model_path.endswith(".gguf"):
        cands.append(model_path)
    elif os.path.isdir(model_path) and not any(Path(model_path).glob("*.safetensors")):
        cands += sorted(str(p) for p in Path(model_path).glob("*.gguf"))
    return cands[0] if cands else None


def load_state_dict(model_path: str, weight_path=()):
    """Safetensors directory (HF layout) or a GGUF file."""
    g = _gguf_file(model_path, weight_path)
    if g is not None:
        return GGUFWeights(g)
    return SafetensorWeights(find_weight_files(model_path, weight_path))


def save_checkpoint(out_dir: str, hf_config: dict, state_dict: dict, max_shard_bytes: int = 4 << 30) -> None:
    """Write an HF-layout directory (config.json + sharded safetensors + index)."""
    from safetensors.torch import save_file

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(hf_config, indent=1))
    shards, cur, cur_bytes = [], {}, 0
    for k, v in state_dict.items():
        nb = v.numel() * v.element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = v.detach().cpu().contiguous()
        cur_bytes += nb
    if cur:
        shards.append(cur)
    weight_map = {}
    for i, sh in enumerate(shards):
        name = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, str(out / name), metadata={"format": "pt"})
        weight_map.update({k: name for k in sh})
    if len(shards) > 1:
        (out / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))


def upload_async(t: torch.Tensor, device, dtype=None, pool=None) -> torch.Tensor:
    """Host tensor -> device through pinned staging (copy runs on the native pool when given)."""
    dev = torch.device(device)
    if dev.type != "cuda":
        return t.to(dtype=dtype or t.dtype)
    src = t if dtype is None or t.dtype == dtype else t.to(dtype)
    src = src.contiguous()
    pinned = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
    if pool is not None and src.numel() * src.element_size() > (8 << 20):
        pool.parallel_memcpy(pinned.data_ptr(), src.data_ptr(), src.numel() * src.element_size())
    else:
        pinned.copy_(src)
    return pinned.to(dev, non_blocking=True)
