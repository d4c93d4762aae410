"""GGUF checkpoints: reader, K-quant dequantisation, llama.cpp -> HF tensor names, and a small writer.

Supported tensor types: F32, F16, BF16, Q8_0, Q4_0, Q4_K, Q6_K (the types of the common
``Q4_K_M`` / ``Q6_K`` / ``Q8_0`` releases). Quantised tensors are expanded to the requested float
dtype at load time; the GEMMs then run on the bf16 tcgen05 path.

Reference: max/python/max/graph/weights/load_gguf.py:71 (``GGUFWeights``), the GGUF v3 layout of
llama.cpp (header, typed key/value metadata, tensor infos, aligned data section), and the K-quant
block formats handled by max/kernels/src/quantization/qmatmul_k.mojo.
"""

from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import BinaryIO, Optional

import numpy as np
import torch

GGUF_MAGIC = 0x46554747
(T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64) = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f",
           T_BOOL: "<?", T_U64: "<Q", T_I64: "<q", T_F64: "<d"}

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 2, 8, 12, 14, 30
# type -> (values per block, bytes per block)
BLOCK = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2), GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34),
         GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210)}


@dataclass
class GGUFTensorInfo:
    name: str
    shape: tuple          # row-major (outermost first), i.e. reversed GGUF dims
    ggml_type: int
    offset: int           # from the start of the data section

    @property
    def nbytes(self) -> int:
        per, size = BLOCK[self.ggml_type]
        return int(np.prod(self.shape)) // per * size


def _read(f: BinaryIO, fmt: str):
    return struct.unpack(fmt, f.read(struct.calcsize(fmt)))[0]


def _read_str(f: BinaryIO) -> str:
    return f.read(_read(f, "<Q")).decode("utf-8")


def _read_value(f: BinaryIO, t: int):
    if t in _SCALAR:
        return _read(f, _SCALAR[t])
    if t == T_STR:
        return _read_str(f)
    if t == T_ARR:
        et, n = _read(f, "<I"), _read(f, "<Q")
        if et in _SCALAR and et != T_BOOL:
            return np.frombuffer(f.read(n * struct.calcsize(_SCALAR[et])), dtype=np.dtype(_SCALAR[et])).tolist()
        return [_read_value(f, et) for _ in range(n)]
    raise ValueError(f"unknown GGUF value type {t}")


# ------------------------------------------------------------------------------ dequantisation
def _f16(raw: np.ndarray) -> np.ndarray:
    return raw.view(np.float16).astype(np.float32)


def dequantize(raw: np.ndarray, ggml_type: int, n: int) -> np.ndarray:
    """raw: uint8 array of the tensor's bytes -> float32 array of n values."""
    if ggml_type == GGML_F32:
        return raw.view(np.float32)[:n].copy()
    if ggml_type == GGML_F16:
        return _f16(raw)[:n]
    if ggml_type == GGML_BF16:
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)[:n]
    per, size = BLOCK[ggml_type]
    blocks = raw.reshape(-1, size)
    if ggml_type == GGML_Q8_0:
        d = _f16(blocks[:, :2].copy()).reshape(-1, 1)
        return (blocks[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1)[:n]
    if ggml_type == GGML_Q4_0:
        d = _f16(blocks[:, :2].copy()).reshape(-1, 1)
        qs = blocks[:, 2:]
        lo, hi = (qs & 0x0F).astype(np.int8) - 8, (qs >> 4).astype(np.int8) - 8
        return (np.concatenate([lo, hi], axis=1).astype(np.float32) * d).reshape(-1)[:n]
    if ggml_type == GGML_Q4_K:
        d = _f16(blocks[:, 0:2].copy()).reshape(-1, 1)
        dmin = _f16(blocks[:, 2:4].copy()).reshape(-1, 1)
        sc = blocks[:, 4:16].astype(np.uint8)
        qs = blocks[:, 16:144]
        scales = np.empty((blocks.shape[0], 8), np.float32)
        mins = np.empty((blocks.shape[0], 8), np.float32)
        for j in range(8):                      # 6-bit scale / min per 32-value sub-block
            if j < 4:
                s, m = sc[:, j] & 63, sc[:, j + 4] & 63
            else:
                s = (sc[:, j + 4] & 0x0F) | ((sc[:, j - 4] >> 6) << 4)
                m = (sc[:, j + 4] >> 4) | ((sc[:, j] >> 6) << 4)
            scales[:, j], mins[:, j] = s, m
        out = np.empty((blocks.shape[0], 256), np.float32)
        for g in range(4):                      # 64 values per 32 bytes: low nibbles then high nibbles
            q = qs[:, 32 * g:32 * (g + 1)]
            out[:, 64 * g:64 * g + 32] = d * scales[:, 2 * g:2 * g + 1] * (q & 0x0F) - dmin * mins[:, 2 * g:2 * g + 1]
            out[:, 64 * g + 32:64 * g + 64] = d * scales[:, 2 * g + 1:2 * g + 2] * (q >> 4) - dmin * mins[:, 2 * g + 1:2 * g + 2]
        return out.reshape(-1)[:n]
    if ggml_type == GGML_Q6_K:
        ql, qh = blocks[:, 0:128], blocks[:, 128:192]
        sc = blocks[:, 192:208].view(np.int8).astype(np.float32)
        d = _f16(blocks[:, 208:210].copy()).reshape(-1, 1)
        out = np.empty((blocks.shape[0], 256), np.float32)
        for half in range(2):
            l_, h_ = ql[:, 64 * half:64 * half + 64], qh[:, 32 * half:32 * half + 32]
            base = 128 * half
            q1 = ((l_[:, :32] & 0x0F) | (((h_ >> 0) & 3) << 4)).astype(np.int8) - 32
            q2 = ((l_[:, 32:] & 0x0F) | (((h_ >> 2) & 3) << 4)).astype(np.int8) - 32
            q3 = ((l_[:, :32] >> 4) | (((h_ >> 4) & 3) << 4)).astype(np.int8) - 32
            q4 = ((l_[:, 32:] >> 4) | (((h_ >> 6) & 3) << 4)).astype(np.int8) - 32
            for k, q in enumerate((q1, q2, q3, q4)):
                s = np.repeat(sc[:, 8 * half + 2 * k:8 * half + 2 * k + 2], 16, axis=1)   # one scale per 16 values
                out[:, base + 32 * k:base + 32 * k + 32] = d * s * q
        return out.reshape(-1)[:n]
    raise ValueError(f"GGML tensor type {ggml_type} is not supported")


# ------------------------------------------------------------------------------ reader
class GGUFReader:
    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            if _read(f, "<I") != GGUF_MAGIC:
                raise ValueError(f"{path} is not a GGUF file")
            self.version = _read(f, "<I")
            if self.version not in (2, 3):
                raise ValueError(f"GGUF version {self.version} is not supported")
            n_tensors, n_kv = _read(f, "<Q"), _read(f, "<Q")
            self.metadata = {}
            for _ in range(n_kv):
                key = _read_str(f)
                self.metadata[key] = _read_value(f, _read(f, "<I"))
            self.tensors: dict[str, GGUFTensorInfo] = {}
            for _ in range(n_tensors):
                name = _read_str(f)
                nd = _read(f, "<I")
                dims = [_read(f, "<Q") for _ in range(nd)]
                t, off = _read(f, "<I"), _read(f, "<Q")
                self.tensors[name] = GGUFTensorInfo(name, tuple(reversed(dims)), t, off)
            align = int(self.metadata.get("general.alignment", 32))
            self.data_start = (f.tell() + align - 1) // align * align
        self._mm = np.memmap(path, dtype=np.uint8, mode="r")

    def get(self, name: str, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        info = self.tensors[name]
        raw = np.asarray(self._mm[self.data_start + info.offset:self.data_start + info.offset + info.nbytes])
        n = int(np.prod(info.shape))
        return torch.from_numpy(dequantize(raw, info.ggml_type, n).reshape(info.shape)).to(dtype)

    def hf_config(self) -> dict:
        """The HF-style config fields recoverable from the metadata of a llama, qwen2 or qwen3 file."""
        md, a = self.metadata, self.metadata.get("general.architecture", "llama")
        if a not in _ARCH:
            raise ValueError(f"GGUF architecture {a!r} is not supported (supported: {sorted(_ARCH)})")
        g = lambda k, d=None: md.get(f"{a}.{k}", d)
        heads = g("attention.head_count")
        emb = g("embedding_length")
        cfg = {"architectures": [_ARCH[a][0]], "model_type": a, "hidden_size": emb,
               "num_hidden_layers": g("block_count"), "num_attention_heads": heads,
               "num_key_value_heads": g("attention.head_count_kv", heads),
               "intermediate_size": g("feed_forward_length"), "rms_norm_eps": g("attention.layer_norm_rms_epsilon", 1e-5),
               "rope_theta": g("rope.freq_base", 10000.0), "max_position_embeddings": g("context_length", 2048),
               "head_dim": g("attention.key_length", emb // heads if emb and heads else None),
               "vocab_size": g("vocab_size") or (self.tensors["token_embd.weight"].shape[0]
                                                 if "token_embd.weight" in self.tensors else None)}
        cfg["tie_word_embeddings"] = "output.weight" not in self.tensors
        return {k: v for k, v in cfg.items() if v is not None}

    def to_hf_state_dict(self, dtype: torch.dtype = torch.bfloat16) -> dict:
        """Dequantised tensors under HF names. For the llama architecture llama.cpp stores Q and K projection rows
        permuted for its interleaved RoPE; they are permuted back to the HF (rotate-half) order. qwen2 / qwen3 files
        keep the HF order (and carry projection biases / per-head norm weights under the same block names)."""
        cfg = self.hf_config()
        permuted = _ARCH[self.metadata.get("general.architecture", "llama")][1]
        out = {}
        for name in self.tensors:
            hf = hf_name(name)
            if hf is None:
                continue
            t = self.get(name, dtype)
            if not permuted:
                pass
            elif name.endswith("attn_q.weight"):
                t = _unpermute_qk(t, cfg["num_attention_heads"])
            elif name.endswith("attn_k.weight"):
                t = _unpermute_qk(t, cfg["num_key_value_heads"])
            out[hf] = t
        return out


_TOP = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
        "output.weight": "lm_head.weight"}
# general.architecture -> (HF architecture, Q / K rows stored in llama.cpp's interleaved-rotary order)
_ARCH = {"llama": ("LlamaForCausalLM", True), "qwen2": ("Qwen2ForCausalLM", False), "qwen3": ("Qwen3ForCausalLM", False)}
_LAYER = {"attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm", "attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "attn_q": "self_attn.q_proj",
          "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj",
          "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}


def hf_name(gguf_name: str) -> Optional[str]:
    if gguf_name in _TOP:
        return _TOP[gguf_name]
    parts = gguf_name.split(".")
    if len(parts) == 4 and parts[0] == "blk" and parts[2] in _LAYER:
        return f"model.layers.{parts[1]}.{_LAYER[parts[2]]}.{parts[3]}"
    return None


def _permute_qk(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """HF -> llama.cpp row order (the converter's permutation)."""
    return w.reshape(n_head, 2, w.shape[0] // n_head // 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def _unpermute_qk(w: torch.Tensor, n_head: int) -> torch.Tensor:
    return w.reshape(n_head, w.shape[0] // n_head // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


# ------------------------------------------------------------------------------ writer (tools and tests)
def quantize_q8_0(x: np.ndarray) -> bytes:
    b = x.astype(np.float32).reshape(-1, 32)
    d = np.abs(b).max(axis=1, keepdims=True) / 127.0
    q = np.where(d > 0, np.round(b / np.where(d > 0, d, 1)), 0).astype(np.int8)
    return np.concatenate([d.astype(np.float16).view(np.uint8), q.view(np.uint8)], axis=1).tobytes()


def quantize_q4_0(x: np.ndarray) -> bytes:
    b = x.astype(np.float32).reshape(-1, 32)
    idx = np.abs(b).argmax(axis=1)
    mx = b[np.arange(b.shape[0]), idx]
    d = (mx / -8.0).reshape(-1, 1)
    q = np.clip(np.round(np.where(d != 0, b / np.where(d != 0, d, 1), 0) + 8), 0, 15).astype(np.uint8)
    packed = q[:, :16] | (q[:, 16:] << 4)
    return np.concatenate([d.astype(np.float16).view(np.uint8), packed], axis=1).tobytes()


def write_gguf(path: str, metadata: dict, tensors: dict, align: int = 32) -> None:
    """tensors: name -> (numpy array, ggml_type) with type in {F32, F16, Q8_0, Q4_0}."""
    def s(v: str) -> bytes:
        b = v.encode("utf-8")
        return struct.pack("<Q", len(b)) + b

    def val(v) -> bytes:
        if isinstance(v, bool):
            return struct.pack("<I?", T_BOOL, v)
        if isinstance(v, int):
            return struct.pack("<Iq", T_I64, v) if v < 0 or v >= 2 ** 32 else struct.pack("<II", T_U32, v)
        if isinstance(v, float):
            return struct.pack("<If", T_F32, v)
        if isinstance(v, str):
            return struct.pack("<I", T_STR) + s(v)
        if isinstance(v, (list, tuple)):
            if all(isinstance(e, str) for e in v):
                return struct.pack("<IIQ", T_ARR, T_STR, len(v)) + b"".join(s(e) for e in v)
            if all(isinstance(e, int) for e in v):
                return struct.pack("<IIQ", T_ARR, T_I32, len(v)) + struct.pack(f"<{len(v)}i", *v)
            return struct.pack("<IIQ", T_ARR, T_F32, len(v)) + struct.pack(f"<{len(v)}f", *v)
        raise TypeError(f"unsupported metadata value {v!r}")

    metadata = dict(metadata)
    metadata.setdefault("general.alignment", align)
    blobs, infos, off = [], [], 0
    for name, (arr, t) in tensors.items():
        if t == GGML_F32:
            raw = arr.astype(np.float32).tobytes()
        elif t == GGML_F16:
            raw = arr.astype(np.float16).tobytes()
        elif t == GGML_Q8_0:
            raw = quantize_q8_0(arr)
        elif t == GGML_Q4_0:
            raw = quantize_q4_0(arr)
        else:
            raise ValueError("writer supports F32, F16, Q8_0 and Q4_0")
        infos.append(s(name) + struct.pack("<I", arr.ndim) + b"".join(struct.pack("<Q", d) for d in reversed(arr.shape))
                     + struct.pack("<IQ", t, off))
        pad = (-len(raw)) % align
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(metadata))
    head += b"".join(s(k) + val(v) for k, v in metadata.items()) + b"".join(infos)
    head += b"\0" * ((-len(head)) % align)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)
