"""Ragged batch packing: contexts + KV pages -> one metadata buffer per step.

Everything the device needs besides weights and cache for one forward pass - token ids,
positions, KV slots, block table, per-sequence lengths, the attention work split, the rows
whose logits are wanted and the per-row sampling parameters - is laid out in **one int32
buffer**, written in pinned host memory and uploaded with a single H2D copy. The native
executor reads the arrays at fixed offsets, so a decode step with a fixed layout replays
under a CUDA graph with only that copy changing.

The reference builds the same inputs as separate tensors (ragged ``tokens`` +
``input_row_offsets`` + KV lookup table + ``cache_lengths``: max/python/max/pipelines/
architectures/llama3/batch_processor.py:43, kv_cache/paged_kv_cache/cache_manager.py:695).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from ..ops import build_attention_plan
from .context import FUTURE_TOKEN, TextContext

# arrays in the packed buffer; (name, words per element, per-"T" | per-"B" | per-"tile" | "bt")
_FIELDS = [
    ("tokens", 2, "T"), ("slots", 2, "T"), ("seeds", 2, "R"),
    ("positions", 1, "T"), ("future_src", 1, "T"),
    ("q_start", 1, "B"), ("q_len", 1, "B"), ("kv_len", 1, "B"), ("decode_seq", 1, "B"),
    ("logit_rows", 1, "R"), ("temperature", 1, "R"), ("top_k", 1, "R"), ("top_p", 1, "R"),
    ("min_p", 1, "R"), ("tile_seq", 1, "tile"), ("tile_q0", 1, "tile"), ("block_table", 1, "bt"),
]


def meta_layout(T_cap: int, B_cap: int, bt_stride: int, tiles_cap: int, rows_cap: int = 0):
    """Offsets (in int32 words) of every array for the given capacities. ``rows_cap``: rows that can ask for
    logits (one per sequence unless draft tokens are verified, then one per token)."""
    sizes = {"T": max(T_cap, 1), "B": max(B_cap, 1), "tile": max(tiles_cap, 1),
             "R": max(rows_cap, B_cap, 1), "bt": max(B_cap, 1) * max(bt_stride, 1)}
    off, cur = {}, 0
    for name, words, kind in _FIELDS:
        if words == 2 and cur % 2:
            cur += 1
        off[name] = cur
        cur += words * sizes[kind]
        cur = (cur + 3) & ~3  # keep every array 16-byte aligned
    return off, cur


@dataclass
class StepBatch:
    ctxs: list
    T: int
    B: int
    bt_stride: int
    n_tiles: int
    n_decode: int
    n_logits: int
    offsets: dict
    words: int
    host: np.ndarray                      # int32 view of the pinned staging buffer
    logit_ctx: list = field(default_factory=list)   # contexts that sample this step, in row order
    all_greedy: bool = True
    has_future: bool = False

    def arr(self, name: str, dtype=np.int32, count: Optional[int] = None) -> np.ndarray:
        o = self.offsets[name]
        if dtype in (np.int64, np.uint64):
            return self.host[o : o + 2 * count].view(dtype)
        return self.host[o : o + count].view(dtype)


class BatchPacker:
    def __init__(self, n_q: int, n_kv: int, page_size: int, max_tokens: int, max_seqs: int,
                 max_pages_per_seq: int, device="cpu", n_staging: int = 4, max_logit_rows: int = 0):
        self.n_q, self.n_kv, self.page_size = n_q, n_kv, page_size
        self.max_tokens, self.max_seqs, self.max_pages = max_tokens, max_seqs, max_pages_per_seq
        self.device = torch.device(device)
        G = n_q // n_kv
        self.tok_per_tile = max(1, 64 // G)
        tiles_cap = max_tokens // self.tok_per_tile + max_seqs + 1
        self.max_logit_rows = max(max_logit_rows, max_seqs)
        _, words = meta_layout(max_tokens, max_seqs, max_pages_per_seq, tiles_cap, self.max_logit_rows)
        self.capacity_words = words
        pin = self.device.type == "cuda"
        self._staging = [torch.empty(words, dtype=torch.int32, pin_memory=pin) for _ in range(n_staging)]
        self._staging_np = [t.numpy() for t in self._staging]
        self._events = [None] * n_staging
        self._next = 0
        self.meta_dev = (torch.empty(words, dtype=torch.int32, device=self.device) if pin else None)

    def _acquire(self) -> int:
        i = self._next
        self._next = (self._next + 1) % len(self._staging)
        ev = self._events[i]
        if ev is not None:
            ev.synchronize()  # the copy that last used this staging buffer has finished
        return i

    def pack(self, ctxs: Sequence[TextContext], kv, fixed: Optional[tuple] = None,
             pad_to: int = 0, all_logits: bool = False) -> StepBatch:
        """Build the metadata for ``ctxs`` (each contributes its active window).

        ``fixed = (T_cap, B_cap, bt_stride, tiles_cap)`` pins the layout (CUDA-graph replay);
        ``pad_to`` pads the batch with dummy single-token sequences on the null page;
        ``all_logits`` asks for the logits of every row of a window that reaches the last known token
        (verification of draft tokens), not only of its last row: the per-row sampling arrays are then laid
        out for one entry per token.
        """
        B_real = len(ctxs)
        B = max(B_real, pad_to)
        q_lens = np.fromiter((c.tokens.active_length for c in ctxs), dtype=np.int32, count=B_real)
        if pad_to > B_real:
            q_lens = np.concatenate([q_lens, np.ones(pad_to - B_real, dtype=np.int32)])
        T = int(q_lens.sum())
        if T > self.max_tokens or B > self.max_seqs:
            raise ValueError(f"batch ({T} tokens, {B} sequences) exceeds limits "
                             f"({self.max_tokens}, {self.max_seqs})")
        tile_seq, tile_q0, decode_seq = build_attention_plan(q_lens, self.n_q, self.n_kv)
        if fixed is None:
            bt_stride = max([len(kv.blocks_of(c.request_id)) for c in ctxs] + [1])
            if all_logits and T > self.max_logit_rows:
                raise ValueError(f"{T} rows ask for logits; the pipeline was built for {self.max_logit_rows}")
            off, words = meta_layout(T, B, bt_stride, len(tile_seq), T if all_logits else 0)
        else:
            T_cap, B_cap, bt_stride, tiles_cap = fixed
            off, words = meta_layout(T_cap, B_cap, bt_stride, tiles_cap)
        si = self._acquire()
        host = self._staging_np[si]
        sb = StepBatch(list(ctxs), T, B, bt_stride, len(tile_seq), len(decode_seq), 0, off, words, host)
        sb._staging_index = si

        tokens = sb.arr("tokens", np.int64, T)
        slots = sb.arr("slots", np.int64, T)
        positions = sb.arr("positions", np.int32, T)
        future_src = sb.arr("future_src", np.int32, T)
        q_start = sb.arr("q_start", np.int32, B)
        q_len = sb.arr("q_len", np.int32, B)
        kv_len = sb.arr("kv_len", np.int32, B)
        bt = sb.arr("block_table", np.int32, B * bt_stride).reshape(B, bt_stride)
        n_rows_cap = max(B, T) if all_logits else B
        logit_rows = sb.arr("logit_rows", np.int32, n_rows_cap)
        temperature = sb.arr("temperature", np.float32, n_rows_cap)
        top_k = sb.arr("top_k", np.int32, n_rows_cap)
        top_p = sb.arr("top_p", np.float32, n_rows_cap)
        min_p = sb.arr("min_p", np.float32, n_rows_cap)
        seeds = sb.arr("seeds", np.int64, n_rows_cap)

        q_len[:] = q_lens
        q_start[0] = 0
        if B > 1:
            np.cumsum(q_lens[:-1], out=q_start[1:])
        future_src[:] = -1
        bt[:] = 0
        n_logits = 0
        ps = self.page_size
        row = 0
        for i, c in enumerate(ctxs):
            tb = c.tokens
            n = tb.active_length
            p0 = tb.processed
            tokens[row : row + n] = tb.active
            positions[row : row + n] = np.arange(p0, p0 + n, dtype=np.int32)
            blocks = kv.blocks_of(c.request_id)
            nb = len(blocks)
            bt[i, :nb] = blocks
            if n == 1:
                slots[row] = blocks[p0 // ps] * ps + p0 % ps
                if tokens[row] == FUTURE_TOKEN:
                    future_src[row] = c.sample_slot
                    sb.has_future = True
            else:
                pos = positions[row : row + n].astype(np.int64)
                slots[row : row + n] = bt[i, pos // ps].astype(np.int64) * ps + pos % ps
            kv_len[i] = tb.active_end
            if tb.active_end == len(tb):
                # the window reaches the last known token: this pass produces a new token
                sp = c.sampling_params
                for r in (range(row, row + n) if all_logits else (row + n - 1,)):
                    logit_rows[n_logits] = r
                    temperature[n_logits] = 0.0 if sp.is_greedy else sp.temperature
                    top_k[n_logits] = sp.top_k if sp.top_k > 0 else 0
                    top_p[n_logits] = sp.top_p
                    min_p[n_logits] = sp.min_p
                    seeds[n_logits] = sp.seed * 1000003 + c.seq
                    sb.logit_ctx.append(c)
                    n_logits += 1
                if not sp.is_greedy:
                    sb.all_greedy = False
            row += n
        # dummy padding sequences: one token each on the null page, logits wanted (graph shape)
        for i in range(B_real, B):
            tokens[row] = 0
            positions[row] = 0
            slots[row] = -1
            kv_len[i] = 1
            logit_rows[n_logits] = row
            temperature[n_logits] = 0.0
            top_k[n_logits] = 0
            top_p[n_logits] = 1.0
            min_p[n_logits] = 0.0
            seeds[n_logits] = 0
            n_logits += 1
            row += 1
        sb.n_logits = n_logits
        sb.arr("tile_seq", np.int32, len(tile_seq))[:] = tile_seq
        sb.arr("tile_q0", np.int32, len(tile_q0))[:] = tile_q0
        sb.arr("decode_seq", np.int32, len(decode_seq))[:] = decode_seq
        return sb

    def upload(self, sb: StepBatch) -> torch.Tensor:
        """Single H2D copy of the packed buffer (async on the current stream)."""
        si = sb._staging_index
        self.meta_dev[: sb.words].copy_(self._staging[si][: sb.words], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[si] = ev
        return self.meta_dev

    @staticmethod
    def tensors(sb: StepBatch, device="cpu") -> dict:
        """Per-array torch tensors (CPU op-by-op path and tests)."""
        t = lambda name, dt, n: torch.from_numpy(sb.arr(name, dt, n).copy()).to(device)
        return dict(
            tokens=t("tokens", np.int64, sb.T), positions=t("positions", np.int32, sb.T),
            slots=t("slots", np.int64, sb.T), q_start=t("q_start", np.int32, sb.B),
            q_len=t("q_len", np.int32, sb.B), kv_len=t("kv_len", np.int32, sb.B),
            block_table=t("block_table", np.int32, sb.B * sb.bt_stride).view(sb.B, sb.bt_stride),
            logit_rows=t("logit_rows", np.int32, sb.n_logits),
            temperature=t("temperature", np.float32, sb.n_logits),
            top_k=t("top_k", np.int32, sb.n_logits), top_p=t("top_p", np.float32, sb.n_logits),
            min_p=t("min_p", np.float32, sb.n_logits), seeds=t("seeds", np.int64, sb.n_logits),
            future_src=t("future_src", np.int32, sb.T))
