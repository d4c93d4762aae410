"""Wire format of the API <-> model-worker hop: msgpack through msgspec, no pickle.

Every message is a msgpack map ``{"t": kind, ...}`` built from plain types only, so a malformed or hostile
frame can at worst fail to decode; nothing on the wire can name a Python callable. Kinds:

    ctx    a new request: ids as raw little-endian int64 bytes, sampling parameters as a map
    out    a batch of per-request outputs of one scheduler step
    emb    the answer to an embeddings request
    raw    anything else made of msgpack-native values (cancel ids, RPC tuples, metric maps)

Reference: the msgspec (de)serialisation of contexts and ``SchedulerResult`` in
max/python/max/serve/worker_interface/zmq_interface.py:50 and ``_zmq_queue.py``.
"""

from __future__ import annotations

import dataclasses

import msgspec
import numpy as np

from ...pipelines.context import (EmbeddingsOutput, GenerationStatus, SamplingParams, TextContext,
                                  TextGenerationOutput, TokenBuffer)

_enc = msgspec.msgpack.Encoder()
_dec = msgspec.msgpack.Decoder()
_SP_FIELDS = tuple(f.name for f in dataclasses.fields(SamplingParams))


def _plain(v):
    """numpy scalars / arrays -> builtins (log-probability entries carry them)."""
    if isinstance(v, np.generic):
        return v.item()
    if isinstance(v, np.ndarray):
        return v.tolist()
    if isinstance(v, dict):
        return {k: _plain(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    return v


def _ctx_to_wire(c: TextContext) -> dict:
    if c.tokens.generated_length or c.tokens.processed:
        raise ValueError("only fresh requests cross the process hop")
    return {"t": "ctx", "id": c.request_id, "ids": c.tokens.prompt.astype("<i8").tobytes(), "max_length": c.max_length,
            "sp": {k: getattr(c.sampling_params, k) for k in _SP_FIELDS}, "eos": sorted(int(t) for t in c.eos_token_ids),
            "model": c.model_name, "task": c.task, "pooling": c.pooling, "lora": c.lora_name,
            "salt": int(c.cache_salt), "schema": c.json_schema, "arrival": c.arrival_time}


def _ctx_from_wire(m: dict) -> TextContext:
    ids = np.frombuffer(m["ids"], dtype="<i8")
    c = TextContext(request_id=m["id"], tokens=TokenBuffer(ids), max_length=m["max_length"],
                    sampling_params=SamplingParams(**m["sp"]), eos_token_ids=frozenset(m["eos"]), model_name=m["model"])
    c.task, c.pooling, c.lora_name = m["task"], m["pooling"], m["lora"]
    c.cache_salt, c.json_schema, c.arrival_time = m["salt"], m["schema"], m["arrival"]
    return c


def _out_to_wire(o) -> list:
    if isinstance(o, EmbeddingsOutput):
        return ["emb", o.request_id, [float(x) for x in o.embedding], o.prompt_tokens]
    return ["gen", o.request_id, [int(t) for t in o.tokens], o.final_status.value, _plain(o.log_probabilities),
            getattr(o, "error", None)]


def _out_from_wire(w: list):
    if w[0] == "emb":
        return EmbeddingsOutput(w[1], w[2], w[3])
    lps = w[4]
    if lps is not None:
        lps = [dict(e, top=[tuple(p) for p in e.get("top", [])]) if isinstance(e, dict) else e for e in lps]
    return TextGenerationOutput(w[1], w[2], GenerationStatus(w[3]), lps, w[5] if len(w) > 5 else None)


def encode(obj) -> bytes:
    if isinstance(obj, TextContext):
        return _enc.encode(_ctx_to_wire(obj))
    if isinstance(obj, dict) and obj and all(isinstance(v, (TextGenerationOutput, EmbeddingsOutput)) for v in obj.values()):
        return _enc.encode({"t": "out", "items": [_out_to_wire(v) for v in obj.values()]})
    return _enc.encode({"t": "raw", "v": _plain(obj)})


def decode(buf: bytes):
    m = _dec.decode(buf)
    kind = m.get("t") if isinstance(m, dict) else None
    if kind == "ctx":
        return _ctx_from_wire(m)
    if kind == "out":
        outs = [_out_from_wire(w) for w in m["items"]]
        return {o.request_id: o for o in outs}
    if kind == "raw":
        v = m["v"]
        return tuple(v) if isinstance(v, list) else v
    raise ValueError("unknown message kind on the worker queue")
