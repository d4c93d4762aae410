"""Grammar-constrained decoding on CPU: a random tiny model must still emit text that matches the grammar."""

import json
import re

import numpy as np
import pytest
import torch

from modular_b200 import ops
from modular_b200.entrypoints.llm import LLM
from modular_b200.models.llama3 import Llama3Config
from modular_b200.pipelines.context import SamplingParams
from modular_b200.pipelines.structured_output import apply_token_bitmask_reference, response_format_to_spec
from modular_b200.pipelines.tokenizer import ByteTokenizer

pytest.importorskip("xgrammar")


def _llm(**kw):
    cfg = Llama3Config.tiny(vocab_size=258)
    llm = LLM(cfg, device="cpu", dtype=torch.float32, max_length=256, max_batch_size=4, max_batch_input_tokens=64,
              page_size=16, num_kv_pages=64, eos_token_ids=(ByteTokenizer.EOS,), **kw)
    llm.pipeline.enable_structured_output(ByteTokenizer())
    return llm


def test_regex_and_schema_constrained_generation():
    llm = _llm()
    tok = ByteTokenizer()
    prompts = [tok.encode("answer:"), tok.encode("json:"), tok.encode("free:")]
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"enum": [1, 2, 3]}},
              "required": ["ok", "n"], "additionalProperties": False}
    sps = [SamplingParams(temperature=0.9, seed=1, max_new_tokens=40, response_format={"type": "regex", "pattern": "(yes|no|maybe)!"}),
           SamplingParams(temperature=0.9, seed=2, max_new_tokens=80,
                          response_format={"type": "json_schema", "schema": json.dumps(schema), "compact": True}),
           SamplingParams(temperature=0.0, max_new_tokens=5, ignore_eos=True)]
    out = llm.generate(prompts, sps)
    text = [tok.decode([t for t in r.tokens if t < 256]) for r in out]
    assert re.fullmatch(r"(yes|no|maybe)!", text[0]), text[0]
    assert out[0].tokens[-1] == ByteTokenizer.EOS
    obj = json.loads(text[1])
    assert set(obj) == {"ok", "n"} and isinstance(obj["ok"], bool) and obj["n"] in (1, 2, 3)
    assert len(out[2].tokens) == 5      # the unconstrained request in the same batch is untouched


def test_bitmask_reference_and_response_format_parsing():
    logits = torch.zeros(2, 70)
    bm = torch.full((2, 3), -1, dtype=torch.int32)
    bm[0, 0] = 0b101
    bm[0, 1:] = 0
    apply_token_bitmask_reference(logits, bm)
    assert torch.isfinite(logits[0]).nonzero().flatten().tolist() == [0, 2] and torch.isfinite(logits[1]).all()
    assert response_format_to_spec(None) is None and response_format_to_spec({"type": "text"}) is None
    assert response_format_to_spec({"type": "json_object"}) == {"type": "json_object"}
    spec = response_format_to_spec({"type": "json_schema", "json_schema": {"name": "x", "schema": {"type": "object"}}})
    assert spec["type"] == "json_schema" and json.loads(spec["schema"]) == {"type": "object"}
    with pytest.raises(ValueError):
        response_format_to_spec({"type": "yaml"})


@pytest.mark.gpu
def test_bitmask_kernel_matches_reference():
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(5, 1000, generator=g).cuda()
    bm = torch.randint(-2**31, 2**31 - 1, (5, 32), generator=g, dtype=torch.int64).to(torch.int32)
    want = logits.cpu().clone()
    apply_token_bitmask_reference(want, bm)
    ops.apply_token_bitmask(logits, bm)
    assert torch.equal(logits.cpu(), want)
