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


def test_grammar_compiles_off_the_scheduler_thread_and_failures_stay_local():
    """A constrained request waits for its grammar on a worker thread while other requests are served; a grammar
    that does not compile fails that request with a message and nothing else."""
    import threading
    import time

    import torch

    from modular_b200.entrypoints.llm import LLM
    from modular_b200.models.llama3 import Llama3Config
    from modular_b200.pipelines.context import GenerationStatus, SamplingParams, TextContext
    from modular_b200.pipelines.structured_output import GrammarGate

    class SlowBackend:
        def __init__(self):
            self.release = threading.Event()

        def compile(self, spec):
            if spec.get("pattern") == "bad":
                raise RuntimeError("[00:00:00] /src/grammar.cc:12: unexpected token")
            self.release.wait(5.0)

            class State:
                def accept(self, t):
                    return True
            return State()

    backend = SlowBackend()
    gate = GrammarGate(backend, workers=2)
    mk = lambda rid, spec: TextContext.from_prompt([1, 2, 3], 32, rid, SamplingParams(
        temperature=0.0, max_new_tokens=2, response_format=spec))
    plain, slow, bad = mk("p", None), mk("s", {"type": "regex", "pattern": "ok"}), mk("b", {"type": "regex", "pattern": "bad"})
    assert gate.submit(plain) is False and gate.ready(plain)
    assert gate.submit(slow) and gate.submit(bad)
    deadline = time.time() + 5
    while not gate.ready(bad) and time.time() < deadline:
        time.sleep(0.01)
    assert gate.ready(bad) and not gate.ready(slow)
    assert gate.install(bad) == "the grammar of this request cannot be compiled: unexpected token"
    backend.release.set()
    while not gate.ready(slow) and time.time() < deadline:
        time.sleep(0.01)
    assert gate.install(slow) is None and slow.grammar_state is not None
    gate.shutdown()

    # through the scheduler: the unconstrained request finishes while the other one still compiles
    cfg = Llama3Config.tiny(num_hidden_layers=1, vocab_size=64)
    llm = LLM(cfg, device="cpu", dtype=torch.float32, max_length=64, max_batch_size=4, max_batch_input_tokens=32,
              page_size=16, num_kv_pages=16)
    backend2 = SlowBackend()
    llm.pipeline.structured = backend2
    llm.pipeline._grammar_bitmask = lambda sb: None           # the stub has no token masks
    sched = llm.scheduler
    a, b, c = mk("plain", None), mk("slow", {"type": "regex", "pattern": "ok"}), mk("bad", {"type": "regex", "pattern": "bad"})
    for x in (a, b, c):
        sched.add_request(x)
    outs = {}
    t_end = time.time() + 20
    while ("plain" not in outs or not outs["plain"].is_done or "bad" not in outs) and time.time() < t_end:
        sched.run_iteration()
        while True:
            try:
                for rid, o in sched.response_queue.get_nowait().items():
                    prev = outs.get(rid)
                    outs[rid] = o if prev is None else type(o)(rid, list(prev.tokens) + list(o.tokens), o.final_status,
                                                               None, o.error)
            except Exception:      # noqa: BLE001 - queue empty
                break
    assert outs["plain"].is_done and len(outs["plain"].tokens) == 2
    assert outs["bad"].final_status is GenerationStatus.ERROR and "unexpected token" in outs["bad"].error
    assert "slow" not in outs and sched.has_work()            # still compiling, nobody waited for it
    backend2.release.set()
    while ("slow" not in outs or not outs["slow"].is_done) and time.time() < t_end:
        sched.run_iteration()
        try:
            for rid, o in sched.response_queue.get_nowait().items():
                prev = outs.get(rid)
                outs[rid] = o if prev is None else type(o)(rid, list(prev.tokens) + list(o.tokens), o.final_status, None, o.error)
        except Exception:      # noqa: BLE001
            time.sleep(0.005)
    assert outs["slow"].is_done and len(outs["slow"].tokens) == 2
