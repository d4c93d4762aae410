"""Server tests on CPU: OpenAI routes end to end through the real worker process (ZMQ IPC),
with the echo pipeline and with the tiny Llama preset."""

import json
import os

import pytest
from fastapi.testclient import TestClient

from modular_b200.pipelines.config import PipelineArgs, PipelineConfig
from modular_b200.pipelines.registry import PIPELINE_REGISTRY
from modular_b200.pipelines.tokenizer import ByteTokenizer
from modular_b200.serve.api_server import fastapi_app
from modular_b200.serve.config import Settings
from modular_b200.serve.pipelines.echo_gen import EchoPipeline
from modular_b200.serve.pipelines.incremental_detokenizer import IncrementalDetokenizer


def _config(**flat):
    return PipelineConfig.from_args(PipelineArgs.from_flat_kwargs(None, **flat))


@pytest.fixture(scope="module")
def echo_client():
    settings = Settings(metric_recording="ASYNCIO", max_queue_size=64)
    pc = _config(model_path="echo", devices="cpu")
    app = fastapi_app(settings, pc, ByteTokenizer(), EchoPipeline, "echo", 4096)
    with TestClient(app) as c:
        yield c


def test_health_models_metrics(echo_client):
    assert echo_client.get("/health").json() == {"status": "ok"}
    assert echo_client.get("/version").json()["version"]
    assert [m["id"] for m in echo_client.get("/v1/models").json()["data"]] == ["echo"]
    assert echo_client.get("/v1/models/nope").status_code == 404
    assert b"maxserve_request_count" in echo_client.get("/metrics").content


def test_completion_echo(echo_client):
    r = echo_client.post("/v1/completions", json={"model": "echo", "prompt": "hello world", "max_tokens": 64})
    assert r.status_code == 200, r.text
    body = r.json()
    assert body["choices"][0]["text"] == "hello world"
    assert body["choices"][0]["finish_reason"] == "stop"
    assert body["usage"]["prompt_tokens"] == 12 and body["usage"]["completion_tokens"] >= 11


def test_completion_max_tokens_and_stop(echo_client):
    r = echo_client.post("/v1/completions", json={"model": "echo", "prompt": "abcdefghij", "max_tokens": 4})
    assert r.json()["choices"][0]["finish_reason"] == "length"
    r = echo_client.post("/v1/completions", json={"model": "echo", "prompt": "one two three", "max_tokens": 64,
                                                  "stop": ["two"]})
    c = r.json()["choices"][0]
    assert c["text"] == "one " and c["finish_reason"] == "stop"


def test_chat_stream(echo_client):
    with echo_client.stream("POST", "/v1/chat/completions", json={
            "model": "echo", "stream": True, "max_tokens": 200, "stream_options": {"include_usage": True},
            "messages": [{"role": "user", "content": "ping"}]}) as r:
        assert r.status_code == 200
        chunks = [l[6:] for l in r.iter_lines() if l.startswith("data: ")]
    assert chunks[-1] == "[DONE]"
    objs = [json.loads(c) for c in chunks[:-1]]
    assert objs[0]["choices"][0]["delta"]["role"] == "assistant"
    text = "".join(o["choices"][0]["delta"].get("content") or "" for o in objs if o["choices"])
    assert "ping" in text
    assert objs[-1]["usage"]["completion_tokens"] > 0
    assert any(o["choices"] and o["choices"][0].get("finish_reason") == "stop" for o in objs)


def test_errors(echo_client):
    r = echo_client.post("/v1/completions", json={"model": "other", "prompt": "x"})
    assert r.status_code == 404 and r.json()["error"]["type"] == "not_found_error"
    r = echo_client.post("/v1/completions", json={"model": "echo"})
    assert r.status_code == 400 and "prompt" in r.json()["error"]["message"]
    r = echo_client.post("/v1/completions", json={"model": "echo", "prompt": "x", "temperature": -1})
    assert r.status_code == 400


def test_embeddings_unavailable_on_echo(echo_client):
    r = echo_client.post("/v1/embeddings", json={"model": "echo", "input": "x"})
    assert r.status_code == 400 and "embeddings" in r.json()["error"]["message"]


def test_worker_rpc(echo_client):
    assert echo_client.get("/max_internal/worker_stats").json()["steps"] > 0
    # the worker's per-step metrics reach the API process's registry
    import time
    for _ in range(50):
        body = echo_client.get("/metrics").content
        if b"maxserve_batch_size_count 0.0" not in body:
            break
        time.sleep(0.1)
    assert b"maxserve_batch_size_count" in body and b"maxserve_batch_size_count 0.0" not in body
    for name in (b"maxserve_batch_execution_time_ms", b"maxserve_cache_used_kv_pct", b"maxserve_batch_pending_reqs",
                 b"maxserve_batch_generation_throughput", b"maxserve_cache_preemption_count"):
        assert name in body
    assert echo_client.post("/reset_prefix_cache").json() == {"success": False}  # echo has no cache
    assert echo_client.get("/health/live").json() == {"status": "ok"}
    assert echo_client.get("/health/ready").status_code == 200


def test_tiny_llama_server():
    pc = _config(model_path="preset:tiny-llama", devices="cpu", max_length=256, max_batch_size=4,
                 max_batch_input_tokens=128, kv_cache_page_size=16)
    tokenizer, factory = PIPELINE_REGISTRY.retrieve_factory(pc)
    app = fastapi_app(Settings(), pc, tokenizer, factory, "tiny", 256)
    with TestClient(app) as c:
        a = c.post("/v1/completions", json={"model": "tiny", "prompt": [5, 6, 7, 8, 9], "max_tokens": 6,
                                            "temperature": 0, "ignore_eos": True}).json()
        b = c.post("/v1/completions", json={"model": "tiny", "prompt": [5, 6, 7, 8, 9], "max_tokens": 6,
                                            "temperature": 0, "ignore_eos": True}).json()
        assert a["usage"]["completion_tokens"] == 6 and a["choices"][0]["finish_reason"] == "length"
        assert a["choices"][0]["text"] == b["choices"][0]["text"]
        assert c.post("/reset_prefix_cache").json() == {"success": True}
        # log-probabilities: greedy token is the most likely alternative, values are valid log-probs
        lp = c.post("/v1/completions", json={"model": "tiny", "prompt": [5, 6, 7, 8, 9], "max_tokens": 4,
                                             "temperature": 0, "ignore_eos": True, "logprobs": 3}).json()
        info = lp["choices"][0]["logprobs"]
        assert len(info["token_logprobs"]) == 4 and all(v <= 0 for v in info["token_logprobs"])
        assert all(1 <= len(t) <= 3 for t in info["top_logprobs"])      # byte tokenizer: ids above 255 share a text
        assert lp["choices"][0]["text"] == a["choices"][0]["text"][: len(lp["choices"][0]["text"])]
        ch = c.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "hi"}],
                                                   "max_tokens": 3, "logprobs": True, "top_logprobs": 2}).json()
        assert len(ch["choices"][0]["logprobs"]["content"]) == ch["usage"]["completion_tokens"]
        # embeddings from the same worker: unit vectors, deterministic, pooled per input
        e = c.post("/v1/embeddings", json={"model": "tiny", "input": [[5, 6, 7], [9, 9], [5, 6, 7]]}).json()
        v = [d["embedding"] for d in e["data"]]
        assert len(v) == 3 and e["usage"]["prompt_tokens"] == 8
        assert abs(sum(x * x for x in v[0]) - 1.0) < 1e-4 and v[0] == v[2] and v[0] != v[1]
        m = c.post("/v1/embeddings", json={"model": "tiny", "input": "hello", "pooling": "mean",
                                           "encoding_format": "base64", "dimensions": 16}).json()
        import base64
        assert len(base64.b64decode(m["data"][0]["embedding"])) == 64


def test_encoder_and_state_space_presets_behind_the_server():
    """An encoder-only preset answers /v1/embeddings with its own default pooling and refuses generation with a
    client error; a state-space preset generates through the same routes."""
    pc = _config(model_path="preset:tiny-bert", devices="cpu", max_length=128, max_batch_size=4,
                 max_batch_input_tokens=128, quantization_encoding="float32")
    tokenizer, factory = PIPELINE_REGISTRY.retrieve_factory(pc)
    with TestClient(fastapi_app(Settings(), pc, tokenizer, factory, "enc", 128)) as c:
        e = c.post("/v1/embeddings", json={"model": "enc", "input": [[5, 6, 7], [9, 9]]}).json()
        v = [d["embedding"] for d in e["data"]]
        assert len(v) == 2 and abs(sum(x * x for x in v[0]) - 1.0) < 1e-4
        cls = c.post("/v1/embeddings", json={"model": "enc", "input": [[5, 6, 7]], "pooling": "cls"}).json()
        assert cls["data"][0]["embedding"] != v[0]
        r = c.post("/v1/completions", json={"model": "enc", "prompt": [5, 6, 7], "max_tokens": 2})
        assert r.status_code == 400 and "embeddings" in r.json()["error"]["message"], r.text
        assert c.get("/health").status_code == 200
    pc = _config(model_path="preset:tiny-mamba", devices="cpu", max_length=128, max_batch_size=4,
                 max_batch_input_tokens=64, quantization_encoding="float32")
    tokenizer, factory = PIPELINE_REGISTRY.retrieve_factory(pc)
    with TestClient(fastapi_app(Settings(), pc, tokenizer, factory, "ssm", 128)) as c:
        a = c.post("/v1/completions", json={"model": "ssm", "prompt": [5, 6, 7, 8], "max_tokens": 5, "temperature": 0,
                                            "ignore_eos": True}).json()
        b = c.post("/v1/completions", json={"model": "ssm", "prompt": [5, 6, 7, 8], "max_tokens": 5, "temperature": 0,
                                            "ignore_eos": True}).json()
        assert a["usage"]["completion_tokens"] == 5 and a["choices"][0]["text"] == b["choices"][0]["text"]


def test_incremental_detokenizer_utf8_and_stop():
    tok = ByteTokenizer()
    d = IncrementalDetokenizer(tok, stop=["END"])
    ids = tok.encode("héllo wörld EN", add_special_tokens=False)
    out = "".join(d.push([i]) for i in ids)
    assert out == "héllo wörld "          # "EN" is held back: it may become "END"
    assert d.push(tok.encode("X", add_special_tokens=False)) == "ENX"
    d2 = IncrementalDetokenizer(tok, stop=["END"])
    out = "".join(d2.push([i]) for i in tok.encode("abcENDdef", add_special_tokens=False))
    assert out == "abc" and d2.stopped


# ------------------------------------------------------------------ other API front ends
@pytest.fixture(scope="module")
def multi_api_client(tmp_path_factory):
    rec = tmp_path_factory.mktemp("rec") / "transactions.jsonl"
    settings = Settings(api_types=["openai", "kserve", "sagemaker"], transaction_recording_file=str(rec),
                        transaction_recording_include_responses=True)
    pc = _config(model_path="echo", devices="cpu")
    app = fastapi_app(settings, pc, ByteTokenizer(), EchoPipeline, "echo", 4096)
    with TestClient(app) as c:
        c.recording = rec
        c.asgi_app = app
        yield c


def test_kserve_routes(multi_api_client):
    c = multi_api_client
    assert c.get("/v2/health/live").json() == {"live": True}
    assert c.get("/v2/health/ready").json() == {"ready": True}
    assert c.get("/v2/models/echo").json()["inputs"][0]["name"] == "text_input"
    assert c.get("/v2/models/nope").status_code == 404
    r = c.post("/v2/models/echo/infer", json={"inputs": [{"name": "text_input", "datatype": "BYTES", "shape": [2],
                                                           "data": ["hello", "abc"]}],
                                               "parameters": {"max_tokens": 32}})
    assert r.status_code == 200, r.text
    out = r.json()["outputs"][0]
    assert out["name"] == "text_output" and out["shape"] == [2] and out["data"][0] == "hello"
    bad = c.post("/v2/models/echo/infer", json={"inputs": [{"name": "x", "datatype": "FP32", "data": [1.0]}]})
    assert bad.status_code == 400


def test_sagemaker_routes(multi_api_client):
    c = multi_api_client
    assert c.get("/ping").status_code == 200
    r = c.post("/invocations", json={"prompt": "sage", "max_tokens": 16})
    assert r.status_code == 200 and r.json()["choices"][0]["text"] == "sage"
    r = c.post("/invocations", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 64})
    assert r.status_code == 200 and r.json()["choices"][0]["message"]["role"] == "assistant"
    assert c.post("/invocations", content=b"not json").status_code == 400


def test_openresponses_route(multi_api_client):
    c = multi_api_client
    r = c.post("/v1/responses", json={"model": "echo", "input": "ping", "max_output_tokens": 64})
    body = r.json()
    assert r.status_code == 200 and body["object"] == "response" and body["status"] == "completed"
    assert "ping" in body["output"][0]["content"][0]["text"] and body["usage"]["output_tokens"] > 0
    with c.stream("POST", "/v1/responses", json={"model": "echo", "stream": True, "max_output_tokens": 64,
                                                  "input": [{"role": "user", "content": [{"type": "input_text", "text": "xy"}]}]}) as s:
        events = [l for l in s.iter_lines() if l.startswith("event:")]
    assert events[0] == "event: response.created" and events[-1] == "event: response.completed"
    assert any(e == "event: response.output_text.delta" for e in events)


def test_record_and_replay(multi_api_client):
    import asyncio

    from modular_b200.serve.recordreplay import read_jsonl, replay_recording

    c = multi_api_client
    c.post("/v1/completions", json={"model": "echo", "prompt": "recorded", "max_tokens": 16},
           headers={"authorization": "Bearer secret"})
    c.post("/v1/completions", json={"model": "missing", "prompt": "x"})
    recs = list(read_jsonl(str(c.recording)))
    mine = [r for r in recs if "recorded" in r["body"]]
    assert mine and mine[-1]["status"] == 200 and "recorded" in mine[-1]["response"]
    assert all("authorization" not in r["headers"] for r in recs)
    assert any(r["status"] == 404 for r in recs)

    class Adapter:      # the app lives on the TestClient's event loop: drive it through the sync client
        async def request(self, method, url, content=None, headers=None):
            return await asyncio.to_thread(c.request, method, url.replace("http://test", ""), content=content,
                                           headers=headers)

    res = asyncio.run(replay_recording(str(c.recording), "http://test", concurrency=4, client=Adapter()))
    assert res.sent == len(recs) and res.status_match == res.sent, res.failures


def test_data_parallel_replicas_share_the_load():
    pc = _config(model_path="echo", devices="cpu", data_parallel_degree=2)
    app = fastapi_app(Settings(), pc, ByteTokenizer(), EchoPipeline, "echo", 4096)
    with TestClient(app) as c:
        for i in range(6):
            r = c.post("/v1/completions", json={"model": "echo", "prompt": f"req {i}", "max_tokens": 16})
            assert r.status_code == 200 and r.json()["choices"][0]["text"] == f"req {i}"
        stats = c.get("/max_internal/worker_stats").json()["replicas"]
        assert len(stats) == 2 and all(s["steps"] > 0 for s in stats)
        assert c.app.state.proxy.assigned == [3, 3]
        assert c.post("/reset_prefix_cache").json() == {"success": False}


def test_step_token_alignment_trims_overshoot():
    """A prompt chunk that would push a step slightly past a multiple of the alignment is cut to land on it."""
    import numpy as np
    from modular_b200.pipelines.context import SamplingParams, TextContext
    from modular_b200.serve.scheduler.token_budget import ActiveTokenBudget, BudgetStatus

    def ctx(n):
        return TextContext.from_prompt(np.arange(n, dtype=np.int64) % 100, 8192, f"r{n}", SamplingParams(), ())

    b = ActiveTokenBudget(2176, True, 16, align=1024)
    b.used = 64                                   # decode tokens already in the step
    c = ctx(1024)
    assert b.status_after_context(c) is BudgetStatus.BUDGET_REACHED
    assert c.tokens.active_length == 960 and b.used == 1024
    # far from a boundary: untouched
    b2 = ActiveTokenBudget(2176, True, 16, align=1024)
    b2.used = 64
    c2 = ctx(500)
    assert b2.status_after_context(c2) is BudgetStatus.BUDGET_AVAILABLE and c2.tokens.active_length == 500
    # large overshoot (more than a quarter of the alignment): untouched
    b3 = ActiveTokenBudget(4096, True, 16, align=1024)
    b3.used = 64
    c3 = ctx(1400)
    assert b3.status_after_context(c3) is BudgetStatus.BUDGET_AVAILABLE and c3.tokens.active_length == 1400
    # alignment off
    b4 = ActiveTokenBudget(2176, True, 16)
    b4.used = 64
    c4 = ctx(1024)
    assert b4.status_after_context(c4) is BudgetStatus.BUDGET_AVAILABLE and c4.tokens.active_length == 1024


# ---------------------------------------------------------------------------- tool calls, reasoning, n > 1, LoRA admin
def test_tool_and_reasoning_parsers():
    from modular_b200.serve.parser import (ReasoningSplitter, get_tool_parser, parse_json_objects, split_reasoning)

    assert parse_json_objects('x {"a": "}{"} y {"b": {"c": 1}} {bad') == [{"a": "}{"}, {"b": {"c": 1}}]
    p = get_tool_parser("llama")
    r = p.parse_complete('<|python_tag|>{"name": "get_weather", "parameters": {"city": "Paris"}}; '
                         '{"name": "f", "parameters": {}}')
    assert [c.name for c in r.tool_calls] == ["get_weather", "f"] and r.content is None
    assert json.loads(r.tool_calls[0].arguments) == {"city": "Paris"} and r.tool_calls[0].id.startswith("call_")
    assert p.parse_complete("plain answer").tool_calls == []
    with pytest.raises(ValueError):
        p.parse_complete('{"name": "no_parameters"}')
    # streaming: nothing leaks while the JSON is open, the call comes out when it closes, plain text passes through
    p.reset()
    outs = [p.parse_delta(c) for c in ['{"name": "g', 'et", "param', 'eters": {"a": 1}}']] + [p.parse_delta("", True)]
    assert all(t == "" for t, _ in outs) and sum(len(c) for _, c in outs) == 1 and outs[2][1][0].name == "get"
    p.reset()
    assert [p.parse_delta(c)[0] for c in ["Hel", "lo {", "}"]] == ["Hel", "lo {", "}"]
    h = get_tool_parser("hermes")
    r = h.parse_complete('ok <tool_call>{"name": "a", "arguments": {"x": 1}}</tool_call> done')
    assert r.content == "ok  done" and r.tool_calls[0].to_openai()["function"] == {"name": "a", "arguments": '{"x": 1}'}
    with pytest.raises(ValueError):
        get_tool_parser("nope")
    assert split_reasoning("<think>abc</think>\nanswer") == ("abc", "answer")
    assert split_reasoning("no tags") == (None, "no tags")
    s = ReasoningSplitter()
    parts = [s.push(c) for c in ["<th", "ink>rea", "son</th", "ink>\nvis", "ible"]] + [s.push("", True)]
    assert "".join(a for a, _ in parts) == "reason" and "".join(b for _, b in parts) == "visible"


def test_chat_tool_calls_and_n(echo_client):
    echo_client.app.state.tool_parser = "hermes"
    tools = [{"type": "function", "function": {"name": "lookup", "parameters": {"type": "object"}}}]
    call = '<tool_call>{"name": "lookup", "arguments": {"q": "x"}}</tool_call>'
    body = {"model": "echo", "max_tokens": 400, "tools": tools, "messages": [{"role": "user", "content": call}]}
    r = echo_client.post("/v1/chat/completions", json=body).json()
    ch = r["choices"][0]
    assert ch["finish_reason"] == "tool_calls" and ch["message"]["tool_calls"][0]["function"]["name"] == "lookup"
    assert json.loads(ch["message"]["tool_calls"][0]["function"]["arguments"]) == {"q": "x"}
    # without tools in the request the same text stays content
    plain = echo_client.post("/v1/chat/completions", json={k: v for k, v in body.items() if k != "tools"}).json()
    assert plain["choices"][0]["message"].get("tool_calls") is None and "<tool_call>" in plain["choices"][0]["message"]["content"]
    # streaming: the call arrives as a tool_calls delta, the stream ends with finish_reason tool_calls
    calls, reasons, text = [], [], ""
    with echo_client.stream("POST", "/v1/chat/completions", json=dict(body, stream=True)) as resp:
        for line in resp.iter_lines():
            if not line.startswith("data: ") or line == "data: [DONE]":
                continue
            for c in json.loads(line[6:])["choices"]:
                calls += c["delta"].get("tool_calls") or []
                text += c["delta"].get("content") or ""
                if c.get("finish_reason"):
                    reasons.append(c["finish_reason"])
    assert len(calls) == 1 and calls[0]["index"] == 0 and calls[0]["function"]["name"] == "lookup"
    assert reasons == ["tool_calls"] and "<tool_call>" not in text
    # n > 1: one choice per sample, usage counts the prompt once
    r = echo_client.post("/v1/completions", json={"model": "echo", "prompt": "abc", "max_tokens": 16, "n": 3}).json()
    assert [c["index"] for c in r["choices"]] == [0, 1, 2] and all(c["text"] == "abc" for c in r["choices"])
    assert r["usage"]["prompt_tokens"] == 4 and r["usage"]["completion_tokens"] >= 9
    r = echo_client.post("/v1/chat/completions", json={"model": "echo", "n": 2, "max_tokens": 64,
                                                       "messages": [{"role": "user", "content": "hi"}]}).json()
    assert len(r["choices"]) == 2 and r["choices"][0]["message"]["content"] == r["choices"][1]["message"]["content"]
    seen = set()
    with echo_client.stream("POST", "/v1/completions", json={"model": "echo", "prompt": "abcd", "max_tokens": 16,
                                                             "n": 2, "stream": True}) as resp:
        for line in resp.iter_lines():
            if line.startswith("data: {"):
                seen |= {c["index"] for c in json.loads(line[6:])["choices"]}
    assert seen == {0, 1}
    assert echo_client.post("/v1/completions", json={"model": "echo", "prompt": "a", "n": 0}).status_code == 400


def test_lora_admin_routes(tmp_path):
    """Load an adapter over HTTP, address it with ``model = <adapter name>``, unload it again."""
    import torch
    from safetensors.torch import save_file

    from modular_b200.models.llama3 import Llama3Config

    cfg = Llama3Config.tiny()
    g = torch.Generator().manual_seed(3)
    sd = {}
    for i in range(cfg.num_hidden_layers):
        sd[f"base_model.model.model.layers.{i}.self_attn.q_proj.lora_A.weight"] = torch.randn(8, cfg.hidden_size, generator=g) * 0.3
        sd[f"base_model.model.model.layers.{i}.self_attn.q_proj.lora_B.weight"] = torch.randn(cfg.q_dim, 8, generator=g) * 0.3
    (tmp_path / "ad").mkdir()
    save_file(sd, str(tmp_path / "ad" / "adapter_model.safetensors"))
    (tmp_path / "ad" / "adapter_config.json").write_text(json.dumps({"r": 8, "lora_alpha": 64}))
    pc = _config(model_path="preset:tiny-llama", devices="cpu", max_length=256, max_batch_size=4,
                 max_batch_input_tokens=128, kv_cache_page_size=16)
    tokenizer, factory = PIPELINE_REGISTRY.retrieve_factory(pc)
    app = fastapi_app(Settings(), pc, tokenizer, factory, "tiny", 256)
    # the byte tokenizer renders ids above 255 alike, so outputs are compared through their log-probabilities
    req = {"prompt": [5, 6, 7, 8, 9, 10, 11, 12], "max_tokens": 8, "temperature": 0, "ignore_eos": True, "logprobs": 1}
    lps = lambda r: [round(v, 4) for v in r.json()["choices"][0]["logprobs"]["token_logprobs"]]
    with TestClient(app) as c:
        assert c.post("/v1/completions", json=dict(req, model="ad1")).status_code == 404
        bad = c.post("/v1/load_lora_adapter", json={"lora_name": "ad1", "lora_path": str(tmp_path / "missing")})
        assert bad.status_code == 400
        ok = c.post("/v1/load_lora_adapter", json={"lora_name": "ad1", "lora_path": str(tmp_path / "ad")})
        assert ok.status_code == 200, ok.text
        assert "ad1" in [m["id"] for m in c.get("/v1/models").json()["data"]]
        base = lps(c.post("/v1/completions", json=dict(req, model="tiny")))
        tuned = lps(c.post("/v1/completions", json=dict(req, model="ad1")))
        again = lps(c.post("/v1/completions", json=dict(req, model="tiny")))
        assert tuned != base and again == base          # the adapter changes the output; the base model is untouched
        assert c.post("/v1/unload_lora_adapter", json={"lora_name": "ad1"}).status_code == 200
        assert c.post("/v1/unload_lora_adapter", json={"lora_name": "ad1"}).status_code == 404
        assert c.post("/v1/completions", json=dict(req, model="ad1")).status_code == 404


def test_worker_hop_codec_roundtrip():
    """Requests, step outputs (with log-probabilities), embeddings, cancels and RPC frames survive the msgpack hop."""
    import numpy as np

    from modular_b200.pipelines.context import (EmbeddingsOutput, GenerationStatus, SamplingParams, TextContext,
                                                TextGenerationOutput)
    from modular_b200.serve.worker_interface import codec

    sp = SamplingParams(temperature=0.5, top_k=7, stop=["x"], stop_token_ids=[3], seed=9, logprobs=2,
                        response_format={"type": "json_object"})
    ctx = TextContext.from_prompt(np.arange(5, 40), 128, "r1", sp, eos_token_ids=(2, 9), model_name="m")
    ctx.lora_name, ctx.cache_salt, ctx.task, ctx.pooling = "ad", 12345678901234, "generate", "mean"
    got = codec.decode(codec.encode(ctx))
    assert got.request_id == "r1" and got.tokens.prompt.tolist() == list(range(5, 40)) and got.max_length == 128
    assert got.sampling_params == sp and got.eos_token_ids == frozenset((2, 9)) and got.model_name == "m"
    assert (got.lora_name, got.cache_salt, got.pooling) == ("ad", 12345678901234, "mean")
    outs = {"a": TextGenerationOutput("a", [np.int64(4), 5], GenerationStatus.ACTIVE,
                                      [{"token": 4, "logprob": np.float32(-0.5), "top": [(4, -0.5), (7, -1.5)]}]),
            "b": TextGenerationOutput("b", [], GenerationStatus.MAXIMUM_LENGTH)}
    back = codec.decode(codec.encode(outs))
    assert back["a"].tokens == [4, 5] and back["a"].log_probabilities[0]["top"] == [(4, -0.5), (7, -1.5)]
    assert back["b"].is_done and back["b"].final_status is GenerationStatus.MAXIMUM_LENGTH
    emb = codec.decode(codec.encode({"e": EmbeddingsOutput("e", [0.5, 0.25], 3)}))["e"]
    assert emb.embedding == [0.5, 0.25] and emb.prompt_tokens == 3
    assert codec.decode(codec.encode("rid-7")) == "rid-7"
    assert codec.decode(codec.encode(("stats", None))) == ("stats", None)
    with pytest.raises(Exception):
        codec.decode(b"\\x80\\x04garbage")


def test_tracing_spans_for_requests_and_batches(tmp_path):
    """With telemetry on and a destination configured, a request produces a server span that continues the caller's
    trace, with tokenise / generate children; without a destination nothing is recorded."""
    from opentelemetry.sdk.trace.export.in_memory_span_exporter import InMemorySpanExporter

    from modular_b200.serve.config import Settings
    from modular_b200.serve.telemetry import tracing

    assert tracing.configure_tracing(Settings()) is False and not tracing.tracing_enabled()
    with tracing.span("nothing") as s:
        assert s is None
    exp = InMemorySpanExporter()
    assert tracing.configure_tracing(Settings(disable_telemetry=False, kernel_trace_level=1), exporter=exp)
    assert tracing.batch_spans_enabled()
    parent = "00-0af7651916cd43dd8448eb211c80319c-b7ad6b7169203331-01"
    with tracing.span("POST /v1/completions", {"request.id": "r1"}, traceparent=parent, kind="server") as sp:
        with tracing.span("max.tokenize"):
            pass
        tracing.set_attributes(sp, **{"http.status_code": 200})
        assert tracing.current_traceparent().split("-")[1] == "0af7651916cd43dd8448eb211c80319c"
    spans = {s.name: s for s in exp.get_finished_spans()}
    assert set(spans) == {"POST /v1/completions", "max.tokenize"}
    server = spans["POST /v1/completions"]
    assert f"{server.get_span_context().trace_id:032x}" == "0af7651916cd43dd8448eb211c80319c"
    assert spans["max.tokenize"].parent.span_id == server.get_span_context().span_id
    assert server.attributes["http.status_code"] == 200
    # the file destination writes one JSON object per span
    tracing.shutdown_tracing()
    path = tmp_path / "spans.jsonl"
    os.environ["MAX_SERVE_TRACE_FILE"] = str(path)
    try:
        assert tracing.configure_tracing(Settings(disable_telemetry=False))
        with tracing.span("max.batch", {"batch.size": 3}):
            pass
        tracing.shutdown_tracing()
    finally:
        del os.environ["MAX_SERVE_TRACE_FILE"]
    rec = json.loads(path.read_text().splitlines()[0])
    assert rec["name"] == "max.batch" and rec["attributes"]["batch.size"] == 3


def test_benchmark_client_loads_datasets_and_sweeps(tmp_path):
    """The benchmark client against a real HTTP server (echo model): closed loop, Poisson open loop, a concurrency
    sweep, and the ShareGPT / JSONL dataset readers."""
    import asyncio
    import socket
    import threading
    import time

    import uvicorn

    from modular_b200.benchmark.benchmark_serving import load_dataset, run_benchmark, run_sweep

    share = tmp_path / "share.json"
    share.write_text(json.dumps([
        {"conversations": [{"from": "human", "value": "tell me a story"}, {"from": "gpt", "value": "once upon a time " * 3}]},
        {"conversations": [{"from": "gpt", "value": "no human turn"}]},
        {"conversations": [{"from": "human", "value": "second prompt"}, {"from": "gpt", "value": "short"}]}]))
    reqs = load_dataset("sharegpt", 5, str(share))
    assert len(reqs) == 5 and {r.prompt for r in reqs} == {"tell me a story", "second prompt"}
    assert {r.output_len for r in reqs} == {16, 1}
    jl = tmp_path / "reqs.jsonl"
    jl.write_text('{"prompt": [1, 2, 3], "output_len": 4}\n{"prompt": "text prompt"}\n')
    assert [r.output_len for r in load_dataset("jsonl", 2, str(jl), output_len=7, seed=1)] in ([4, 7], [7, 4])

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    app = fastapi_app(Settings(max_queue_size=64), _config(model_path="echo", devices="cpu"), ByteTokenizer(),
                      EchoPipeline, "echo", 4096)
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    try:
        for _ in range(200):
            if server.started:
                break
            time.sleep(0.05)
        assert server.started
        base = f"http://127.0.0.1:{port}"
        closed = asyncio.run(run_benchmark(base, "echo", 6, 3, 16, 4))
        assert closed["completed"] == 6 and closed["failed"] == 0 and closed["output_token_throughput"] > 0
        opened = asyncio.run(run_benchmark(base, "echo", 5, 0, 16, 4, request_rate=200.0))
        assert opened["completed"] == 5 and opened["config"]["request_rate"] == 200.0
        sweep = asyncio.run(run_sweep(base, "echo", 4, concurrencies=(1, 4), request_rates=(100.0,), input_len=8, output_len=3))
        assert [p["load"] for p in sweep] == [{"max_concurrency": 1}, {"max_concurrency": 4}, {"request_rate": 100.0}]
        assert all(p["completed"] >= 4 for p in sweep)
        chat = asyncio.run(run_benchmark(base, "echo", 2, 2, 8, 3, dataset="jsonl", dataset_path=str(jl), chat=True))
        assert chat["completed"] == 2, chat
    finally:
        server.should_exit = True
        th.join(timeout=10)


def test_gc_pause_monitor_and_heap_freeze():
    import gc

    from modular_b200.serve.telemetry import gc_utils

    seen = []
    mon = gc_utils.install_gc_monitor(True, slow_ms=0.0, top_types=3, observe=seen.append)
    try:
        junk = [[] for _ in range(1000)]
        for a in junk:
            a.append(a)                 # cycles for the collector
        del junk
        gc.collect()
    finally:
        gc_utils.remove_gc_monitor(mon)
    assert mon.collections >= 1 and len(seen) == mon.collections and mon.max_ms >= 0.0 and mon._census
    assert gc_utils.install_gc_monitor(False) is None
    n = gc_utils.freeze_startup_heap()
    try:
        assert n > 0 and gc.get_freeze_count() > 0
    finally:
        gc.unfreeze()
    assert gc_utils.trim_host_heap() in (True, False)


def test_request_profiling_is_opt_in(tmp_path):
    settings = Settings(metric_recording="NOOP", profiling_enabled=True, profile_dir=str(tmp_path))
    pc = _config(model_path="echo", devices="cpu")
    app = fastapi_app(settings, pc, ByteTokenizer(), EchoPipeline, "echo", 4096)
    with TestClient(app) as c:
        body = {"model": "echo", "prompt": "hello", "max_tokens": 4}
        plain = c.post("/v1/completions", json=body)
        assert plain.status_code == 200 and "x-profile-file" not in plain.headers and not list(tmp_path.iterdir())
        prof = c.post("/v1/completions?profile=1", json=body, headers={"x-request-id": "abc"})
        assert prof.status_code == 200 and prof.json()["choices"][0]["text"] == plain.json()["choices"][0]["text"]
        path = tmp_path / "profile.abc.txt"
        assert prof.headers["x-profile-file"] == str(path) and "cumulative" in path.read_text()
        c.post("/v1/completions?profile=1&profile_format=pstats", json=body, headers={"x-request-id": "bin"})
        assert (tmp_path / "profile.bin.pstats").stat().st_size > 0
    off = fastapi_app(Settings(metric_recording="NOOP"), pc, ByteTokenizer(), EchoPipeline, "echo", 4096)
    with TestClient(off) as c:
        r = c.post("/v1/completions?profile=1", json={"model": "echo", "prompt": "hi", "max_tokens": 2})
        assert r.status_code == 200 and "x-profile-file" not in r.headers


def test_uncompilable_grammar_fails_the_request_not_the_server():
    pytest.importorskip("xgrammar")
    pc = _config(model_path="preset:tiny-llama", devices="cpu", max_length=256, max_batch_size=4,
                 max_batch_input_tokens=128, kv_cache_page_size=16, enable_structured_output=True)
    tokenizer, factory = PIPELINE_REGISTRY.retrieve_factory(pc)
    app = fastapi_app(Settings(), pc, tokenizer, factory, "tiny", 256)
    bad_schema = {"type": "object", "properties": {"a": {"$ref": "#/nope"}}}
    with TestClient(app) as c:
        msgs = [{"role": "user", "content": "hi"}]
        bad = c.post("/v1/chat/completions", json={"model": "tiny", "messages": msgs, "max_tokens": 8, "response_format": {
            "type": "json_schema", "json_schema": {"name": "x", "schema": bad_schema}}})
        assert bad.status_code == 400 and "cannot be compiled" in bad.json()["error"]["message"]
        good = c.post("/v1/chat/completions", json={"model": "tiny", "messages": msgs, "max_tokens": 24, "temperature": 0,
                                                    "response_format": {"type": "json_schema", "json_schema": {
                                                        "name": "y", "schema": {"properties": {"ok": {"type": "boolean"}},
                                                                                "required": ["ok"]}}}})
        assert good.status_code == 200
        plain = c.post("/v1/chat/completions", json={"model": "tiny", "messages": msgs, "max_tokens": 4, "temperature": 0})
        assert plain.status_code == 200 and plain.json()["usage"]["completion_tokens"] == 4


def test_a_failing_step_fails_its_requests_and_the_worker_goes_on():
    """An exception inside a scheduler step answers the requests in flight with an error; later requests are served."""
    import torch

    from modular_b200.entrypoints.llm import LLM
    from modular_b200.models.llama3 import Llama3Config
    from modular_b200.pipelines.context import GenerationStatus, SamplingParams, TextContext

    cfg = Llama3Config.tiny(num_hidden_layers=1, vocab_size=64)
    llm = LLM(cfg, device="cpu", dtype=torch.float32, max_length=64, max_batch_size=4, max_batch_input_tokens=32,
              page_size=16, num_kv_pages=16)
    sched = llm.scheduler
    sp = SamplingParams(temperature=0.0, max_new_tokens=3, ignore_eos=True)
    real = llm.pipeline.execute
    calls = {"n": 0}

    def flaky(batch):
        calls["n"] += 1
        if calls["n"] == 2:
            raise RuntimeError("boom")
        return real(batch)

    llm.pipeline.execute = flaky
    sched.add_request(TextContext.from_prompt([1, 2, 3], 32, "a", sp))
    sched.run_iteration()
    with pytest.raises(RuntimeError):
        sched.run_iteration()
    assert sched.recover("internal error: RuntimeError") is True
    outs = {}
    while True:
        try:
            outs.update(sched.response_queue.get_nowait())
        except Exception:      # noqa: BLE001
            break
    assert outs["a"].final_status is GenerationStatus.ERROR and "internal error" in outs["a"].error
    assert not sched.has_work() and llm.kv.pool.used_blocks == 0
    rec = llm.generate([[4, 5, 6]], sp)[0]
    assert len(rec.tokens) == 3


def test_requests_get_503_when_the_model_worker_dies():
    """Waiting requests and later ones are answered with an error when the worker process is gone."""
    import asyncio

    from modular_b200.pipelines.context import SamplingParams, TextContext
    from modular_b200.serve.worker_interface.interface import ModelWorkerProxy, WorkerGone, WorkerQueues
    import queue

    async def run():
        q = WorkerQueues(queue.SimpleQueue(), queue.SimpleQueue(), queue.SimpleQueue())
        proxy = ModelWorkerProxy(q)
        proxy.start()
        ctx = TextContext.from_prompt([1, 2, 3], 16, "r1", SamplingParams(max_new_tokens=4))
        got = []

        async def consume():
            async for out in proxy.stream(ctx):
                got.append(out)

        task = asyncio.create_task(consume())
        await asyncio.sleep(0.05)                   # the request is waiting: nobody answers
        assert proxy.pending == 1 and not task.done()
        proxy.abort_all("the model worker is gone: exit code 1")
        await asyncio.wait_for(task, 2.0)
        assert got and got[-1].is_done and "gone" in got[-1].error
        with pytest.raises(WorkerGone):
            async for _ in proxy.stream(TextContext.from_prompt([1], 16, "r2", SamplingParams(max_new_tokens=1))):
                pass
        await proxy.stop()
        # replicas: a dead one stops receiving requests; the router is dead once all are
        from modular_b200.serve.worker_interface.interface import ReplicaRouter

        a = ModelWorkerProxy(WorkerQueues(queue.SimpleQueue(), queue.SimpleQueue(), queue.SimpleQueue()))
        b = ModelWorkerProxy(WorkerQueues(queue.SimpleQueue(), queue.SimpleQueue(), queue.SimpleQueue()))
        router = ReplicaRouter([a, b])
        a.abort_all("gone")
        assert router.dead is None and all(router.pick() == 1 for _ in range(4))
        b.abort_all("gone too")
        assert router.dead == "gone"

    asyncio.run(run())


def test_odd_requests_get_an_answer_and_leave_the_worker_alone():
    """Ids outside the vocabulary, a negative token budget and an enormous seed are answered (400 or a normal
    completion); none of them reaches the worker as something it cannot pack."""
    pc = _config(model_path="preset:tiny-llama", devices="cpu", max_length=64, max_batch_size=4,
                 max_batch_input_tokens=32, kv_cache_page_size=16)
    tokenizer, factory = PIPELINE_REGISTRY.retrieve_factory(pc)
    app = fastapi_app(Settings(), pc, tokenizer, factory, "tiny", 64)
    with TestClient(app) as c:
        post = lambda **kw: c.post("/v1/completions", json=dict(kw, model="tiny"))
        assert post(prompt=[5, 99999999], max_tokens=2).status_code == 400
        assert post(prompt=[5, -4], max_tokens=2).status_code == 400
        assert post(prompt=[5, 6], max_tokens=-3).status_code == 400
        big = post(prompt=[5, 6], max_tokens=2, seed=2 ** 62, temperature=1.0)
        assert big.status_code == 200 and big.json()["usage"]["completion_tokens"] == 2
        # an image part must not silently drop out of the prompt: the server takes text
        img = c.post("/v1/chat/completions", json={"model": "tiny", "max_tokens": 2, "messages": [{"role": "user", "content": [
            {"type": "text", "text": "what is this?"}, {"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}}]}]})
        assert img.status_code == 400 and "image_url" in img.json()["error"]["message"]
        txt = c.post("/v1/chat/completions", json={"model": "tiny", "max_tokens": 2, "messages": [{"role": "user", "content": [
            {"type": "text", "text": "hello"}]}]})
        assert txt.status_code == 200
        assert c.get("/health/ready").status_code == 200
