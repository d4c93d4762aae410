"""Serving benchmark client over HTTP.

Load shapes: closed loop at a fixed concurrency, open loop at a request rate (Poisson arrivals, optionally
capped by a concurrency), and sweeps over either. Datasets: ``random`` (uniform token ids of fixed lengths),
``sharegpt`` (a ShareGPT-format JSON file: first human turn as the prompt, the length of the first answer as the
output length) and ``jsonl`` (one ``{"prompt": text or ids, "output_len": n}`` per line).

Metric definitions follow the reference's client (max/python/max/benchmark/
benchmark_serving.py, benchmark_shared/metrics.py, benchmark_shared/datasets/): TTFT = time to the first
streamed chunk, TPOT = (latency - TTFT) / (output tokens - 1), ITL = gaps between chunks, request throughput
and output-token throughput over the wall time of the run.
"""

from __future__ import annotations

import asyncio
import json
import statistics
import time
from dataclasses import dataclass, field
from typing import Optional

import numpy as np


@dataclass
class RequestResult:
    ok: bool = False
    ttft: float = 0.0
    latency: float = 0.0
    itl: list = field(default_factory=list)
    output_tokens: int = 0
    prompt_tokens: int = 0
    error: Optional[str] = None


def percentile(xs, q):
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q / 100.0 * len(xs)))]


@dataclass
class SampleRequest:
    prompt: object          # token ids or text
    output_len: int


def load_dataset(name: str, num_prompts: int, path: Optional[str] = None, input_len: int = 128, output_len: int = 32,
                 vocab_size: int = 256, seed: int = 0, max_output_len: int = 4096) -> list:
    """``num_prompts`` requests of the named dataset (files are cycled when they hold fewer)."""
    rng = np.random.default_rng(seed)
    if name == "random":
        return [SampleRequest(rng.integers(0, vocab_size, size=input_len).tolist(), output_len) for _ in range(num_prompts)]
    if not path:
        raise ValueError(f"dataset {name!r} needs a file")
    items = []
    if name == "sharegpt":
        with open(path) as f:
            for conv in json.load(f):
                turns = conv.get("conversations") or conv.get("items") or []
                human = next((t for t in turns if t.get("from") in ("human", "user")), None)
                answer = next((t for t in turns if t.get("from") in ("gpt", "assistant", "chatgpt")), None)
                if human is None or not human.get("value"):
                    continue
                # answer length in whitespace words x 4/3 as a token estimate (no tokenizer on the client side)
                n_out = int(len(answer["value"].split()) * 4 / 3) if answer and answer.get("value") else output_len
                items.append(SampleRequest(human["value"], max(1, min(n_out, max_output_len))))
    elif name == "jsonl":
        with open(path) as f:
            for line in f:
                if line.strip():
                    o = json.loads(line)
                    items.append(SampleRequest(o["prompt"], int(o.get("output_len", output_len))))
    else:
        raise ValueError(f"unknown dataset {name!r} (random | sharegpt | jsonl)")
    if not items:
        raise ValueError(f"{path} holds no usable request")
    order = rng.permutation(len(items))
    return [items[order[i % len(items)]] for i in range(num_prompts)]


async def _one(session, url, model, prompt_ids, output_len, chat: bool = False) -> RequestResult:
    body = {"model": model, "max_tokens": output_len, "temperature": 0.0,
            "ignore_eos": True, "stream": True, "stream_options": {"include_usage": True}}
    if chat:
        body["messages"] = [{"role": "user", "content": prompt_ids if isinstance(prompt_ids, str) else
                             " ".join(map(str, prompt_ids))}]
    else:
        body["prompt"] = prompt_ids
    r = RequestResult(prompt_tokens=len(prompt_ids) if not isinstance(prompt_ids, str) else 0)
    t0 = time.perf_counter()
    last = t0
    try:
        async with session.post(url, json=body) as resp:
            if resp.status != 200:
                r.error = f"HTTP {resp.status}: {(await resp.text())[:200]}"
                return r
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data:"):
                    continue
                data = line[5:].strip()
                if data == "[DONE]":
                    break
                obj = json.loads(data)
                now = time.perf_counter()
                if obj.get("usage"):
                    r.output_tokens = obj["usage"]["completion_tokens"]
                    r.prompt_tokens = obj["usage"].get("prompt_tokens", r.prompt_tokens)
                if obj.get("choices"):
                    if r.ttft == 0.0:
                        r.ttft = now - t0
                    else:
                        r.itl.append(now - last)
                    last = now
        r.latency = last - t0
        r.ok = True
    except Exception as e:  # noqa: BLE001
        r.error = repr(e)
    return r


async def run_benchmark(base_url: str, model: str, num_prompts: int, max_concurrency: int, input_len: int,
                        output_len: int, vocab_size: int = 256, seed: int = 0, request_rate: float = 0.0,
                        dataset: str = "random", dataset_path: Optional[str] = None, chat: bool = False) -> dict:
    """One run. ``request_rate`` > 0: requests arrive as a Poisson process of that rate (requests / s) and
    ``max_concurrency`` (0 = unbounded) only caps how many are in flight; otherwise a closed loop keeps
    ``max_concurrency`` requests in flight."""
    import aiohttp

    reqs = load_dataset(dataset, num_prompts, dataset_path, input_len, output_len, vocab_size, seed)
    sem = asyncio.Semaphore(max_concurrency) if max_concurrency > 0 else None
    url = base_url.rstrip("/") + ("/v1/chat/completions" if chat else "/v1/completions")
    timeout = aiohttp.ClientTimeout(total=6 * 3600)
    gaps = np.random.default_rng(seed + 1).exponential(1.0 / request_rate, size=num_prompts) if request_rate > 0 else None
    async with aiohttp.ClientSession(timeout=timeout) as session:
        async def guarded(q):
            if sem is None:
                return await _one(session, url, model, q.prompt, q.output_len, chat)
            async with sem:
                return await _one(session, url, model, q.prompt, q.output_len, chat)

        t0 = time.perf_counter()
        if gaps is None:
            results = await asyncio.gather(*(guarded(q) for q in reqs))
        else:
            tasks = []
            for q, gap in zip(reqs, gaps):
                tasks.append(asyncio.create_task(guarded(q)))
                await asyncio.sleep(float(gap))
            results = await asyncio.gather(*tasks)
        wall = time.perf_counter() - t0
    ok = [r for r in results if r.ok]
    tpots = [(r.latency - r.ttft) / (r.output_tokens - 1) for r in ok if r.output_tokens > 1]
    itls = [x for r in ok for x in r.itl]
    out_tok = sum(r.output_tokens for r in ok)
    ms = lambda v: None if v is None else round(v * 1e3, 3)
    return {
        "completed": len(ok), "failed": len(results) - len(ok), "duration_s": round(wall, 3),
        "request_throughput": round(len(ok) / wall, 3), "output_token_throughput": round(out_tok / wall, 2),
        "total_token_throughput": round((out_tok + sum(r.prompt_tokens for r in ok)) / wall, 2),
        "mean_ttft_ms": ms(statistics.mean(r.ttft for r in ok)) if ok else None,
        "p50_ttft_ms": ms(percentile([r.ttft for r in ok], 50)), "p99_ttft_ms": ms(percentile([r.ttft for r in ok], 99)),
        "p50_tpot_ms": ms(percentile(tpots, 50)), "p99_tpot_ms": ms(percentile(tpots, 99)),
        "p50_itl_ms": ms(percentile(itls, 50)), "p99_itl_ms": ms(percentile(itls, 99)),
        "errors": [r.error for r in results if r.error][:3],
        "config": {"num_prompts": num_prompts, "max_concurrency": max_concurrency, "input_len": input_len,
                   "output_len": output_len, "request_rate": request_rate, "dataset": dataset, "chat": chat},
    }


async def run_sweep(base_url: str, model: str, num_prompts: int, concurrencies=(), request_rates=(), rate_cap: int = 0,
                    **kw) -> list:
    """The same workload at several concurrencies (closed loop) and / or request rates (open loop): one result per
    point, in order, each tagged with its load."""
    out = []
    for c in concurrencies:
        r = await run_benchmark(base_url, model, max(num_prompts, int(c)), int(c), **kw)
        out.append(dict(r, load={"max_concurrency": int(c)}))
    for rate in request_rates:
        r = await run_benchmark(base_url, model, num_prompts, rate_cap, request_rate=float(rate), **kw)
        out.append(dict(r, load={"request_rate": float(rate)}))
    return out
