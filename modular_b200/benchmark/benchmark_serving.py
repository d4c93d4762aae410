"""Serving benchmark client: random-token requests at fixed concurrency over HTTP.

Metric definitions follow the reference's client (max/python/max/benchmark/
benchmark_serving.py, benchmark_shared/metrics.py): TTFT = time to the first streamed chunk,
TPOT = (latency - TTFT) / (output tokens - 1), ITL = gaps between chunks, request throughput
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


async def _one(session, url, model, prompt_ids, output_len) -> RequestResult:
    body = {"model": model, "prompt": prompt_ids, "max_tokens": output_len, "temperature": 0.0,
            "ignore_eos": True, "stream": True, "stream_options": {"include_usage": True}}
    r = RequestResult(prompt_tokens=len(prompt_ids))
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
                        output_len: int, vocab_size: int = 256, seed: int = 0) -> dict:
    import aiohttp

    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, vocab_size, size=input_len).tolist() for _ in range(num_prompts)]
    sem = asyncio.Semaphore(max_concurrency)
    url = base_url.rstrip("/") + "/v1/completions"
    timeout = aiohttp.ClientTimeout(total=6 * 3600)
    async with aiohttp.ClientSession(timeout=timeout) as session:
        async def guarded(p):
            async with sem:
                return await _one(session, url, model, p, output_len)

        t0 = time.perf_counter()
        results = await asyncio.gather(*(guarded(p) for p in prompts))
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
                   "output_len": output_len},
    }
