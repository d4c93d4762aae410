"""Replay a recording against a server, optionally preserving the recorded arrival times."""

from __future__ import annotations

import asyncio
import time
from dataclasses import dataclass, field
from typing import Optional

from .middleware import read_jsonl


@dataclass
class ReplayResult:
    sent: int = 0
    status_match: int = 0
    failures: list = field(default_factory=list)
    latencies_ms: list = field(default_factory=list)

    def summary(self) -> dict:
        lat = sorted(self.latencies_ms)
        pct = lambda p: lat[min(len(lat) - 1, int(p * len(lat)))] if lat else None
        return {"sent": self.sent, "status_match": self.status_match, "failures": len(self.failures),
                "p50_ms": pct(0.5), "p99_ms": pct(0.99)}


async def replay_recording(path: str, base_url: str, concurrency: int = 8, preserve_timing: bool = False,
                           speedup: float = 1.0, client=None, limit: Optional[int] = None) -> ReplayResult:
    """Send every recorded request to ``base_url``. ``client`` may be any object with an async
    ``request(method, url, content=..., headers=...)`` returning an object with ``status_code``
    (an ``httpx.AsyncClient``; tests pass an in-process ASGI client)."""
    recs = list(read_jsonl(path))[:limit]
    res = ReplayResult()
    own = client is None
    if own:
        import httpx
        client = httpx.AsyncClient(timeout=600.0)
    sem = asyncio.Semaphore(max(1, concurrency))
    t_first = recs[0]["ts"] if recs else 0.0
    t_start = time.time()

    async def one(rec: dict) -> None:
        if preserve_timing:
            delay = (rec["ts"] - t_first) / max(speedup, 1e-6) - (time.time() - t_start)
            if delay > 0:
                await asyncio.sleep(delay)
        async with sem:
            url = base_url.rstrip("/") + rec["path"] + (("?" + rec["query"]) if rec.get("query") else "")
            headers = {k: v for k, v in rec.get("headers", {}).items()
                       if k.lower() in ("content-type", "accept", "x-request-id")}
            t0 = time.time()
            try:
                r = await client.request(rec["method"], url, content=rec.get("body", "").encode(), headers=headers)
                res.latencies_ms.append((time.time() - t0) * 1e3)
                res.sent += 1
                if r.status_code == rec.get("status"):
                    res.status_match += 1
                else:
                    res.failures.append((rec["path"], rec.get("status"), r.status_code))
            except Exception as e:  # noqa: BLE001
                res.sent += 1
                res.failures.append((rec["path"], rec.get("status"), repr(e)))

    try:
        await asyncio.gather(*(one(r) for r in recs))
    finally:
        if own:
            await client.aclose()
    return res
