"""ASGI middleware that appends one JSON line per HTTP transaction.

Each line: ``{"ts", "method", "path", "query", "headers", "body", "status", "latency_ms"}`` and,
when ``include_responses`` is set, ``"response"`` (the body as text; streamed bodies are joined).
Request bodies are buffered and re-played to the application unchanged, so recording does not
alter behaviour. Secrets do not belong in a recording: the ``authorization`` and ``cookie``
headers are dropped.
"""

from __future__ import annotations

import json
import threading
import time
from typing import Iterator

_DROP_HEADERS = {b"authorization", b"cookie", b"proxy-authorization"}


class RecordingMiddleware:
    def __init__(self, app, path: str, include_responses: bool = False,
                 skip_paths: tuple = ("/health", "/metrics", "/version")):
        self.app, self.path, self.include_responses = app, path, include_responses
        self.skip_paths = skip_paths
        self._lock = threading.Lock()

    def _write(self, rec: dict) -> None:
        line = json.dumps(rec, ensure_ascii=False)
        with self._lock, open(self.path, "a", encoding="utf-8") as f:
            f.write(line + "\n")

    async def __call__(self, scope, receive, send):
        if scope["type"] != "http" or scope["path"] in self.skip_paths:
            await self.app(scope, receive, send)
            return
        t0 = time.time()
        chunks, more = [], True
        while more:
            msg = await receive()
            if msg["type"] == "http.disconnect":
                break
            chunks.append(msg.get("body", b""))
            more = msg.get("more_body", False)
        body = b"".join(chunks)
        sent = False

        async def replay_receive():
            nonlocal sent
            if not sent:
                sent = True
                return {"type": "http.request", "body": body, "more_body": False}
            return await receive()

        status = {"code": 0}
        out = []

        async def capture_send(msg):
            if msg["type"] == "http.response.start":
                status["code"] = msg["status"]
            elif msg["type"] == "http.response.body" and self.include_responses:
                out.append(msg.get("body", b""))
            await send(msg)

        try:
            await self.app(scope, replay_receive, capture_send)
        finally:
            rec = {"ts": t0, "method": scope["method"], "path": scope["path"],
                   "query": scope.get("query_string", b"").decode("latin-1"),
                   "headers": {k.decode("latin-1"): v.decode("latin-1") for k, v in scope.get("headers", [])
                               if k.lower() not in _DROP_HEADERS},
                   "body": body.decode("utf-8", "replace"), "status": status["code"],
                   "latency_ms": round((time.time() - t0) * 1e3, 3)}
            if self.include_responses:
                rec["response"] = b"".join(out).decode("utf-8", "replace")
            self._write(rec)


def read_jsonl(path: str) -> Iterator[dict]:
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                yield json.loads(line)
