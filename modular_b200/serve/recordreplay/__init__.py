"""Record HTTP transactions to JSONL and replay them against a server.

Reference: max/python/max/serve/recordreplay/middleware.py, replay.py, jsonl.py and the CLI
``_entrypoints/replay_recording.py``; enabled by ``Settings.transaction_recording_file``.
"""

from .middleware import RecordingMiddleware, read_jsonl
from .replay import replay_recording

__all__ = ["RecordingMiddleware", "read_jsonl", "replay_recording"]
