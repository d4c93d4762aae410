"""Per-request profiling of the API process.

With ``MAX_SERVE_PROFILING_ENABLED=1`` a request that carries ``?profile=1`` is served under a profiler and
leaves ``profile.<request id>.<ext>`` in the profile directory (``MAX_SERVE_PROFILE_DIR``, default the working
directory): what the event-loop thread did while that request was in flight - tokenisation, queue hops,
detokenisation, streaming. ``profile_format``: ``text`` (sorted cumulative-time table, the default) or ``pstats``
(binary, for ``python -m pstats`` / snakeviz). The profiler is the standard library's; nothing is installed and
requests without the parameter run untouched. One request is profiled at a time: a second ``?profile=1`` that
arrives meanwhile is served unprofiled.

Reference: max/python/max/serve/debug.py (DebugSettings :40, profile_call :109, register_debug :126; the reference
uses pyinstrument and adds html / speedscope renderers).
"""

from __future__ import annotations

import cProfile
import io
import logging
import os
import pstats
import threading

logger = logging.getLogger("modular_b200.serve")
_FORMATS = {"text": "txt", "pstats": "pstats"}


def render_profile(prof: cProfile.Profile, fmt: str, limit: int = 60) -> bytes:
    if fmt == "pstats":
        import marshal

        st = pstats.Stats(prof)
        return marshal.dumps(st.stats)
    out = io.StringIO()
    pstats.Stats(prof, stream=out).sort_stats("cumulative").print_stats(limit)
    return out.getvalue().encode()


def register_debug(app, enabled: bool, out_dir: str = ".") -> None:
    """Adds the profiling middleware to ``app`` when ``enabled``."""
    if not enabled:
        return
    busy = threading.Lock()

    @app.middleware("http")
    async def profile_request(request, call_next):
        params = request.query_params
        if params.get("profile", "") in ("", "0", "false") or not busy.acquire(blocking=False):
            return await call_next(request)
        fmt = params.get("profile_format", "text")
        fmt = fmt if fmt in _FORMATS else "text"
        prof = cProfile.Profile()
        try:
            prof.enable()
            try:
                response = await call_next(request)
            finally:
                prof.disable()
            rid = getattr(request.state, "request_id", None) or response.headers.get("x-request-id") or "request"
            path = os.path.join(out_dir, f"profile.{rid}.{_FORMATS[fmt]}")
            with open(path, "wb") as f:
                f.write(render_profile(prof, fmt))
            logger.info("wrote %s", path)
            response.headers["x-profile-file"] = path
            return response
        finally:
            busy.release()
