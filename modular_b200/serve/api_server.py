"""FastAPI application and its lifespan.

``fastapi_app(settings, pipeline_config, tokenizer, factory)`` builds the app; its lifespan
starts the model worker process (``subprocess_manager``), wires the ZMQ queues into a
``ModelWorkerProxy`` and a ``TokenGeneratorPipeline`` and tears everything down on exit. A
worker that dies takes the server down with it (the watcher task is awaited next to uvicorn).
Reference: max/python/max/serve/api_server.py:110 (lifespan), :330 (``fastapi_app``), :389
(``/reset_prefix_cache``), :307 (``RequestQueueFull`` -> 429).
"""

from __future__ import annotations

import asyncio
import contextlib
import logging
import queue
import time
import uuid
from typing import Callable, Optional

from fastapi import FastAPI, Request
from fastapi.exceptions import RequestValidationError
from fastapi.responses import JSONResponse, Response
from starlette.exceptions import HTTPException as StarletteHTTPException

from .. import __version__
from .config import Settings
from .model_worker import model_worker_main
from .pipelines.llm import TokenGeneratorPipeline
from .process_control import SubprocessExit, subprocess_manager
from .router import extra_routes, openai_routes
from .router.openai_routes import error_response
from .telemetry.metrics import METRICS, configure_metrics, record_batch_metrics
from .worker_interface import ModelWorkerProxy, ReplicaRouter, RequestQueueFull, WorkerQueues, ZmqQueueSpec

logger = logging.getLogger("modular_b200.serve")


class _Rpc:
    """API-side end of the worker side channel."""

    def __init__(self, req: ZmqQueueSpec, resp: ZmqQueueSpec):
        self.req = req.push(bind=False)
        self.resp = resp.pull(bind=True)
        self.lock = asyncio.Lock()

    async def call(self, name: str, arg=None, timeout_s: float = 10.0):
        async with self.lock:
            self.req.put_nowait((name, arg))
            t0 = time.monotonic()
            while time.monotonic() - t0 < timeout_s:
                try:
                    got, ok, val = self.resp.get_nowait()
                except queue.Empty:
                    await asyncio.sleep(0.005)
                    continue
                if got == name:
                    if not ok:
                        raise RuntimeError(val)
                    return val
            raise TimeoutError(f"worker RPC {name} timed out")


def _replica_config(pipeline_config, replica: int, n_replicas: int):
    """The pipeline config of one data-parallel replica: its share of the configured devices."""
    if n_replicas <= 1 or pipeline_config is None:
        return pipeline_config
    import copy
    pc = copy.deepcopy(pipeline_config)
    m = pc.model
    if m.uses_gpu:
        ids = m.device_ids
        per = max(1, len(ids) // n_replicas)
        mine = ids[replica * per:(replica + 1) * per] or [ids[replica % len(ids)]]
        m.devices = "gpu:" + ",".join(str(i) for i in mine)
    m.data_parallel_degree = 1
    return pc


class _MultiRpc:
    """Side-channel calls fan out to every replica; results come back as a list (one replica: the value)."""

    def __init__(self, rpcs):
        self.rpcs = rpcs

    async def call(self, name: str, arg=None, timeout_s: float = 10.0):
        vals = [await r.call(name, arg, timeout_s) for r in self.rpcs]
        if len(vals) == 1:
            return vals[0]
        if name == "reset_prefix_cache":
            return all(vals)
        return {"replicas": vals}


def make_lifespan(settings: Settings, pipeline_config, tokenizer, factory: Callable, model_name: str,
                  max_length: int, factories: Optional[list] = None):
    """``factories``: one pipeline factory per data-parallel replica (default: ``factory`` for each of
    ``pipeline_config.model.data_parallel_degree`` replicas)."""
    n_rep = len(factories) if factories else max(1, getattr(getattr(pipeline_config, "model", None),
                                                            "data_parallel_degree", 1) or 1)
    factories = factories or [factory] * n_rep

    @contextlib.asynccontextmanager
    async def lifespan(app: FastAPI):
        t_start = time.monotonic()
        async with contextlib.AsyncExitStack() as stack:
            proxies, rpcs, watchers, metric_pulls = [], [], [], []
            for i in range(n_rep):
                specs = {k: ZmqQueueSpec.create(f"{k}{i}")
                         for k in ("request", "response", "cancel", "rpc_req", "rpc_resp", "metrics")}
                response_pull = specs["response"].pull(bind=True)
                metric_pulls.append(specs["metrics"].pull(bind=True))
                _pm, watcher = await stack.enter_async_context(subprocess_manager(
                    f"model-worker-{i}", model_worker_main,
                    (factories[i], _replica_config(pipeline_config, i, n_rep), specs, settings),
                    ready_timeout_s=settings.mw_timeout_s, use_heartbeat=settings.use_heartbeat,
                    health_fail_s=settings.mw_health_fail_s,
                    # a tensor-parallel worker starts the other ranks itself
                    daemon=max(getattr(pipeline_config, "tensor_parallel_degree", 1) or 1,
                               getattr(pipeline_config, "expert_parallel_degree", 1) or 1) <= 1))
                queues = WorkerQueues(request=specs["request"].push(bind=False), response=response_pull,
                                      cancel=specs["cancel"].push(bind=False))
                proxies.append(ModelWorkerProxy(queues, settings.max_queue_size))
                rpcs.append(_Rpc(specs["rpc_req"], specs["rpc_resp"]))
                watchers.append(watcher)
            proxy = proxies[0] if n_rep == 1 else ReplicaRouter(proxies)
            proxy.start()
            app.state.pipeline = TokenGeneratorPipeline(model_name, tokenizer, proxy, max_length,
                                                        settings.stream_min_chunk_tokens)
            app.state.rpc = _MultiRpc(rpcs)
            async def first_failure():
                done, _ = await asyncio.wait(watchers, return_when=asyncio.FIRST_COMPLETED)
                for t in done:
                    t.result()          # re-raises SubprocessExit of the replica that died

            # a replica that dies answers what waits on it with an error (503) instead of leaving it hanging
            def _on_exit(task, p):
                if not task.cancelled() and task.exception() is not None:
                    p.abort_all(f"the model worker is gone: {task.exception()}")

            for w, p in zip(watchers, proxies):
                w.add_done_callback(lambda t, p=p: _on_exit(t, p))
            app.state.worker_watcher = watchers[0] if n_rep == 1 else asyncio.ensure_future(first_failure())
            app.state.proxy = proxy
            METRICS.pipeline_load.inc(n_rep)
            METRICS.model_load_time_ms.set((time.monotonic() - t_start) * 1e3)

            async def consume_worker_metrics():
                """Replays the workers' per-step metrics into this process's instruments."""
                while True:
                    idle = True
                    for q_ in metric_pulls:
                        for _ in range(256):
                            try:
                                record_batch_metrics(q_.get_nowait())
                                idle = False
                            except queue.Empty:
                                break
                    METRICS.queue_depth.set(getattr(proxy, "pending", 0) or 0)
                    await asyncio.sleep(0.05 if idle else 0.0)

            metrics_task = asyncio.ensure_future(consume_worker_metrics())
            logger.info("server ready: model %s on %d replica(s)", model_name, n_rep)
            try:
                yield
            finally:
                metrics_task.cancel()
                await proxy.stop()
                app.state.pipeline = None
    return lifespan


def fastapi_app(settings: Settings, pipeline_config=None, tokenizer=None, factory: Optional[Callable] = None,
                model_name: str = "model", max_length: int = 4096, lifespan=None) -> FastAPI:
    configure_metrics(settings.metric_recording.value)
    if lifespan is None:
        lifespan = make_lifespan(settings, pipeline_config, tokenizer, factory, model_name, max_length)
    app = FastAPI(title="modular_b200 serve", version=__version__, lifespan=lifespan)
    app.state.pipeline = None
    app.state.model_names = {model_name}
    app.state.structured_output = bool(pipeline_config and pipeline_config.sampling.enable_structured_output)
    app.state.lora_names = set()
    rt = getattr(pipeline_config, "runtime", None)
    app.state.tool_parser = getattr(rt, "tool_parser", None)
    app.state.reasoning_parser = getattr(rt, "reasoning_parser", None)
    app.state.settings = settings

    from .telemetry import tracing

    tracing.configure_tracing(settings)

    from .debug import register_debug

    register_debug(app, settings.profiling_enabled, settings.profile_dir)     # inside the request-id middleware

    @app.middleware("http")
    async def request_id_middleware(request: Request, call_next):
        rid = request.headers.get("x-request-id") or uuid.uuid4().hex
        request.state.request_id = rid
        if not tracing.tracing_enabled():
            resp = await call_next(request)
            resp.headers["x-request-id"] = rid
            return resp
        # one server span per request, continuing the caller's trace when it sent a W3C traceparent
        with tracing.span(f"{request.method} {request.url.path}", {"http.method": request.method,
                          "http.target": request.url.path, "request.id": rid},
                          traceparent=request.headers.get("traceparent"), kind="server") as sp:
            resp = await call_next(request)
            tracing.set_attributes(sp, **{"http.status_code": resp.status_code})
            tp = tracing.current_traceparent()
            if tp:
                resp.headers["traceparent"] = tp
        resp.headers["x-request-id"] = rid
        return resp

    @app.exception_handler(RequestQueueFull)
    async def _queue_full(_r: Request, exc: RequestQueueFull):
        return error_response(429, str(exc), "rate_limit_error")

    @app.exception_handler(StarletteHTTPException)
    async def _http_exc(_r: Request, exc: StarletteHTTPException):
        kind = {404: "not_found_error", 429: "rate_limit_error", 503: "service_unavailable"}.get(exc.status_code, "invalid_request_error")
        return error_response(exc.status_code, str(exc.detail), kind)

    @app.exception_handler(RequestValidationError)
    async def _validation(_r: Request, exc: RequestValidationError):
        first = exc.errors()[0] if exc.errors() else {}
        loc = ".".join(str(x) for x in first.get("loc", []) if x != "body")
        return error_response(400, f"{loc}: {first.get('msg', 'invalid request')}" if loc else str(exc))

    @app.exception_handler(Exception)
    async def _unhandled(_r: Request, exc: Exception):
        METRICS.request_errors.inc()
        logger.exception("unhandled error")
        return error_response(500, f"{type(exc).__name__}: {exc}", "server_error")

    def _readiness():
        """200 while a model worker can take requests; 503 while it starts and after it has exited."""
        if app.state.pipeline is None:
            return JSONResponse(status_code=503, content={"status": "starting"})
        proxy = getattr(app.state, "proxy", None)
        gone = getattr(proxy, "dead", None) if proxy is not None else None      # a router: once all replicas are gone
        if gone:
            return JSONResponse(status_code=503, content={"status": "unavailable", "reason": gone})
        return {"status": "ok"}

    @app.get("/health")
    async def health():
        return _readiness()

    @app.get("/health/ready")
    async def health_ready():
        return _readiness()

    @app.get("/health/live")
    async def health_live():
        return {"status": "ok"}      # the API process answers

    @app.get("/version")
    async def version():
        return {"version": __version__}

    @app.get("/metrics")
    async def metrics():
        return Response(METRICS.render(), media_type="text/plain; version=0.0.4")

    @app.post("/reset_prefix_cache")
    async def reset_prefix_cache():
        ok = await app.state.rpc.call("reset_prefix_cache")
        return {"success": bool(ok)}

    @app.get("/max_internal/worker_stats")
    async def worker_stats():
        return await app.state.rpc.call("stats")

    @app.get("/max_internal/eplb_stats")
    async def eplb_stats(slots_per_rank: Optional[int] = None):
        """Expert load over all ranks of an expert-parallel engine and the balancer's plan for the worst layer."""
        try:
            return await app.state.rpc.call("eplb_stats", {"slots_per_rank": slots_per_rank})
        except Exception as e:  # noqa: BLE001
            return error_response(409, str(e), "invalid_request_error")

    api_types = {getattr(t, "value", t) for t in settings.api_types}
    if "openai" in api_types:
        app.include_router(openai_routes.router)
        app.include_router(extra_routes.responses_router)
    if "kserve" in api_types:
        app.include_router(extra_routes.kserve_router)
    if "sagemaker" in api_types:
        if "openai" not in api_types:      # /invocations dispatches to the OpenAI handlers
            app.include_router(openai_routes.router)
        app.include_router(extra_routes.sagemaker_router)
    if settings.transaction_recording_file:
        from .recordreplay import RecordingMiddleware
        app.add_middleware(RecordingMiddleware, path=settings.transaction_recording_file,
                           include_responses=settings.transaction_recording_include_responses)
    return app


async def serve_until_done(app: FastAPI, settings: Settings) -> None:
    """Run uvicorn; if the worker watcher fails first, stop the server and re-raise."""
    import uvicorn

    config = uvicorn.Config(app, host=settings.host, port=settings.port, log_level=settings.log_level.lower(),
                            lifespan="on")
    server = uvicorn.Server(config)
    serve_task = asyncio.create_task(server.serve())

    async def watch():
        while getattr(app.state, "worker_watcher", None) is None and not serve_task.done():
            await asyncio.sleep(0.1)
        w = getattr(app.state, "worker_watcher", None)
        if w is not None:
            try:
                await w
            except asyncio.CancelledError:
                return
            except SubprocessExit:
                server.should_exit = True
                raise

    watch_task = asyncio.create_task(watch())
    done, _ = await asyncio.wait({serve_task, watch_task}, return_when=asyncio.FIRST_COMPLETED)
    server.should_exit = True
    await serve_task
    watch_task.cancel()
    for t in done:
        if t is watch_task and t.exception() is not None:
            raise t.exception()
