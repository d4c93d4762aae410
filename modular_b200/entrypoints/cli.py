"""Command line: ``serve``, ``generate``, ``encode``, ``list``, ``warm-cache``, ``benchmark``.

    python -m modular_b200.entrypoints.cli serve --model-path /ckpt/llama --devices gpu:0
    python -m modular_b200.entrypoints.cli generate --model-path preset:tiny-llama --devices cpu --prompt "hi"

Every ``PipelineConfig`` field is a ``--flag`` (built lazily from the pydantic models, so
``--help`` of a sub-command lists them all). Reference: max/python/max/_entrypoints/
pipelines.py:179 (``main``), :304 ``serve``, :415 ``generate``, :546 ``encode``, :574
``warm-cache``, :771 ``list``, :803 ``benchmark``; option generation in cli/config.py.
"""

from __future__ import annotations

import asyncio
import enum
import json
import logging
import os
import signal
import sys
import time
import typing
from typing import Optional

import click

from .. import __version__


def _click_type(annotation):
    origin = typing.get_origin(annotation)
    if origin is typing.Union:
        args = [a for a in typing.get_args(annotation) if a is not type(None)]
        return _click_type(args[0]) if args else str
    if origin in (list, typing.List):
        return None
    if isinstance(annotation, type) and issubclass(annotation, enum.Enum):
        return click.Choice([e.value for e in annotation])
    if annotation in (int, float, str):
        return annotation
    if annotation is bool:
        return bool
    return str


def pipeline_config_options(fn):
    """Attach one option per flat PipelineConfig field."""
    from ..pipelines.config import PipelineArgs

    for name, (_sec, info) in reversed(list(PipelineArgs.flat_fields().items())):
        flag = "--" + name.replace("_", "-")
        t = _click_type(info.annotation)
        kw = dict(default=None, help=(info.description or f"{_sec}.{name}"), show_default=False)
        if t is bool:
            fn = click.option(flag + "/--no-" + name.replace("_", "-"), name, **kw)(fn)
        elif t is None:
            fn = click.option(flag, name, multiple=True, **kw)(fn)
        else:
            fn = click.option(flag, name, type=t, **kw)(fn)
    fn = click.option("--config-file", type=click.Path(exists=True), default=None,
                      help="YAML/JSON file with sections model/kv_cache/runtime/sampling/...")(fn)
    return fn


def _build_config(config_file, flat):
    from ..pipelines.config import PipelineArgs, PipelineConfig

    flat = {k: (list(v) if isinstance(v, tuple) else v) for k, v in flat.items()
            if v is not None and v != ()}
    args = PipelineArgs.from_flat_kwargs(config_file, **flat)
    return PipelineConfig.from_args(args)


@click.group()
@click.version_option(__version__, prog_name="modular_b200")
@click.option("--log-level", default="INFO", type=click.Choice(["DEBUG", "INFO", "WARNING", "ERROR"]))
def main(log_level):
    logging.basicConfig(level=getattr(logging, log_level), format="%(asctime)s %(levelname)s %(name)s: %(message)s")


@main.command("list")
@click.option("--json", "as_json", is_flag=True)
def list_cmd(as_json):
    """List the registered architectures."""
    from ..pipelines.registry import PIPELINE_REGISTRY

    rows = [dict(architecture=a.name, task=a.task, encodings=list(a.supported_encodings),
                 presets=sorted(a.preset_configs), examples=list(a.example_repo_ids))
            for a in PIPELINE_REGISTRY.list_architectures()]
    if as_json:
        click.echo(json.dumps(rows, indent=1))
    else:
        for r in rows:
            click.echo(f"{r['architecture']:28s} {r['task']:18s} encodings={','.join(r['encodings'])} "
                       f"presets={','.join('preset:' + p for p in r['presets'])}")


@main.command()
@pipeline_config_options
@click.option("--prompt", required=True)
@click.option("--max-new-tokens", default=64, type=int)
@click.option("--temperature", default=0.0, type=float)
@click.option("--top-k", default=-1, type=int)
@click.option("--top-p", default=1.0, type=float)
@click.option("--seed", default=0, type=int)
@click.option("--num-warmups", default=0, type=int)
@click.option("--ignore-eos", is_flag=True)
def generate(config_file, prompt, max_new_tokens, temperature, top_k, top_p, seed, num_warmups, ignore_eos,
             **flat):
    """Generate text for one prompt and print it with throughput metrics."""
    from ..pipelines.context import SamplingParams
    from ..pipelines.registry import PIPELINE_REGISTRY

    pc = _build_config(config_file, flat)
    tokenizer, llm = PIPELINE_REGISTRY.retrieve(pc)
    sp = SamplingParams(top_k=top_k if top_k > 0 else -1, top_p=top_p, temperature=temperature,
                        max_new_tokens=max_new_tokens, seed=seed, ignore_eos=ignore_eos)
    ids = tokenizer.encode(prompt)
    for _ in range(num_warmups):
        llm.generate([ids], sp)
    t0 = time.perf_counter()
    rec = llm.generate([ids], sp)[0]
    dt = time.perf_counter() - t0
    click.echo(tokenizer.decode(rec.tokens))
    click.echo(json.dumps({"prompt_tokens": len(ids), "output_tokens": len(rec.tokens),
                           "ttft_ms": round((rec.ttft or 0) * 1e3, 2),
                           "tpot_ms": round((rec.tpot or 0) * 1e3, 3),
                           "tokens_per_s": round(len(rec.tokens) / dt, 1)}), err=True)


@main.command()
@pipeline_config_options
@click.option("--prompt", required=True)
def encode(config_file, prompt, **flat):
    """Tokenise a prompt and print the ids (embedding pipelines are not built yet)."""
    from ..pipelines.registry import PIPELINE_REGISTRY

    pc = _build_config(config_file, flat)
    tokenizer, _ = PIPELINE_REGISTRY.retrieve_factory(pc)
    click.echo(json.dumps(tokenizer.encode(prompt)))


@main.command("warm-cache")
def warm_cache():
    """Compile every CUDA source for sm_100a into the in-tree library."""
    from .._native.build import build

    click.echo(str(build(verbose=False)))


@main.command()
@pipeline_config_options
@click.option("--port", default=None, type=int)
@click.option("--host", default=None)
@click.option("--max-queue-size", default=None, type=int)
@click.option("--headless", is_flag=True, help="run the model worker loop without the HTTP server")
@click.option("--pretty-print-config", is_flag=True)
def serve(config_file, port, host, max_queue_size, headless, pretty_print_config, **flat):
    """Start the OpenAI-compatible server and its model worker."""
    from ..pipelines.registry import PIPELINE_REGISTRY
    from ..serve.api_server import fastapi_app, serve_until_done
    from ..serve.config import Settings

    settings = Settings()
    if port is not None:
        settings.port = port
    if host is not None:
        settings.host = host
    if max_queue_size is not None:
        settings.max_queue_size = max_queue_size
    pc = _build_config(config_file, flat)
    if pretty_print_config:
        click.echo(json.dumps(pc.summary(), indent=1))
    if settings.dummy_model or os.environ.get("MAX_SERVE_DUMMY_MODEL"):
        from ..pipelines.tokenizer import ByteTokenizer
        from ..serve.pipelines.echo_gen import EchoPipeline

        tokenizer, factory, max_length = ByteTokenizer(), EchoPipeline, 1 << 16
        name = pc.model.name or "echo"
    else:
        tokenizer, factory = PIPELINE_REGISTRY.retrieve_factory(pc)
        _arch, cfg, _hf = PIPELINE_REGISTRY.resolve_model(pc)
        max_length = min(pc.model.max_length or cfg.max_position_embeddings, cfg.max_position_embeddings)
        name = pc.model.name
    app = fastapi_app(settings, pc, tokenizer, factory, name, max_length)

    def _sigterm(*_a):
        raise SystemExit(0)

    signal.signal(signal.SIGTERM, _sigterm)
    try:
        import uvloop

        uvloop.run(serve_until_done(app, settings))
    except ImportError:
        asyncio.run(serve_until_done(app, settings))


@main.command()
@click.option("--base-url", default="http://127.0.0.1:8000")
@click.option("--model", required=True)
@click.option("--num-prompts", default=64, type=int)
@click.option("--max-concurrency", default=16, type=int)
@click.option("--input-len", default=128, type=int)
@click.option("--output-len", default=32, type=int)
@click.option("--vocab-size", default=256, type=int)
@click.option("--seed", default=0, type=int)
@click.option("--request-rate", default=0.0, type=float, help="open loop: Poisson arrivals at this rate (requests / s)")
@click.option("--dataset-name", default="random", type=click.Choice(["random", "sharegpt", "jsonl"]))
@click.option("--dataset-path", default=None, type=click.Path())
@click.option("--chat", is_flag=True, help="send /v1/chat/completions requests")
@click.option("--sweep-concurrency", default=None, help="comma-separated concurrencies: one closed-loop run each")
@click.option("--sweep-request-rate", default=None, help="comma-separated request rates: one open-loop run each")
@click.option("--result-file", default=None, type=click.Path(), help="also write the result JSON here")
def benchmark(base_url, model, num_prompts, max_concurrency, input_len, output_len, vocab_size, seed, request_rate,
              dataset_name, dataset_path, chat, sweep_concurrency, sweep_request_rate, result_file):
    """Serving benchmark against a running server: closed loop (--max-concurrency), open loop (--request-rate) or
    a sweep over either; random, ShareGPT-format or JSONL requests."""
    from ..benchmark.benchmark_serving import run_benchmark, run_sweep

    common = dict(input_len=input_len, output_len=output_len, vocab_size=vocab_size, seed=seed, dataset=dataset_name,
                  dataset_path=dataset_path, chat=chat)
    if sweep_concurrency or sweep_request_rate:
        cs = [int(x) for x in (sweep_concurrency or "").split(",") if x]
        rs = [float(x) for x in (sweep_request_rate or "").split(",") if x]
        res = asyncio.run(run_sweep(base_url, model, num_prompts, cs, rs, **common))
    else:
        res = asyncio.run(run_benchmark(base_url, model, num_prompts, max_concurrency, request_rate=request_rate, **common))
    text = json.dumps(res, indent=1)
    if result_file:
        with open(result_file, "w") as f:
            f.write(text)
    click.echo(text)


if __name__ == "__main__":
    main()


@main.command("replay-recording")
@click.argument("recording", type=click.Path(exists=True))
@click.option("--base-url", default="http://127.0.0.1:8000")
@click.option("--concurrency", default=8, type=int)
@click.option("--preserve-timing", is_flag=True, help="keep the recorded gaps between requests")
@click.option("--speedup", default=1.0, type=float)
@click.option("--limit", default=None, type=int)
def replay_recording_cmd(recording, base_url, concurrency, preserve_timing, speedup, limit):
    """Replay a JSONL transaction recording (see MAX_SERVE_TRANSACTION_RECORDING_FILE) against a server."""
    import asyncio
    import json

    from ..serve.recordreplay import replay_recording

    res = asyncio.run(replay_recording(recording, base_url, concurrency, preserve_timing, speedup, limit=limit))
    click.echo(json.dumps(res.summary()))
    if res.failures:
        raise SystemExit(1)
