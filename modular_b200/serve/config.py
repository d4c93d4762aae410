"""Server settings: every field can be set by a ``MAX_SERVE_*`` environment variable.

Reference: max/python/max/serve/config.py:93 ``Settings`` (port 8000 :133, ``max_queue_size``
:158, ``use_heartbeat`` :304, ``mw_timeout_s`` :309, ``metric_recording`` :364,
``stream_min_chunk_tokens`` :370, ``transaction_recording_file`` :384).
"""

from __future__ import annotations

import enum
from typing import Optional

from pydantic import Field
from pydantic_settings import BaseSettings, SettingsConfigDict


class APIType(str, enum.Enum):
    OPENAI = "openai"
    KSERVE = "kserve"
    SAGEMAKER = "sagemaker"


class MetricRecordingMethod(str, enum.Enum):
    NOOP = "NOOP"
    SYNC = "SYNC"
    ASYNCIO = "ASYNCIO"
    PROCESS = "PROCESS"


class MetricLevel(enum.IntEnum):
    NONE = 0
    BASIC = 10
    DETAILED = 20


class Settings(BaseSettings):
    model_config = SettingsConfigDict(env_prefix="MAX_SERVE_", extra="ignore", populate_by_name=True)

    # network
    host: str = Field(default="0.0.0.0", alias="MAX_SERVE_HOST")
    port: int = Field(default=8000, alias="MAX_SERVE_PORT")
    api_types: list[APIType] = Field(default_factory=lambda: [APIType.OPENAI])
    offline_inference: bool = False
    headless: bool = False
    # queues / transport
    max_queue_size: int = Field(default=0, description="pending requests before 429 (0 = unbounded)")
    max_pending_requests: int = 0
    stream_min_chunk_tokens: int = 1
    # model worker supervision
    use_heartbeat: bool = False
    mw_timeout_s: float = 20 * 60.0
    mw_health_fail_s: float = 60.0
    # telemetry
    log_level: str = "INFO"
    log_prefix: Optional[str] = None
    structured_logging: bool = False
    disable_telemetry: bool = True
    metric_recording: MetricRecordingMethod = MetricRecordingMethod.ASYNCIO
    metric_level: MetricLevel = MetricLevel.BASIC
    metrics_port: int = 8001
    detailed_buffer_factor: int = 20
    kernel_trace_level: int = 0
    profiling_enabled: bool = False     # ?profile=1 on a request writes profile.<request id>.txt (serve/debug.py)
    profile_dir: str = "."
    gc_debug: bool = False              # log slow garbage collections of the model worker (MAX_SERVE_GC_DEBUG)
    gc_debug_top_objects: int = 0       # with gc_debug: also the N most common types of the collected generation
    # record / replay
    transaction_recording_file: Optional[str] = None
    transaction_recording_include_responses: bool = False
    # misc
    dummy_model: bool = Field(default=False, alias="MAX_SERVE_DUMMY_MODEL")
    allowed_image_roots: list[str] = Field(default_factory=list)
    di_bind_address: str = "tcp://127.0.0.1:5555"
