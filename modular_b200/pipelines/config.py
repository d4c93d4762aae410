"""Configuration system.

Mirrors the reference's layering (max/python/max/config/__init__.py:591 ``MAXConfig``,
max/python/max/pipelines/lib/config/config.py:122 ``PipelineConfig``, model_config.py:666
``MAXModelConfig``, pipeline_runtime_config.py:34, kv_cache/config.py:186 ``KVCacheConfig``,
sampling/sampling_config.py:60):

* every section is a pydantic model; a YAML/JSON ``config_file`` is read first, explicit
  keyword arguments (CLI flags) override it field by field, and ``MB200_<FIELD>`` /
  ``MAX_<FIELD>`` environment variables fill anything still unset;
* ``PipelineArgs.from_flat_kwargs`` turns the flat ``--flag value`` namespace of the CLI into
  the nested sections; ``PipelineConfig.from_args`` resolves defaults that depend on each
  other (overlap scheduler, graph capture, chunked prefill, roles).
"""

from __future__ import annotations

import enum
import json
import os
from pathlib import Path
from typing import Any, Optional

import yaml
from pydantic import BaseModel, ConfigDict, Field, model_validator


class ConfigFileModel(BaseModel):
    """Base for all sections: file + kwargs + env merge."""

    model_config = ConfigDict(extra="forbid", validate_assignment=True, arbitrary_types_allowed=True)

    @classmethod
    def env_prefixes(cls) -> tuple[str, ...]:
        return ("MB200_", "MAX_")

    @classmethod
    def load(cls, config_file: Optional[str] = None, section: Optional[str] = None, **overrides):
        data: dict[str, Any] = {}
        if config_file:
            text = Path(config_file).read_text()
            raw = json.loads(text) if config_file.endswith(".json") else yaml.safe_load(text)
            raw = raw or {}
            if section and section in raw:
                raw = raw[section]
            data.update({k: v for k, v in raw.items() if k in cls.model_fields})
        for name in cls.model_fields:
            if name in overrides and overrides[name] is not None:
                data[name] = overrides[name]
            elif name not in data:
                for pre in cls.env_prefixes():
                    v = os.environ.get(pre + name.upper())
                    if v is not None:
                        data[name] = v
                        break
        return cls(**data)

    def merged(self, **overrides):
        d = self.model_dump()
        d.update({k: v for k, v in overrides.items() if v is not None})
        return type(self)(**d)


class PipelineRole(str, enum.Enum):
    PREFILL_AND_DECODE = "prefill_and_decode"
    PREFILL_ONLY = "prefill_only"
    DECODE_ONLY = "decode_only"


class KVCacheConfig(ConfigFileModel):
    cache_strategy: str = "paged"
    kv_cache_page_size: int = 128
    enable_prefix_caching: bool = True
    device_memory_utilization: float = 0.9
    kv_cache_format: Optional[str] = None          # None = model dtype, "float8_e4m3fn" = fp8 KV
    host_kvcache_swap_space_gb: float = 0.0        # pinned host memory for evicted prefix pages
    disk_kvcache_dir: Optional[str] = None         # file tier below the host tier
    disk_kvcache_space_gb: float = 0.0
    kv_block_hash_algorithm: str = "native64"       # native64 | sha256
    enable_kv_head_replication: bool = False        # TP degree > kv heads

    @model_validator(mode="after")
    def _check(self):
        if self.cache_strategy != "paged":
            raise ValueError("only the paged KV cache strategy exists")
        if self.kv_cache_page_size < 16 or self.kv_cache_page_size % 16:
            raise ValueError("kv_cache_page_size must be a positive multiple of 16")
        if not (0.0 < self.device_memory_utilization <= 1.0):
            raise ValueError("device_memory_utilization must be in (0, 1]")
        return self


class SamplingConfig(ConfigFileModel):
    in_dtype: str = "float32"
    enable_structured_output: bool = False
    enable_variable_logits: bool = False
    enable_penalties: bool = True
    enable_min_tokens: bool = True
    do_penalties: bool = False


class ProfilingConfig(ConfigFileModel):
    gpu_profiling: str = "off"                      # off | on | detailed
    profile_output: Optional[str] = None


class LoRAConfig(ConfigFileModel):
    enable_lora: bool = False
    lora_paths: list[str] = Field(default_factory=list)
    max_lora_rank: int = 16
    max_num_loras: int = 1


class SpeculativeConfig(ConfigFileModel):
    speculative_method: Optional[str] = None        # ngram | standalone (draft_model_path) are served; eagle | mtp are names only
    num_speculative_tokens: int = 0
    draft_model_path: Optional[str] = None


class ModelConfig(ConfigFileModel):
    """Which model, where its weights are, on which devices (reference: MAXModelConfig)."""

    model_path: str = ""
    served_model_name: Optional[str] = None
    weight_path: list[str] = Field(default_factory=list)
    quantization_encoding: Optional[str] = None     # bfloat16 | float32 | float8_e4m3fn | ...
    devices: str = "gpu"                            # "cpu", "gpu", "gpu:0,1,2,3"
    data_parallel_degree: int = 1
    tensor_parallel_degree: Optional[int] = None
    max_length: Optional[int] = None
    trust_remote_code: bool = False
    rope_type: Optional[str] = None
    random_weights: bool = False                    # build from config only (benchmarks, tests)
    kv_cache: KVCacheConfig = Field(default_factory=KVCacheConfig)

    @property
    def device_ids(self) -> list[int]:
        d = self.devices.lower()
        if d.startswith("cpu"):
            return []
        if ":" in d:
            return [int(x) for x in d.split(":", 1)[1].split(",") if x != ""]
        return [0]

    @property
    def uses_gpu(self) -> bool:
        return not self.devices.lower().startswith("cpu")

    @property
    def name(self) -> str:
        return self.served_model_name or self.model_path


class PipelineRuntimeConfig(ConfigFileModel):
    pipeline_role: PipelineRole = PipelineRole.PREFILL_AND_DECODE
    max_batch_size: Optional[int] = None
    max_batch_input_tokens: int = 8192
    max_batch_total_tokens: Optional[int] = None
    enable_chunked_prefill: bool = True
    enable_in_flight_batching: bool = False
    max_num_steps: int = 1
    max_queue_size_tg: Optional[int] = None
    min_batch_size_tg: Optional[int] = None
    ep_size: int = 1
    ep_use_allreduce: bool = False
    use_vendor_blas: bool = False
    use_vendor_ccl: bool = False                    # NCCL collectives instead of the fused kernels
    device_graph_capture: Optional[bool] = None
    max_graph_capture_batch_size: int = 128
    fold_sampler_into_graph: bool = True
    max_pending_futures: int = 1
    enable_overlap_scheduler: Optional[bool] = None
    enable_echo: bool = False
    reasoning_parser: Optional[str] = None
    tool_parser: Optional[str] = None
    pool_embeddings: bool = True


class PipelineConfig(ConfigFileModel):
    model: ModelConfig = Field(default_factory=ModelConfig)
    draft_model: Optional[ModelConfig] = None
    sampling: SamplingConfig = Field(default_factory=SamplingConfig)
    profiling: ProfilingConfig = Field(default_factory=ProfilingConfig)
    lora: LoRAConfig = Field(default_factory=LoRAConfig)
    speculative: SpeculativeConfig = Field(default_factory=SpeculativeConfig)
    runtime: PipelineRuntimeConfig = Field(default_factory=PipelineRuntimeConfig)
    task: str = "text_generation"
    # set by the model worker for each tensor-parallel rank it starts (not user options)
    tp_size: int = 1
    tp_rank: int = 0
    # likewise for the ranks of an expert-parallel engine (runtime.ep_size of them)
    ep_rank: int = 0

    @property
    def expert_parallel_degree(self) -> int:
        """Ranks that share the routed experts (``--ep-size``; attention is then data parallel: every rank serves
        its own requests. Reference: pipeline_runtime_config.py:96)."""
        return max(1, int(self.runtime.ep_size or 1)) if self.model.uses_gpu else 1

    @property
    def tensor_parallel_degree(self) -> int:
        """GPUs that share one model replica: the configured devices divided among the data-parallel replicas
        (the reference shards a model over all devices it is given, nn/transformer/distributed_transformer.py)."""
        m = self.model
        if not m.uses_gpu or self.expert_parallel_degree > 1:
            return 1
        if m.tensor_parallel_degree:
            return max(1, min(int(m.tensor_parallel_degree), len(m.device_ids)))
        return max(1, len(m.device_ids) // max(1, m.data_parallel_degree or 1))

    # ---- convenience accessors used across the code base
    @property
    def model_path(self) -> str:
        return self.model.model_path

    @property
    def max_length(self) -> Optional[int]:
        return self.model.max_length

    @classmethod
    def from_args(cls, args: "PipelineArgs") -> "PipelineConfig":
        cfg = cls(model=args.model, sampling=args.sampling, profiling=args.profiling, lora=args.lora,
                  speculative=args.speculative, runtime=args.runtime, task=args.task)
        cfg.resolve()
        return cfg

    def resolve(self) -> None:
        """Fill defaults that depend on other fields (reference: config.py:892, :965)."""
        rt, m = self.runtime, self.model
        gpu = m.uses_gpu
        if rt.enable_overlap_scheduler is None:
            rt.enable_overlap_scheduler = gpu and self.speculative.speculative_method is None
        if rt.device_graph_capture is None:
            rt.device_graph_capture = gpu
        if not gpu:
            rt.enable_overlap_scheduler = False
            rt.device_graph_capture = False
        if m.tensor_parallel_degree is None:
            n = max(1, len(m.device_ids))
            m.tensor_parallel_degree = max(1, n // max(1, m.data_parallel_degree))
        if rt.max_batch_size is None:
            rt.max_batch_size = 256 if gpu else 8
        # structured output keeps overlap scheduling: the pipeline reads back the previous token only for
        # batches that contain a grammar-constrained request
        if rt.pipeline_role is not PipelineRole.PREFILL_AND_DECODE:
            rt.enable_in_flight_batching = False

    def needs_bitmask_constraints(self) -> bool:
        return self.sampling.enable_structured_output

    def summary(self) -> dict:
        return json.loads(self.model_dump_json())


_SECTIONS = {"model": ModelConfig, "sampling": SamplingConfig, "profiling": ProfilingConfig,
             "lora": LoRAConfig, "speculative": SpeculativeConfig, "runtime": PipelineRuntimeConfig,
             "kv_cache": KVCacheConfig}


class PipelineArgs(BaseModel):
    """Nested sections built from flat CLI kwargs (reference: pipeline_args.py:110, :422)."""

    model_config = ConfigDict(arbitrary_types_allowed=True)
    model: ModelConfig
    sampling: SamplingConfig
    profiling: ProfilingConfig
    lora: LoRAConfig
    speculative: SpeculativeConfig
    runtime: PipelineRuntimeConfig
    task: str = "text_generation"

    @classmethod
    def flat_fields(cls) -> dict[str, tuple[str, Any]]:
        """flat flag name -> (section, pydantic FieldInfo); the CLI derives its options from this."""
        out: dict[str, tuple[str, Any]] = {}
        for sec, klass in _SECTIONS.items():
            for name, info in klass.model_fields.items():
                if name == "kv_cache":
                    continue
                out.setdefault(name, (sec, info))
        return out

    @classmethod
    def from_flat_kwargs(cls, config_file: Optional[str] = None, **flat) -> "PipelineArgs":
        fields = cls.flat_fields()
        unknown = [k for k in flat if k not in fields and k != "task"]
        if unknown:
            raise ValueError(f"unknown pipeline options: {sorted(unknown)}")
        by_sec: dict[str, dict] = {s: {} for s in _SECTIONS}
        for k, v in flat.items():
            if k == "task" or v is None:
                continue
            by_sec[fields[k][0]][k] = v
        kv = KVCacheConfig.load(config_file, "kv_cache", **by_sec["kv_cache"])
        model = ModelConfig.load(config_file, "model", **by_sec["model"], kv_cache=kv)
        return cls(
            model=model,
            sampling=SamplingConfig.load(config_file, "sampling", **by_sec["sampling"]),
            profiling=ProfilingConfig.load(config_file, "profiling", **by_sec["profiling"]),
            lora=LoRAConfig.load(config_file, "lora", **by_sec["lora"]),
            speculative=SpeculativeConfig.load(config_file, "speculative", **by_sec["speculative"]),
            runtime=PipelineRuntimeConfig.load(config_file, "runtime", **by_sec["runtime"]),
            task=flat.get("task") or "text_generation")
