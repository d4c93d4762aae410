"""Architecture registry and pipeline factory.

``PIPELINE_REGISTRY.retrieve_factory(pipeline_config)`` returns ``(tokenizer, factory)`` where
``factory()`` builds the ready-to-run pipeline (weights loaded, KV cache allocated, graphs
captured). Building is deferred so the API process can construct the tokenizer while the
model worker process runs the factory. Reference: max/python/max/pipelines/lib/registry.py:330
(``retrieve_factory`` :649, memory plan :731, factory :901) and lib/arch_lookup.py:70
``SupportedArchitecture``.
"""

from __future__ import annotations

import functools
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch

from .config import PipelineConfig
from .memory_estimation import MemoryEstimator, MemoryPlan
from .tokenizer import PipelineTokenizer, load_tokenizer
from .weights import load_hf_config, load_state_dict, parse_quant_config


@dataclass
class SupportedArchitecture:
    name: str                                  # HF architecture string, e.g. "LlamaForCausalLM"
    config_class: Any
    weights_class: Any
    model_class: Any
    default_encoding: str = "bfloat16"
    supported_encodings: tuple = ("bfloat16", "float32")
    example_repo_ids: tuple = ()
    task: str = "text_generation"
    preset_configs: dict = field(default_factory=dict)   # name -> callable returning a config


class PipelineRegistry:
    def __init__(self):
        self.architectures: dict[str, SupportedArchitecture] = {}
        self._lazy: list[Callable[[], None]] = []

    def register(self, arch: SupportedArchitecture, allow_override: bool = False) -> None:
        if arch.name in self.architectures and not allow_override:
            raise ValueError(f"architecture {arch.name} is already registered")
        self.architectures[arch.name] = arch

    def register_lazy(self, fn: Callable[[], None]) -> None:
        self._lazy.append(fn)

    def _materialise(self) -> None:
        while self._lazy:
            self._lazy.pop(0)()

    def list_architectures(self) -> list[SupportedArchitecture]:
        self._materialise()
        return sorted(self.architectures.values(), key=lambda a: a.name)

    def retrieve_architecture(self, hf_config: dict) -> SupportedArchitecture:
        self._materialise()
        for name in hf_config.get("architectures", []):
            if name in self.architectures:
                return self.architectures[name]
        raise ValueError(f"no registered architecture among {hf_config.get('architectures')}; "
                         f"known: {sorted(self.architectures)}")

    # ------------------------------------------------------------ config resolution
    def resolve_model(self, pc: PipelineConfig):
        """Returns (arch, model config object, hf config dict)."""
        self._materialise()
        m = pc.model
        if m.model_path.startswith("preset:"):
            preset = m.model_path.split(":", 1)[1]
            for arch in self.architectures.values():
                if preset in arch.preset_configs:
                    cfg = arch.preset_configs[preset]()
                    return arch, cfg, cfg.to_hf()
            raise ValueError(f"unknown preset {preset!r}")
        hf = load_hf_config(m.model_path)
        arch = self.retrieve_architecture(hf)
        return arch, arch.config_class.from_hf(hf), hf

    def retrieve_tokenizer(self, pc: PipelineConfig, vocab_size: int = 258) -> PipelineTokenizer:
        path = "" if pc.model.model_path.startswith("preset:") else pc.model.model_path
        return load_tokenizer(path, vocab_size, pc.model.trust_remote_code)

    def plan_memory(self, pc: PipelineConfig, cfg, device: torch.device) -> Optional[MemoryPlan]:
        if device.type != "cuda":
            return None
        from ..models import family_for

        dtype_bytes = 2
        fam = family_for(cfg)
        kvp = fam.kv_params(cfg, pc.model.kv_cache.kv_cache_page_size, torch.bfloat16, True)
        free, total = torch.cuda.mem_get_info(device)
        act = fam.activation_bytes(cfg, pc.runtime.max_batch_input_tokens, pc.runtime.max_batch_size or 256)
        return MemoryEstimator.plan_from_sizes(
            free, total, cfg.param_count() * dtype_bytes, act, kvp.bytes_per_page, kvp.page_size,
            pc.model.kv_cache.device_memory_utilization, 0, pc.runtime.max_batch_size,
            pc.model.max_length, cfg.max_position_embeddings)

    # ------------------------------------------------------------ factory
    def retrieve_factory(self, pc: PipelineConfig):
        pc.resolve()
        arch, cfg, hf = self.resolve_model(pc)
        tokenizer = self.retrieve_tokenizer(pc, cfg.vocab_size)
        factory = functools.partial(self._build, pc, arch, cfg, hf, tokenizer)
        return tokenizer, factory

    def retrieve(self, pc: PipelineConfig):
        tokenizer, factory = self.retrieve_factory(pc)
        return tokenizer, factory()

    def _build(self, pc: PipelineConfig, arch: SupportedArchitecture, cfg, hf: dict, tokenizer):
        from ..entrypoints.llm import LLM

        m, rt = pc.model, pc.runtime
        on_gpu = m.uses_gpu and torch.cuda.is_available()
        ep_size, ep_rank = pc.expert_parallel_degree, int(getattr(pc, "ep_rank", 0) or 0)
        if ep_size > 1 and not hasattr(arch.weights_class, "random_init_ep"):
            raise ValueError(f"--ep-size needs a mixture-of-experts architecture ({arch.name} is not)")
        dev_i = int(getattr(pc, "tp_rank", 0) or 0) if int(getattr(pc, "tp_size", 1) or 1) > 1 else (ep_rank if ep_size > 1 else 0)
        device = torch.device(f"cuda:{m.device_ids[dev_i]}" if on_gpu else "cpu")
        enc = m.quantization_encoding or (arch.default_encoding if on_gpu else "float32")
        # float8_e4m3fn: projections are quantised to block-scaled fp8 at load (checkpoints that already are
        # block-scaled fp8 stay fp8 under every encoding); everything else runs in bf16
        to_fp8 = enc in ("float8_e4m3fn", "fp8")
        dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16,
                 "float8_e4m3fn": torch.bfloat16, "fp8": torch.bfloat16}.get(enc)
        if dtype is None:
            raise ValueError(f"encoding {enc!r} is not supported by {arch.name} (supported: {arch.supported_encodings})")
        quant = parse_quant_config(hf)
        if quant is not None and not quant.is_blockscaled_fp8:
            raise ValueError(f"quantisation format {quant.format!r} is not supported yet")
        tp_size, tp_rank = int(getattr(pc, "tp_size", 1) or 1), int(getattr(pc, "tp_rank", 0) or 0)
        sharded = False
        if m.random_weights or m.model_path.startswith("preset:"):
            weights = None
            # models too large to exist whole on one GPU (and fp8 ones) are created at shard size; small ones
            # are created whole and sliced, so that every tensor-parallel degree serves the same weights
            big = hasattr(cfg, "param_count") and cfg.param_count() > 30e9
            if ep_size > 1 and (big or to_fp8):
                # this rank's experts only (block-scaled fp8 under the fp8 encoding), the rest replicated
                weights = arch.weights_class.random_init_ep(cfg, ep_rank, ep_size, device, dtype, seed=0, fp8_experts=to_fp8)
            elif ep_size > 1:
                # small models: the weights every degree of parallelism serves, sliced to this rank's experts
                el = cfg.n_routed_experts // ep_size
                weights = arch.weights_class.random_init(cfg, device, dtype, seed=0, e_begin=ep_rank * el, e_end=(ep_rank + 1) * el)
            elif (to_fp8 or (tp_size > 1 and big)) and hasattr(arch.weights_class, "random_init_shard"):
                weights = arch.weights_class.random_init_shard(cfg, tp_rank, tp_size, device, dtype, seed=0, fp8=to_fp8)
                sharded = tp_size > 1
        else:
            sd = load_state_dict(m.model_path, m.weight_path)
            if ep_size > 1:
                el = cfg.n_routed_experts // ep_size
                weights = arch.weights_class.from_state_dict(cfg, sd.to_dict(), device, dtype, e_begin=ep_rank * el,
                                                             e_end=(ep_rank + 1) * el)
            else:
                weights = arch.weights_class.from_state_dict(cfg, sd.to_dict(), device, dtype)
                if to_fp8:
                    weights = weights.quantize_fp8()
        spec = _speculative_from(pc)
        draft_cfg = draft_weights = None
        if spec is not None and spec.method == "draft_model":
            # the draft model resolves like the served one: a preset or a checkpoint directory of a registered family
            dpath = pc.speculative.draft_model_path
            if not dpath:
                raise ValueError("--speculative-method standalone needs --draft-model-path")
            if dpath.startswith("preset:"):
                name = dpath.split(":", 1)[1]
                hits = [a for a in self.architectures.values() if name in a.preset_configs]
                if not hits:
                    raise ValueError(f"unknown draft preset {name!r}")
                darch, draft_cfg = hits[0], hits[0].preset_configs[name]()
            else:
                dhf = load_hf_config(dpath)
                darch = self.retrieve_architecture(dhf)
                draft_cfg = darch.config_class.from_hf(dhf)
                draft_weights = darch.weights_class.from_state_dict(draft_cfg, load_state_dict(dpath, []).to_dict(),
                                                                    device, dtype)
        plan = self.plan_memory(pc, cfg, device) if on_gpu else None
        max_length = min(m.max_length or cfg.max_position_embeddings, cfg.max_position_embeddings)
        if plan is not None:
            max_length = min(max_length, plan.max_length)
        max_bs = rt.max_batch_size or (plan.max_batch_size if plan else 8)
        llm = LLM(cfg, weights, device=str(device), dtype=dtype, max_length=max_length,
                  max_batch_size=max_bs, max_batch_input_tokens=rt.max_batch_input_tokens,
                  page_size=m.kv_cache.kv_cache_page_size,
                  device_memory_utilization=m.kv_cache.device_memory_utilization,
                  num_kv_pages=None if on_gpu else max(64, max_bs * ((max_length + m.kv_cache.kv_cache_page_size - 1)
                                                                     // m.kv_cache.kv_cache_page_size) + 1),
                  enable_prefix_caching=m.kv_cache.enable_prefix_caching,
                  enable_chunked_prefill=rt.enable_chunked_prefill,
                  enable_in_flight_batching=rt.enable_in_flight_batching,
                  enable_overlap_scheduler=rt.enable_overlap_scheduler,
                  device_graph_capture=bool(rt.device_graph_capture),
                  graph_batch_sizes=[b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256)
                                     if b <= min(max_bs, rt.max_graph_capture_batch_size)],
                  eos_token_ids=tokenizer.eos_token_ids,
                  host_kvcache_swap_space_gb=m.kv_cache.host_kvcache_swap_space_gb,
                  disk_kvcache_dir=m.kv_cache.disk_kvcache_dir,
                  disk_kvcache_space_gb=m.kv_cache.disk_kvcache_space_gb,
                  tp_size=tp_size, tp_rank=tp_rank, weights_are_sharded=sharded,
                  speculative=spec, draft_model_config=draft_cfg, draft_weights=draft_weights,
                  ep_size=ep_size, ep_rank=ep_rank,
                  ep_fp8_dispatch=ep_size > 1 and getattr(cfg, "hidden_size", 0) % 512 == 0)
        llm.tokenizer = tokenizer
        if pc.sampling.enable_structured_output:
            llm.pipeline.enable_structured_output(tokenizer)
        llm.pipeline_config = pc
        llm.memory_plan = plan
        return llm


PIPELINE_REGISTRY = PipelineRegistry()


def _speculative_from(pc):
    """The engine's speculative-decoding settings from the pipeline config: ``--speculative-method ngram``, or
    ``standalone`` (alias ``draft_model``) with ``--draft-model-path``, a separate smaller model of the same
    vocabulary. The reference's ``eagle`` / ``mtp`` methods draft from the target's hidden states with extra
    trained heads; they are not served by this loop."""
    sc = pc.speculative
    if not sc.speculative_method:
        return None
    from .speculative import SpeculativeConfig as EngineSpec

    if sc.speculative_method == "ngram":
        return EngineSpec(method="ngram", num_speculative_tokens=sc.num_speculative_tokens or 4)
    if sc.speculative_method in ("standalone", "draft_model"):
        return EngineSpec(method="draft_model", num_speculative_tokens=sc.num_speculative_tokens or 4)
    raise ValueError(f"speculative method {sc.speculative_method!r} is not available in the serving loop "
                     "(ngram and standalone are)")


def _register_builtin() -> None:
    from ..models.llama3 import Llama3Config, Llama3Model, Llama3Weights

    llama = SupportedArchitecture(
        name="LlamaForCausalLM", config_class=Llama3Config, weights_class=Llama3Weights,
        model_class=Llama3Model, default_encoding="bfloat16",
        supported_encodings=("bfloat16", "float32", "float8_e4m3fn"),
        example_repo_ids=("meta-llama/Llama-3.1-8B-Instruct", "meta-llama/Llama-3.3-70B-Instruct"),
        preset_configs={"llama3.1-8b": Llama3Config.llama31_8b, "llama3.3-70b": Llama3Config.llama33_70b,
                        "tiny-llama": Llama3Config.tiny})
    PIPELINE_REGISTRY.register(llama, allow_override=True)
    from ..models.llama3 import MistralConfig

    # same layers, tensor names and kernels as Llama; full attention only
    mistral = SupportedArchitecture(
        name="MistralForCausalLM", config_class=MistralConfig, weights_class=Llama3Weights,
        model_class=Llama3Model, default_encoding="bfloat16",
        supported_encodings=("bfloat16", "float32", "float8_e4m3fn"),
        example_repo_ids=("mistralai/Mistral-7B-Instruct-v0.3", "mistralai/Mistral-Nemo-Instruct-2407"),
        preset_configs={})
    PIPELINE_REGISTRY.register(mistral, allow_override=True)
    # vision-language checkpoints around a Mistral or Llama language model: that model is served, for text (the
    # vision tower and projector are dropped at load, requests with image parts are refused)
    for name, repo in (("Mistral3ForConditionalGeneration", "mistralai/Mistral-Small-3.1-24B-Instruct-2503"),
                       ("LlavaForConditionalGeneration", "mistral-community/pixtral-12b"),
                       ("Idefics3ForConditionalGeneration", "HuggingFaceTB/SmolVLM-Instruct")):
        PIPELINE_REGISTRY.register(SupportedArchitecture(
            name=name, config_class=MistralConfig, weights_class=Llama3Weights, model_class=Llama3Model,
            default_encoding="bfloat16", supported_encodings=("bfloat16", "float32", "float8_e4m3fn"),
            example_repo_ids=(repo,), preset_configs={}), allow_override=True)
    from ..models.llama3 import Qwen2Config

    # the Llama layer with a bias on the fused query / key / value projection
    qwen2 = SupportedArchitecture(
        name="Qwen2ForCausalLM", config_class=Qwen2Config, weights_class=Llama3Weights,
        model_class=Llama3Model, default_encoding="bfloat16",
        supported_encodings=("bfloat16", "float32", "float8_e4m3fn"),
        example_repo_ids=("Qwen/Qwen2.5-7B-Instruct", "Qwen/Qwen2.5-72B-Instruct"),
        preset_configs={"tiny-qwen2": Qwen2Config.tiny})
    PIPELINE_REGISTRY.register(qwen2, allow_override=True)
    from ..models.llama3 import Qwen3Config

    # the Llama layer with an RMSNorm on every query and key head before the rotation
    qwen3 = SupportedArchitecture(
        name="Qwen3ForCausalLM", config_class=Qwen3Config, weights_class=Llama3Weights,
        model_class=Llama3Model, default_encoding="bfloat16",
        supported_encodings=("bfloat16", "float32", "float8_e4m3fn"),
        example_repo_ids=("Qwen/Qwen3-8B", "Qwen/Qwen3-32B"),
        preset_configs={"tiny-qwen3": Qwen3Config.tiny})
    PIPELINE_REGISTRY.register(qwen3, allow_override=True)
    # Qwen vision-language checkpoints: the language model, served for text (multimodal rotary sections reduce to
    # the plain rotation without images; the vision tower is dropped at load)
    for name, cc, repo in (("Qwen2_5_VLForConditionalGeneration", Qwen2Config, "Qwen/Qwen2.5-VL-7B-Instruct"),
                           ("Qwen2VLForConditionalGeneration", Qwen2Config, "Qwen/Qwen2-VL-7B-Instruct"),
                           ("Qwen3VLForConditionalGeneration", Qwen3Config, "Qwen/Qwen3-VL-8B-Instruct")):
        PIPELINE_REGISTRY.register(SupportedArchitecture(
            name=name, config_class=cc, weights_class=Llama3Weights, model_class=Llama3Model,
            default_encoding="bfloat16", supported_encodings=("bfloat16", "float32", "float8_e4m3fn"),
            example_repo_ids=(repo,), preset_configs={}), allow_override=True)
    from ..models.llama3 import MixtralConfig, Qwen3MoeConfig

    # Llama / Qwen3 attention with a mixture-of-experts feed-forward (softmax top-k routing, grouped GEMMs); these
    # layers run op by op, without the native step executor
    for name, cc, repos, presets in (
            ("MixtralForCausalLM", MixtralConfig, ("mistralai/Mixtral-8x7B-Instruct-v0.1",), {"tiny-mixtral": MixtralConfig.tiny}),
            ("Qwen3MoeForCausalLM", Qwen3MoeConfig, ("Qwen/Qwen3-30B-A3B",), {"tiny-qwen3-moe": Qwen3MoeConfig.tiny})):
        PIPELINE_REGISTRY.register(SupportedArchitecture(
            name=name, config_class=cc, weights_class=Llama3Weights, model_class=Llama3Model,
            default_encoding="bfloat16", supported_encodings=("bfloat16", "float32"), example_repo_ids=repos,
            preset_configs=presets), allow_override=True)
    from ..models.llama3 import GraniteConfig

    PIPELINE_REGISTRY.register(SupportedArchitecture(
        name="GraniteForCausalLM", config_class=GraniteConfig, weights_class=Llama3Weights, model_class=Llama3Model,
        default_encoding="bfloat16", supported_encodings=("bfloat16", "float32"),
        example_repo_ids=("ibm-granite/granite-3.3-8b-instruct",), preset_configs={}), allow_override=True)
    from ..models.llama3 import Gemma3Config

    # Gemma 3 text: norms on block inputs and outputs, tanh-GELU MLP, two rotary bases; op by op
    # (Gemma3ForConditionalGeneration: the language model of the vision-language checkpoints, served for text)
    for name, repo in (("Gemma3ForCausalLM", "google/gemma-3-1b-it"), ("Gemma3ForConditionalGeneration", "google/gemma-3-4b-it")):
        PIPELINE_REGISTRY.register(SupportedArchitecture(
            name=name, config_class=Gemma3Config, weights_class=Llama3Weights, model_class=Llama3Model,
            default_encoding="bfloat16", supported_encodings=("bfloat16", "float32"),
            example_repo_ids=(repo,), preset_configs={}), allow_override=True)
    from ..models.llama3 import Olmo2Config, OlmoConfig

    # OLMo: parameter-free LayerNorms and clamped projections. OLMo 2 / 3: Llama projections with the norms on the
    # block outputs and over the whole query / key projection. Both run op by op
    for name, cc, repos in (("OlmoForCausalLM", OlmoConfig, ("allenai/OLMo-7B-0724-Instruct-hf",)),
                            ("Olmo2ForCausalLM", Olmo2Config, ("allenai/OLMo-2-1124-7B-Instruct",)),
                            ("Olmo3ForCausalLM", Olmo2Config, ("allenai/Olmo-3-7B-Instruct",))):
        PIPELINE_REGISTRY.register(SupportedArchitecture(
            name=name, config_class=cc, weights_class=Llama3Weights, model_class=Llama3Model,
            default_encoding="bfloat16", supported_encodings=("bfloat16", "float32"), example_repo_ids=repos,
            preset_configs={"tiny-olmo2": Olmo2Config.tiny} if name == "Olmo2ForCausalLM" else {}),
            allow_override=True)
    from ..models.mamba import MambaConfig, MambaModel, MambaWeights

    # selective state-space layers: a fixed-size recurrent state per request instead of a KV cache
    PIPELINE_REGISTRY.register(SupportedArchitecture(
        name="MambaForCausalLM", config_class=MambaConfig, weights_class=MambaWeights, model_class=MambaModel,
        default_encoding="bfloat16", supported_encodings=("bfloat16", "float32"),
        example_repo_ids=("state-spaces/mamba-130m-hf", "state-spaces/mamba-2.8b-hf"),
        preset_configs={"tiny-mamba": MambaConfig.tiny, "mamba-130m": MambaConfig.mamba_130m,
                        "mamba-2.8b": MambaConfig.mamba_2_8b}), allow_override=True)
    from ..models.lfm2 import Lfm2Config, Lfm2Model, Lfm2Weights

    # hybrid decoder: gated short-convolution layers (a convolution tail per request) between attention layers
    PIPELINE_REGISTRY.register(SupportedArchitecture(
        name="Lfm2ForCausalLM", config_class=Lfm2Config, weights_class=Lfm2Weights, model_class=Lfm2Model,
        default_encoding="bfloat16", supported_encodings=("bfloat16", "float32"),
        example_repo_ids=("LiquidAI/LFM2-1.2B",), preset_configs={"tiny-lfm2": Lfm2Config.tiny}), allow_override=True)
    from ..models.bert import BertConfig, BertModel, BertWeights

    # encoder-only embedding models (bidirectional attention; MPNet adds relative-position biases); embeddings only
    for name, repos, presets in (
            ("BertModel", ("sentence-transformers/all-MiniLM-L6-v2", "BAAI/bge-base-en-v1.5"), {"tiny-bert": BertConfig.tiny}),
            ("MPNetForMaskedLM", ("sentence-transformers/all-mpnet-base-v2",), {}),
            ("MPNetModel", ("sentence-transformers/all-mpnet-base-v2",), {})):
        PIPELINE_REGISTRY.register(SupportedArchitecture(
            name=name, config_class=BertConfig, weights_class=BertWeights, model_class=BertModel,
            default_encoding="float32", supported_encodings=("float32", "bfloat16"), example_repo_ids=repos,
            task="embeddings_generation", preset_configs=presets), allow_override=True)
    from ..models.llama3 import Phi3Config

    # the Llama layer with the projections already fused in the checkpoint
    phi3 = SupportedArchitecture(
        name="Phi3ForCausalLM", config_class=Phi3Config, weights_class=Llama3Weights,
        model_class=Llama3Model, default_encoding="bfloat16",
        supported_encodings=("bfloat16", "float32", "float8_e4m3fn"),
        example_repo_ids=("microsoft/Phi-3-mini-4k-instruct", "microsoft/Phi-3.5-mini-instruct"),
        preset_configs={})
    PIPELINE_REGISTRY.register(phi3, allow_override=True)

    from ..models.deepseek_v3 import DeepseekV3Config, DeepseekV3Model, DeepseekV3Weights

    deepseek = SupportedArchitecture(
        name="DeepseekV3ForCausalLM", config_class=DeepseekV3Config, weights_class=DeepseekV3Weights,
        model_class=DeepseekV3Model, default_encoding="bfloat16",
        supported_encodings=("bfloat16", "float32", "float8_e4m3fn"),
        example_repo_ids=("deepseek-ai/DeepSeek-V3", "deepseek-ai/DeepSeek-R1"),
        preset_configs={"deepseek-v3": DeepseekV3Config.deepseek_v3, "tiny-deepseek": DeepseekV3Config.tiny})
    PIPELINE_REGISTRY.register(deepseek, allow_override=True)
    # DeepSeek-V2 / V2-Lite: the same model code with a softmax top-k router (config mapping in from_hf)
    PIPELINE_REGISTRY.register(SupportedArchitecture(
        name="DeepseekV2ForCausalLM", config_class=DeepseekV3Config, weights_class=DeepseekV3Weights,
        model_class=DeepseekV3Model, default_encoding="bfloat16", supported_encodings=("bfloat16", "float32"),
        example_repo_ids=("deepseek-ai/DeepSeek-V2-Lite",), preset_configs={}), allow_override=True)


PIPELINE_REGISTRY.register_lazy(_register_builtin)
