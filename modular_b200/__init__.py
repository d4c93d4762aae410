"""modular_b200: a Blackwell-native LLM inference framework.

Public surface (mirrors the reference's ``max`` package where a user touches it):

* ``modular_b200.entrypoints``  - ``serve`` / ``generate`` / ``encode`` / ``list`` /
  ``benchmark`` / ``warm-cache`` CLI and the offline ``LLM`` class
* ``modular_b200.pipelines``    - ``PipelineConfig``, ``PIPELINE_REGISTRY``, text-generation pipelines
* ``modular_b200.serve``        - OpenAI-compatible API server, scheduler, worker transport
* ``modular_b200.kv_cache``     - paged KV cache manager with prefix caching
* ``modular_b200.nn`` / ``models`` / ``ops`` / ``parallel`` - layers, architectures, sm_100a kernels,
  tensor/expert parallel communication
"""

__version__ = "0.1.0"
