"""Echo pipeline: "generates" the prompt back, one token per step.

Used with ``MAX_SERVE_DUMMY_MODEL=1`` and in tests to exercise the server, transport and
scheduler without a model (reference: max/python/max/serve/pipelines/echo_gen.py).
"""

from __future__ import annotations

from typing import Sequence

from ...pipelines.context import TextContext


class EchoPipeline:
    """Duck-types TextGenerationPipeline: ``execute(batch) -> {request_id: output}``."""

    def __init__(self, max_batch_size: int = 64):
        self.max_batch_size = max_batch_size
        self.kv = None
        self.steps = 0

    def execute(self, batch: Sequence[TextContext]) -> dict:
        self.steps += 1
        out = {}
        for c in batch:
            c.tokens.advance_processed()
            n = c.tokens.generated_length
            prompt = c.tokens.prompt
            eos = next(iter(c.eos_token_ids), None)
            tok = int(prompt[n]) if n < len(prompt) else (eos if eos is not None else int(prompt[-1]))
            c.update(tok)
            if n + 1 >= len(prompt) and not c.is_done:
                from ...pipelines.context import GenerationStatus

                c.status = GenerationStatus.END_OF_SEQUENCE
            out[c.request_id] = c.to_generation_output()
        return out

    def has_pending(self) -> bool:
        return False

    def release(self, request_id: str) -> None:
        pass
