"""API-side pipeline helpers: token generator, incremental detokenizer, echo generator."""
