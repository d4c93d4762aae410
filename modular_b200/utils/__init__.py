"""Small shared helpers (measured hardware peaks, clock sampling, logging glue)."""
