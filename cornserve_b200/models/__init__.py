"""Model definitions built on :mod:`cornserve_b200.ops` (encoders, LLM decoders, generators)."""
