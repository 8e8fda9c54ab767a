"""Model definitions built on :mod:`cornserve.ops` (encoders, LLM decoders, generators)."""
