"""Own LLM executor (replaces the reference's external vLLM fork): paged KV cache, continuous
batching, M-RoPE, encoder-embedding injection, hidden-state forwarding, OpenAI-compatible server."""
