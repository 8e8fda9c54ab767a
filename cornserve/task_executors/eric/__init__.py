"""Eric: the multimodal encoder executor (router -> engine -> tensor-parallel workers)."""
