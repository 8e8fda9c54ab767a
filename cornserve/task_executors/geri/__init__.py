"""Geri: the multimodal generator executor (images in batches, audio as a stream)."""
