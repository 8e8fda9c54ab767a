"""Utilities: checkpoint resolution and safetensors loading, timing helpers."""
