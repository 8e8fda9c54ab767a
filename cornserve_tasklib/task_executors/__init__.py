"""Execution descriptors of the built-in unit tasks."""
