"""Serving benchmark harness (open-loop load generator and latency metrics)."""
