"""Command-line client (``python -m cornserve_b200.cli`` / ``cornserve``)."""
