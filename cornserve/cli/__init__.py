"""Command-line client (``python -m cornserve.cli`` / ``cornserve``)."""
