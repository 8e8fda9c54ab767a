"""Monolithic ("no fission") baseline executor."""
