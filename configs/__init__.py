"""Packaged YAML presets (resolved by name through ``importlib.resources``)."""
