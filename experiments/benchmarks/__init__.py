"""Measurement grids (``python -m stacr benchmarks list|run``)."""
