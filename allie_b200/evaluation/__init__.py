"""Evaluation CLI and engine-based move-quality metrics (reference ``src/evaluation``)."""
