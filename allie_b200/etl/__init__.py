"""Offline data preparation (reference ``src/data/*.py``): PGN -> JSONL, ELO-balanced sampling,
tokenisation into one flat ``uint32`` stream, statistics and synthetic games."""
