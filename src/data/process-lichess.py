"""PGN dump -> games JSONL: python src/data/process-lichess.py dump.pgn.zst games.jsonl [--workers N]"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from allie_b200.etl.pgn import main  # noqa: E402

if __name__ == "__main__":
    main()
