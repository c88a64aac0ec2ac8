"""Rating statistics of a games JSONL: python src/data/compute-elo-stats.py games.jsonl"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from allie_b200.etl.dataset import main  # noqa: E402

if __name__ == "__main__":
    main(["elo-stats", *sys.argv[1:]])
