"""ELO-balanced sample with train / val / test split: python src/data/sample-lichess.py games.jsonl out_prefix"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from allie_b200.etl.dataset import main  # noqa: E402

if __name__ == "__main__":
    main(["sample", *sys.argv[1:]])
