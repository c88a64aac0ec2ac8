"""Random legal games as JSONL: python src/data/random-games.py out.jsonl [--n 1000]"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from allie_b200.etl.dataset import main  # noqa: E402

if __name__ == "__main__":
    main(["random-games", *sys.argv[1:]])
