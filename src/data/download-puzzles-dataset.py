"""Samples mate-in-k puzzles and fetches their source games: python src/data/download-puzzles-dataset.py lichess_db_puzzle.csv out_dir"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from allie_b200.etl.dataset import main  # noqa: E402

if __name__ == "__main__":
    main(["puzzles", *sys.argv[1:], "--download"])
