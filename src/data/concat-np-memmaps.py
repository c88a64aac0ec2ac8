"""Concatenates token streams: python src/data/concat-np-memmaps.py a.bin b.bin out.bin"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from allie_b200.etl.dataset import main  # noqa: E402

if __name__ == "__main__":
    main(["concat", *sys.argv[1:]])
