"""Games JSONL -> flat uint32 token stream: python src/data/create-np-dataset.py train.jsonl train.bin"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from allie_b200.etl.dataset import main  # noqa: E402

if __name__ == "__main__":
    main(["tokenize", *sys.argv[1:]])
