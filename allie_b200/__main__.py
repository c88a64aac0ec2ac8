"""``python -m allie_b200 <command> [args]`` (installed as the ``allie`` console script): one front
for the command line tools of the package."""
from __future__ import annotations

import importlib
import sys

COMMANDS = {
    "build": ("allie_b200.build", "build_all", "compile the native libraries in-tree"),
    "train": ("allie_b200.train.main", "main", "train from a YAML config (under torchrun for several GPUs)"),
    "evaluate": ("allie_b200.evaluation.evaluate", "main", "score a games JSONL with a decode strategy"),
    "annotate": ("allie_b200.evaluation.annotate", "main", "add human move quality and move-type columns to a JSONL"),
    "serve": ("allie_b200.serve.server", "main", "move server of one system alias"),
    "pool": ("allie_b200.serve.pool", "main", "one move server per GPU behind the alias's port"),
    "uci": ("allie_b200.serve.uci", "main", "UCI engine in front of a running move server"),
    "stress-test": ("allie_b200.serve.stress_test", "main", "load test against a running move server"),
    "pgn": ("allie_b200.etl.pgn", "main", "PGN dump -> games JSONL"),
    "dataset": ("allie_b200.etl.dataset", "main", "sample / tokenize / concat / statistics of games files"),
}


def main(argv: list[str] | None = None) -> None:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help") or argv[0] not in COMMANDS:
        width = max(map(len, COMMANDS))
        lines = [f"  {name.ljust(width)}  {info[2]}" for name, info in COMMANDS.items()]
        print("usage: python -m allie_b200 <command> [args]\n\ncommands:\n" + "\n".join(lines))
        raise SystemExit(0 if argv and argv[0] in ("-h", "--help") else 2)
    module, func, _ = COMMANDS[argv[0]]
    fn = getattr(importlib.import_module(module), func)
    if argv[0] == "build":
        fn(force="--force" in argv[1:], verbose="-v" in argv[1:])
    else:
        fn(argv[1:])


if __name__ == "__main__":
    main()
