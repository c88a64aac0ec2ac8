"""Logging set-up: stdout at INFO, ``log.txt`` at INFO and ``debug.txt`` at DEBUG in the run
directory, format ``time - logger - level - message`` (reference ``src/modeling/utils.py:20-41``)."""
from __future__ import annotations

import logging
import os
import sys

_FORMAT = "%(asctime)s - %(name)s - %(levelname)s - %(message)s"
_DATEFMT = "%m-%d %H:%M"


def setup_logging(output_dir: str | None = None, file: bool = False) -> None:
    root = logging.getLogger()
    root.setLevel(logging.DEBUG)
    fmt = logging.Formatter(_FORMAT, _DATEFMT)
    if not any(getattr(h, "_allie", None) == "stdout" for h in root.handlers):
        h = logging.StreamHandler(sys.stdout)
        h.setLevel(logging.INFO)
        h.setFormatter(fmt)
        h._allie = "stdout"
        root.addHandler(h)
    if file and output_dir is not None:
        for name, level in (("log.txt", logging.INFO), ("debug.txt", logging.DEBUG)):
            path = os.path.abspath(os.path.join(output_dir, name))
            if any(getattr(h, "baseFilename", None) == path for h in root.handlers):
                continue
            fh = logging.FileHandler(path)
            fh.setLevel(level)
            fh.setFormatter(fmt)
            root.addHandler(fh)
