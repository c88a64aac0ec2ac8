"""Metric sink: forwards to Weights & Biases when it is importable and allowed, and always mirrors
every row to the debug log and, when a path is given, to a ``metrics.jsonl`` file (one JSON object
per line).  The reference logs ``iter, lr, train/loss, val/*_loss, test/loss`` to the wandb project
``chess-lm`` with ``resume="allow"`` and falls back to offline mode when the service is unreachable
(``src/modeling/trainer.py:88-106,254-261``)."""
from __future__ import annotations

import json
import logging
import os

logger = logging.getLogger(__name__)


class MetricsSink:
    def __init__(self, enabled: bool, project: str, name=None, run_id=None, config=None, path: str | None = None):
        self.run = None
        self.path = path                      # every row is also appended here as one JSON line
        self.history: list[dict] = []
        if not enabled or os.environ.get("ALLIE_NO_WANDB") == "1":
            return
        try:
            import wandb

            mode = os.environ.get("WANDB_MODE")
            try:
                if mode is None and not os.environ.get("WANDB_API_KEY"):
                    raise RuntimeError("no credentials: go offline")
                self.run = wandb.init(project=project, name=name, id=run_id, resume="allow", config=config)
            except Exception:
                logger.warning("wandb is offline")
                self.run = wandb.init(project=project, name=name, id=run_id, resume="allow",
                                      config=config, mode=mode or "offline")
        except Exception as e:  # wandb missing or unusable: metrics stay in the log files
            logger.warning(f"wandb unavailable ({type(e).__name__}); metrics go to the log only")
            self.run = None

    def log(self, row: dict) -> None:
        self.history.append(row)
        logger.debug("metrics " + json.dumps(row))
        if self.path is not None:
            try:
                with open(self.path, "a") as f:
                    f.write(json.dumps(row) + "\n")
            except OSError as e:
                logger.warning(f"cannot write {self.path}: {e}")
                self.path = None
        if self.run is not None:
            try:
                self.run.log(row)
            except Exception:
                pass

    def finish(self) -> None:
        if self.run is not None:
            try:
                self.run.finish()
            except Exception:
                pass
            self.run = None
