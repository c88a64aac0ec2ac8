"""Training CLI (reference ``src/modeling/main.py``): ``python -m allie_b200.train.main <config.yaml>``
(under ``torchrun`` for data parallelism).  Loads the YAML, builds trainer / data / model, trains,
tests, cleans up."""
from __future__ import annotations

import sys

from ..config import load_config
from ..data import load_data
from ..models import initialize_model
from .trainer import Trainer


def main(argv: list[str] | None = None) -> None:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        raise SystemExit("usage: python -m allie_b200.train.main <config.yaml>   (under torchrun for several GPUs)")
    config = load_config(argv[0])
    trainer = Trainer(config, **config.trainer_config)
    trainer.save_config(config)
    tokenizer, (train_dataset, val_dataset, test_dataset) = load_data(**config.data_config)
    model = initialize_model(tokenizer, **config.model_config)
    trainer.setup_dataloaders(tokenizer, train_dataset, val_dataset, test_dataset)
    trainer.setup_model(model)
    trainer.train()
    if not trainer.stopped_early:        # a requested stop leaves right after its checkpoint; the requeued job resumes
        trainer.test()
    trainer.cleanup()


if __name__ == "__main__":
    main()
