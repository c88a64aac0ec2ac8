"""Helpers of the reference's ``modeling.utils`` (``src/modeling/utils.py:20-122``)."""
import logging

import torch

from allie_b200.models.engine import partition_parameter_names
from allie_b200.train.trainer import count_params, to_device  # noqa: F401
from allie_b200.utils.logging import setup_logging  # noqa: F401

logger = logging.getLogger(__name__)


def seed_everything(seed: int) -> None:
    """Deliberately seeds nothing (a requeued job must not replay its data order); only turns on
    cuDNN autotuning, as the reference does."""
    torch.backends.cudnn.benchmark = True
    logger.info(f"not setting manual seed to {seed} due to dataloader behavior after requeue")


def partition_model_parameters(model):
    decay, no_decay = partition_parameter_names(model)
    params = dict(model.named_parameters())
    return [params[n] for n in decay], [params[n] for n in no_decay]


def cycle_dataloader(dataloader, device: str):
    epoch = 0
    while True:
        sampler = getattr(dataloader, "sampler", None)
        if hasattr(sampler, "set_epoch"):
            sampler.set_epoch(epoch)
        for batch in dataloader:
            yield to_device(batch, device)
        epoch += 1
