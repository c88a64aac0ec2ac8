from allie_b200.train.trainer import Trainer  # noqa: F401
