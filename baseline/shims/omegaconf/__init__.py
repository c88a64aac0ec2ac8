"""Stand-in for the small part of ``omegaconf`` the reference trainer imports (the real package is
not installed on this machine).  Used only by the reference benchmark arm."""
import yaml


class DictConfig(dict):
    def __getattr__(self, k):
        try:
            v = self[k]
        except KeyError as e:
            raise AttributeError(k) from e
        return DictConfig(v) if isinstance(v, dict) and not isinstance(v, DictConfig) else v


class OmegaConf:
    @staticmethod
    def load(path):
        with open(path) as f:
            return DictConfig(yaml.safe_load(f))

    @staticmethod
    def create(d):
        return DictConfig(d)

    @staticmethod
    def to_container(cfg):
        return dict(cfg)

    @staticmethod
    def save(cfg, path):
        with open(path, "w") as f:
            yaml.safe_dump(dict(cfg), f)
