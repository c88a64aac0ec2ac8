"""Configuration: YAML files with the three sections ``trainer_config`` / ``data_config`` /
``model_config`` (reference ``src/modeling/main.py:11-19``), an attribute-style mapping that can be
splatted into keyword arguments, and the table that resolves ``base_model`` names to GPT-2
shapes without any network access (the reference asks the HF hub, ``src/modeling/model.py:165``).
"""
from __future__ import annotations

import copy
from dataclasses import asdict, dataclass, field
from typing import Any, Mapping

import yaml


class Config(dict):
    """dict with attribute access, recursive; behaves like the small part of
    ``omegaconf.DictConfig`` the reference uses (``cfg.section``, ``**cfg.section``)."""

    def __init__(self, data: Mapping | None = None):
        super().__init__()
        for k, v in (data or {}).items():
            self[k] = v

    def __setitem__(self, key, value):
        if isinstance(value, Mapping) and not isinstance(value, Config):
            value = Config(value)
        super().__setitem__(key, value)

    def __getattr__(self, key):
        try:
            return self[key]
        except KeyError as e:
            raise AttributeError(key) from e

    def __setattr__(self, key, value):
        self[key] = value

    def to_container(self) -> dict:
        return {k: (v.to_container() if isinstance(v, Config) else copy.deepcopy(v))
                for k, v in self.items()}


def _fix_scalars(node):
    # PyYAML reads "1e-5" (no dot) as a string; the reference's loader reads it as a float.
    if isinstance(node, dict):
        return {k: _fix_scalars(v) for k, v in node.items()}
    if isinstance(node, list):
        return [_fix_scalars(v) for v in node]
    if isinstance(node, str):
        try:
            return float(node) if any(c in node for c in "eE.") and node.strip()[0] in "+-.0123456789" else node
        except ValueError:
            return node
    return node


def _merge(base: dict, over: dict) -> dict:
    out = dict(base)
    for k, v in over.items():
        out[k] = _merge(out[k], v) if isinstance(v, dict) and isinstance(out.get(k), dict) else v
    return out


def load_config(path: str) -> Config:
    """Reads a YAML config.  A top-level ``inherit: other.yaml`` key (path relative to the file)
    loads that file first and lays this file's keys over it, section by section, so that an
    ablation states only what it changes; files without the key load exactly as written."""
    with open(path) as f:
        data = _fix_scalars(yaml.safe_load(f) or {})
    parent = data.pop("inherit", None)
    if parent is not None:
        import os

        base = load_config(os.path.join(os.path.dirname(os.path.abspath(path)), parent))
        data = _merge(base.to_container(), data)
    return Config(data)


def save_config(cfg: Mapping, path: str) -> None:
    data = cfg.to_container() if isinstance(cfg, Config) else dict(cfg)
    with open(path, "w") as f:
        yaml.safe_dump(data, f, sort_keys=False)


# GPT-2 family shapes (the public OpenAI GPT-2 configurations).
BASE_MODELS: dict[str, dict[str, int]] = {
    "gpt2": dict(n_layer=12, n_embd=768, n_head=12),
    "gpt2-medium": dict(n_layer=24, n_embd=1024, n_head=16),
    "gpt2-large": dict(n_layer=36, n_embd=1280, n_head=20),
    "gpt2-xl": dict(n_layer=48, n_embd=1600, n_head=25),
}


@dataclass
class ModelConfig:
    vocab_size: int = 2048
    n_positions: int = 1024
    n_embd: int = 1024
    n_layer: int = 24
    n_head: int = 16
    n_inner: int | None = None
    activation_function: str = "gelu_new"
    resid_pdrop: float = 0.1
    embd_pdrop: float = 0.1
    attn_pdrop: float = 0.1
    layer_norm_epsilon: float = 1e-5
    initializer_range: float = 0.02
    norm_type: str = "layernorm"          # or "rmsnorm"
    bos_token_id: int | None = None
    eos_token_id: int | None = None
    pad_token_id: int | None = None
    # mixture-of-experts extension (0 experts = dense)
    num_experts: int = 0
    moe_top_k: int = 2
    moe_ffn: int | None = None
    moe_layer_freq: int = 3               # every k-th block is MoE (block index % k == k-1)
    aux_loss_coef: float = 0.01
    capacity_factor: float = 2.0
    # expert parallelism at construction time: build only experts [ep_rank*E/ep_world, ...) per rank
    ep_world: int = 1
    ep_rank: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def ffn_dim(self) -> int:
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    def is_moe_layer(self, i: int) -> bool:
        return self.num_experts > 0 and (i % self.moe_layer_freq) == self.moe_layer_freq - 1

    def to_dict(self) -> dict:
        return asdict(self)


def resolve_model_config(base_model: str, **overrides: Any) -> ModelConfig:
    """``base_model`` is a GPT-2 family name, or a directory / json file holding a HF-style
    ``config.json``; extra keys override fields (this is how the reference reaches arbitrary
    shapes: unknown ``model_config`` keys become HF config overrides, ``model.py:163-172``)."""
    import json
    import os

    fields = dict()
    if base_model in BASE_MODELS:
        fields.update(BASE_MODELS[base_model])
    else:
        path = base_model
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        if not os.path.exists(path):
            raise ValueError(f"unknown base_model {base_model!r}: not one of {sorted(BASE_MODELS)} "
                             "and not a local config")
        with open(path) as f:
            fields.update(json.load(f))
    fields.update(overrides)
    known = ModelConfig.__dataclass_fields__.keys()
    cfg = ModelConfig(**{k: v for k, v in fields.items() if k in known and k != "extra"})
    cfg.extra = {k: v for k, v in fields.items() if k not in known}
    assert cfg.n_embd % cfg.n_head == 0
    return cfg
