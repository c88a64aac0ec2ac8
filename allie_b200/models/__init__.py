"""Model construction (``initialize_model`` mirrors reference ``src/modeling/model.py:155-198``)."""
from __future__ import annotations

import logging
import os
from typing import Any

import torch

from ..config import ModelConfig, resolve_model_config
from .oracle import (CausalLMWithControlToken, CausalLMWithRegressionHead, GPT2LM)

logger = logging.getLogger(__name__)

Model = GPT2LM | CausalLMWithControlToken | CausalLMWithRegressionHead


def _load_pretrained_body(model: GPT2LM, base_model: str) -> bool:
    """Copies GPT-2 body weights (everything except the token embedding / LM head) from a local
    HF checkpoint directory (or the local Hugging Face cache of ``base_model``) and re-draws ``wte`` from N(mean, std) of the pretrained embedding
    (reference ``model.py:175-188``).  Returns False when no local weights exist."""
    import glob

    # a local checkpoint directory, or the Hugging Face cache of a model fetched earlier
    # (<HF_HOME>/hub/models--<name>/snapshots/<revision>/)
    hub = os.path.join(os.environ.get("HF_HOME", os.path.join(os.path.expanduser("~"), ".cache", "huggingface")), "hub")
    dirs = [base_model] + sorted(glob.glob(os.path.join(hub, "models--" + base_model.replace("/", "--"), "snapshots", "*")))
    cand = [os.path.join(d, n) for d in dirs for n in ("model.safetensors", "pytorch_model.bin")]
    path = next((p for p in cand if os.path.exists(p)), None)
    if path is None:
        return False
    logger.info("loading pretrained GPT-2 body from %s", path)
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file

        sd = load_file(path)
    else:
        sd = torch.load(path, map_location="cpu")
    sd = {k.removeprefix("transformer.") if not k.startswith("lm_head") else k: v for k, v in sd.items()}
    wte = sd.get("wte.weight")
    body = {"transformer." + k: v for k, v in sd.items()
            if k not in ("wte.weight", "lm_head.weight") and not k.endswith(".attn.bias")
            and not k.endswith(".attn.masked_bias")}
    _, unexpected = model.load_state_dict(body, strict=False)
    if unexpected:
        logger.warning("unexpected pretrained keys: %s", unexpected[:5])
    if wte is not None:
        torch.nn.init.normal_(model.transformer.wte.weight, wte.float().mean().item(),
                              wte.float().std().item())
    return True


def load_model_state(model, state_dict: dict) -> None:
    """``model.load_state_dict`` for checkpoints of the reference or of this framework: strict about
    parameters, tolerant of the causal-mask buffers (``attn.bias`` / ``attn.masked_bias``) that
    older Hugging Face GPT-2 versions wrote into their state dicts, and of a ``module.`` /
    ``_orig_mod.`` prefix left by a DDP or ``torch.compile`` wrapper."""
    clean = {}
    for k, v in state_dict.items():
        for prefix in ("module.", "_orig_mod."):
            while k.startswith(prefix):
                k = k[len(prefix):]
        if k.endswith(".attn.bias") or k.endswith(".attn.masked_bias"):
            continue
        clean[k] = v
    model.load_state_dict(clean)


def initialize_model(tokenizer, base_model: str, use_control_token: bool = False,
                     use_regression_head: bool = False, use_pretrained: bool = False,
                     lm_loss_coef: float = 1.0, value_loss_coef: float = 1.0,
                     **overrides: Any) -> Model:
    cfg: ModelConfig = resolve_model_config(
        base_model, vocab_size=len(tokenizer), bos_token_id=tokenizer.bos_token_id,
        eos_token_id=tokenizer.eos_token_id, pad_token_id=tokenizer.pad_token_id, **overrides)
    model: Any = GPT2LM(cfg)
    if use_pretrained:
        if not _load_pretrained_body(model, base_model):
            logger.warning("use_pretrained: no local GPT-2 weights for %r (no network access); "
                           "continuing from random initialisation", base_model)
    if use_control_token:
        model = CausalLMWithControlToken(model)
    if use_regression_head:
        model = CausalLMWithRegressionHead(model, lm_loss_coef, value_loss_coef)
    return model


def unwrap(model) -> tuple[GPT2LM, CausalLMWithControlToken | None, CausalLMWithRegressionHead | None]:
    """(decoder, control wrapper or None, regression wrapper or None)."""
    reg = model if isinstance(model, CausalLMWithRegressionHead) else None
    inner = reg.model if reg is not None else model
    ctrl = inner if isinstance(inner, CausalLMWithControlToken) else None
    lm = ctrl.model if ctrl is not None else inner
    assert isinstance(lm, GPT2LM)
    return lm, ctrl, reg
