"""Model runners: how the decode strategies get (policy logits, value, think time) for positions.

* :class:`TorchRunner` - the plain-PyTorch model (CPU path, ground truth).
* :class:`EngineRunner` - the sm_100a engine; a batch of games is collated on the host, runs as one
  forward pass of hand-scheduled kernels, and only the last-position rows come back, in a single
  device-to-host copy (the reference pays three ``.item()`` synchronisations per position,
  ``src/evaluation/decode.py:204-218``).
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass

import torch

from ..data import Game, UCITokenizer
from ..models import unwrap


@dataclass
class Evaluation:
    logits: torch.Tensor      # [n, vocab] float32, host
    value: torch.Tensor       # [n] float32 (white advantage, tanh range), host
    time: torch.Tensor        # [n] float32 (normalised think time), host


# model -> the engine that runs it (one engine per model: its parameters live in the engine's arenas).
# Kept beside the model, not as an attribute of it, so copying or pickling a model never drags the
# engine (arenas, streams, buffers) along.
_ENGINES: "weakref.WeakKeyDictionary" = weakref.WeakKeyDictionary()


def engine_of(model):
    return _ENGINES.get(model)


def attach_engine(model, engine) -> None:
    _ENGINES[model] = engine


class ModelRunner:
    has_value_head = True

    def evaluate(self, games: list[Game]) -> Evaluation:
        raise NotImplementedError


def _last_index(batch) -> torch.Tensor:
    return batch["attention_mask"].sum(-1).long() - 1


class TorchRunner(ModelRunner):
    def __init__(self, model, tokenizer: UCITokenizer, device: str = "cpu"):
        self.model, self.tokenizer, self.device = model, tokenizer, device
        self.has_value_head = unwrap(model)[2] is not None
        self.calls = 0

    @torch.no_grad()
    def evaluate(self, games: list[Game]) -> Evaluation:
        self.model.eval()
        self.calls += 1
        batch = self.tokenizer.pad_and_collate(list(games))
        batch = {k: v.to(self.device) for k, v in batch.items()}
        out = self.model(**batch)
        idx = _last_index(batch)
        rows = torch.arange(len(games), device=idx.device)
        n = len(games)
        value = out["value_logits"][rows, idx].float().cpu() if "value_logits" in out else torch.zeros(n)
        time = out["time_logits"][rows, idx].float().cpu() if "time_logits" in out else torch.zeros(n)
        return Evaluation(out["logits"][rows, idx].float().cpu(), value, time)


class EngineRunner(ModelRunner):
    def __init__(self, model, tokenizer: UCITokenizer, device: str = "cuda"):
        from ..models.engine import B200Engine

        self.tokenizer = tokenizer
        eng = engine_of(model)
        if eng is None:
            eng = B200Engine(model, device)
            attach_engine(model, eng)
        self.engine = eng
        self.has_value_head = eng.reg is not None
        self.calls = 0

    @torch.no_grad()
    def evaluate(self, games: list[Game]) -> Evaluation:
        self.calls += 1
        batch = self.tokenizer.pad_and_collate(list(games), return_labels=False)
        out = self.engine.evaluate_batch(batch, with_loss=False)
        idx = _last_index(batch).to(self.engine.device)
        rows = torch.arange(len(games), device=idx.device)
        V = out["logits"].size(-1)
        packed = torch.empty(len(games), V + 2, dtype=torch.float32, device=idx.device)
        packed[:, :V] = out["logits"][rows, idx].float()
        if self.has_value_head:
            packed[:, V] = out["value_logits"][rows, idx]
            packed[:, V + 1] = out["time_logits"][rows, idx]
        else:
            packed[:, V:] = 0
        host = packed.cpu()          # the one device-to-host copy of this evaluation
        return Evaluation(host[:, :V], host[:, V], host[:, V + 1])


PRECISIONS = (None, "float32", "bfloat16")


def make_runner(model, tokenizer: UCITokenizer, device: str, precision: str | None = None) -> ModelRunner:
    """Who evaluates positions.  On a CUDA device: ``precision`` None or ``"bfloat16"`` -> the
    sm_100a engine (bf16 tensor-core math, fp32 accumulation and residual stream); ``"float32"`` ->
    the plain PyTorch model in fp32 on the GPU with TF32 matrix multiplications, which is how the
    reference's evaluation CLI runs its model (``src/evaluation/evaluate.py:249``,
    ``src/evaluation/decode.py:58-81``), for numbers that are comparable with it weight for weight.
    On the CPU everything is fp32."""
    if precision not in PRECISIONS:
        raise ValueError(f"precision must be one of 'float32', 'bfloat16' (or None for the device's default), not {precision!r}")
    if str(device).startswith("cuda") and torch.cuda.is_available():
        if precision == "float32":
            torch.backends.cuda.matmul.allow_tf32 = True
            torch.backends.cudnn.allow_tf32 = True
            # a model whose parameters already live in an engine's arenas keeps them there: they are
            # ordinary fp32 tensors on the device (views of the master arena), shared with the engine
            if engine_of(model) is None:
                model = model.float().to(device)
            return TorchRunner(model, tokenizer, device)
        return EngineRunner(model, tokenizer, device)
    return TorchRunner(model, tokenizer, "cpu")
