"""External baselines of the reference registry: ``maia`` (lc0 with Maia weights over UCI) and
``gpt-3.5-turbo`` (OpenAI completions).  Both need things this package cannot ship (the lc0 binary
and weight files; network access and credentials), so they register themselves but raise a clear
error on construction when their dependency is missing (reference ``src/evaluation/decode.py:128-182,
661-731``)."""
from __future__ import annotations

import os

import torch

from ..data import Game
from ..evaluation.uci import EngineUnavailable, UCIEngine
from .strategies import DECODE_STRATEGIES, DecodeStrategy, ScoreResult


class Maia(DecodeStrategy):
    """Closest-rated Maia network (1100..1900), one node per move."""

    def __init__(self, model=None, tokenizer=None, sample=False, device=None, precision="float32",
                 maia_dir: str = "maia-weights", **kwargs):
        self.model, self.tokenizer, self.sample = model, tokenizer, sample
        self.engines: dict[int, UCIEngine] = {}
        for elo in range(1100, 2000, 100):
            w = os.path.join(maia_dir, f"maia-{elo}.pb.gz")
            if os.path.exists(w):
                self.engines[elo] = UCIEngine("lc0", args=[f"--weights={w}"])
        if not self.engines:
            raise EngineUnavailable("Maia needs the lc0 binary and maia-<elo>.pb.gz weights")

    def score_full(self, game: Game, legal_moves: list[str]) -> ScoreResult:
        elo = game.white_elo if game.board.turn else game.black_elo
        best = min(self.engines, key=lambda e: abs(e - (elo or 1500)))
        _, _, mv = self.engines[best].analyse(game.moves, nodes=1)
        probs = torch.zeros(len(legal_moves))
        probs[legal_moves.index(mv)] = 1.0
        return ScoreResult(probs, None, False)

    def cleanup(self) -> None:
        for e in self.engines.values():
            e.quit()


class GPT35Turbo(DecodeStrategy):
    def __init__(self, *a, **k):
        raise EngineUnavailable("the gpt-3.5-turbo baseline needs network access to the OpenAI API")


DECODE_STRATEGIES.setdefault("maia", Maia)
DECODE_STRATEGIES.setdefault("gpt-3.5-turbo", GPT35Turbo)
