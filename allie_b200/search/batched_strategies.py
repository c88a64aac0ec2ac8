"""Decode strategies that answer many games per call.

The reference decodes one game at a time (``src/evaluation/decode.py:90-113``; its server handles
one request per accept, ``src/server/main.py:53-92``).  On a B200 one position is far too little
work for the device, so these strategies keep the reference's semantics per game and add
``decode_batch(games)``:

* :class:`BatchedPolicy` - one forward pass for all games (``policy-batched``).
* :class:`BatchedMCTSStrategy` / :class:`BatchedAdaptiveMCTS` - one search tree per game inside the
  C++ batched search (``csrc/mcts.cpp``); on a GPU the leaves of all trees are evaluated by the
  KV-cached evaluator in one CUDA-graph step per simulation, on the CPU by re-encoding through the
  plain runner (``mcts-batched``, ``adaptive-mcts-batched``).

``decode_full`` / ``score_full`` are the batch of one, so every strategy here is a drop-in entry of
the ``DECODE_STRATEGIES`` registry, the evaluation CLI and the move server.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..moves import NUM_CHESS_MOVES
from ..data import TIME_MEAN, TIME_STDEV, Game, apply_time_normalization, undo_time_normalization
from .strategies import DECODE_STRATEGIES, DecodeResult, DecodeStrategy, Policy, ScoreResult


def pick_move(strategy: DecodeStrategy, game: Game, legal: list[str], probs: torch.Tensor) -> str:
    """Sampling rule shared with ``DecodeStrategy.decode_full``: sample, take the arg-max, or decide by
    rating (arg-max iff the side to move is rated at least 2200 and more than 8 plies were played)."""
    if strategy.sample not in (True, False):
        assert strategy.sample == "rating-based"
        elo = game.white_elo if game.board.turn else game.black_elo
        sample = not (elo >= 2200 and len(game.board.move_stack) > 8)
    else:
        sample = strategy.sample
    return legal[int(probs.multinomial(1)[0]) if sample else int(probs.argmax())]


class BatchedPolicy(Policy):
    def score_batch(self, games: list[Game]) -> list[ScoreResult]:
        ev = self.runner.evaluate(list(games))
        out = []
        for i, g in enumerate(games):
            legal = g.legal_moves
            logits = ev.logits[i]
            ids = torch.tensor([self.tokenizer.token_to_id[m] for m in legal], dtype=torch.int64)
            move_logits = logits[ids]
            think = undo_time_normalization(float(ev.time[i])) if self.time_prediction else None
            raw = float(ev.value[i])
            pov = 1 if g.board.turn else -1
            resigned = bool(float(logits[self.tokenizer.resigned_token_id]) > float(move_logits.max())
                            and pov * raw < -0.9)
            all_probs = F.softmax(logits[:NUM_CHESS_MOVES] / self.temperature, dim=0)
            top_legal = self.tokenizer.tokens[int(all_probs.argmax())] in legal
            out.append(ScoreResult(F.softmax(move_logits / self.temperature, dim=0), think, resigned, all_probs,
                                   top_legal, float(all_probs[ids].sum()), raw))
        return out

    def decode_batch(self, games: list[Game]) -> list[DecodeResult]:
        return [DecodeResult(pick_move(self, g, g.legal_moves, s.legal_move_probabilities), s.think_time, s.resigned)
                for g, s in zip(games, self.score_batch(games))]


class BatchedMCTSStrategy(DecodeStrategy):
    """``mcts`` for up to ``n_trees`` games per call."""

    adaptive = False

    def init(self, n_trees: int = 64, n_sims: int = 50, depth_limit: int = 100, c_puct: float = 1.25,
             c_base: float = 19652.0, dummy_value_function: bool = False, kl_reg_solution: bool = True,
             anc_max: int = 128, legal_max: int = 224, max_nodes: int | None = None,
             use_graph: bool = True, **kwargs) -> None:
        from .batched import BatchedMCTS, KVStepEvaluator, RunnerStepEvaluator

        self.n_trees, self.n_sims, self.c_puct = n_trees, n_sims, c_puct
        most = self.max_sims()
        engine = getattr(self.runner, "engine", None)
        if engine is not None:
            # one KV slot per evaluated node of a tree, after the slots of the game so far
            nodes = max_nodes if max_nodes is not None else -(-(most + 2) // 64) * 64
            self.evaluator = KVStepEvaluator(engine, self.tokenizer, n_trees, anc_max, legal_max,
                                             max_prefix=self.tokenizer.max_length, max_nodes=nodes,
                                             use_graph=use_graph)
        else:
            self.evaluator = RunnerStepEvaluator(self.runner, self.tokenizer, n_trees, anc_max, legal_max)
        self.search = BatchedMCTS(self.tokenizer, self.evaluator, n_trees, n_sims=n_sims, c_puct=c_puct,
                                  c_base=c_base, depth_limit=depth_limit, kl_reg_solution=kl_reg_solution,
                                  dummy_value_function=dummy_value_function, anc_max=anc_max,
                                  legal_max=legal_max)

    def check(self) -> None:
        assert self.runner.has_value_head, "model does not provide a value prediction"

    def max_sims(self) -> int:
        return self.n_sims

    def _budget(self):
        return self.n_sims, None

    def score_batch(self, games: list[Game]) -> list[ScoreResult]:
        out: list[ScoreResult] = []
        n_sims, c_puct_fn = self._budget()
        for lo in range(0, len(games), self.n_trees):
            chunk = list(games[lo:lo + self.n_trees])
            for g, r in zip(chunk, self.search.search(chunk, n_sims=n_sims, c_puct_per_tree=c_puct_fn)):
                by_move = dict(zip(r.legal_moves, r.policy.tolist()))
                probs = torch.tensor([by_move[m] for m in g.legal_moves], dtype=torch.float32)
                out.append(ScoreResult(probs, r.think_time, r.resigned, white_advantage=r.root_value))
        return out

    def score_full(self, game: Game, legal_moves: list[str]) -> ScoreResult:
        return self.score_batch([game])[0]

    def decode_batch(self, games: list[Game]) -> list[DecodeResult]:
        return [DecodeResult(pick_move(self, g, g.legal_moves, s.legal_move_probabilities), s.think_time, s.resigned)
                for g, s in zip(games, self.score_batch(games))]

    def run_stats(self) -> dict:
        return {"total_rollouts": self.search.total_rollouts, "positions_evaluated": self.evaluator.positions,
                **{f"seconds_{k}": round(v, 4) for k, v in self.search.phase_seconds.items()}}


class BatchedAdaptiveMCTS(BatchedMCTSStrategy):
    """``adaptive-mcts`` for many games per call: every tree gets the budget its own root's think-time
    prediction (or the human's actual move time) asks for, and its own rescaled ``c_puct``."""

    adaptive = True

    def init(self, mean_n_sims: int = 50, scale_c_puct: bool = True, use_human_move_time: bool = False,
             conversion_strategy: str = "linear", **kwargs) -> None:
        assert conversion_strategy in ("linear", "binary")
        self.mean_n_sims, self.scale_c_puct = mean_n_sims, scale_c_puct
        self.use_human_move_time, self.conversion_strategy = use_human_move_time, conversion_strategy
        kwargs.pop("n_sims", None)
        super().init(n_sims=mean_n_sims, **kwargs)

    def max_sims(self) -> int:
        return 200

    def convert_time_to_sims(self, time_encoding: float) -> int:
        if self.conversion_strategy == "linear":
            n = round(self.mean_n_sims * TIME_STDEV / TIME_MEAN * time_encoding + self.mean_n_sims)
        else:
            n = 0 if time_encoding < 0 else self.mean_n_sims
        return min(max(n, 0), 200)

    def _budget(self):
        def sims(time_encoding: float, game: Game) -> int:
            if self.use_human_move_time:
                assert game.next_move_seconds is not None, "missing human move seconds"
                time_encoding = apply_time_normalization(game.next_move_seconds)
            return self.convert_time_to_sims(time_encoding)

        def c_puct(n_sims: int) -> float:
            if not self.scale_c_puct or n_sims <= 0:
                return self.c_puct
            return self.c_puct * math.sqrt(self.mean_n_sims) / math.sqrt(n_sims)

        return sims, c_puct


def decode_batch(strategy: DecodeStrategy, games: list[Game]) -> list[DecodeResult]:
    """``strategy.decode_batch(games)`` when the strategy has one, else one ``decode_full`` per game."""
    if hasattr(strategy, "decode_batch"):
        return strategy.decode_batch(list(games))
    return [strategy.decode_full(g) for g in games]


DECODE_STRATEGIES.setdefault("policy-batched", BatchedPolicy)
DECODE_STRATEGIES.setdefault("mcts-batched", BatchedMCTSStrategy)
DECODE_STRATEGIES.setdefault("adaptive-mcts-batched", BatchedAdaptiveMCTS)
