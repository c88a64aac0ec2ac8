"""Decode strategies with the reference semantics (``src/evaluation/decode.py``): ``Policy``,
``ActionValue``, ``MCTS`` and ``AdaptiveMCTS`` behind the ``DecodeStrategy`` interface
(``decode`` / ``decode_full`` / ``score_full`` / ``run_stats`` / ``cleanup``) and the
``DECODE_STRATEGIES`` registry.

What is kept exactly: legal-move softmax with temperature, think time = de-normalised time head,
the resign rule (resign-token logit above every legal move and side-to-move value < -0.9), the
"rating-based" sampling switch (argmax iff ELO >= 2200 and more than 8 plies), PUCT with
``c_base`` / ``c_puct``, values from the parent's point of view, eager child creation in legal-move
order with first-maximum tie-breaking, terminal values (0 draw / +1 mate delivered), the second root
evaluation, the KL-regularised policy solved by bisection to rtol 1e-3, and the time-adaptive
simulation budget with its ``c_puct`` rescaling.

What differs is how positions reach the network.  The strategies talk to a *runner*
(:mod:`allie_b200.search.runner`): the plain runner re-encodes whole games like the reference; the
cached runner keeps the keys/values of everything a search tree has already seen on the GPU and
evaluates whole batches of leaves in one step.  ``MCTS`` here is the sequential statement of the
algorithm (and the oracle for the batched C++ search in :mod:`allie_b200.search.batched`).
"""
from __future__ import annotations

import math
from abc import ABC
from dataclasses import dataclass
from typing import Any, Optional, Type

import torch
import torch.nn.functional as F

from ..data import (TIME_MEAN, TIME_STDEV, Game, UCITokenizer, apply_time_normalization,
                    undo_time_normalization)
from ..moves import NUM_CHESS_MOVES
from .runner import ModelRunner, make_runner


@dataclass(frozen=True)
class DecodeResult:
    move: str
    think_time: float | None
    resigned: bool


@dataclass(frozen=True)
class ScoreResult:
    legal_move_probabilities: torch.Tensor
    think_time: float | None = None
    resigned: bool | None = None
    all_move_probabilities: torch.Tensor | None = None
    top_move_legal: bool | None = None
    sampled_move_legal: float | None = None
    white_advantage: float | None = None


class DecodeStrategy(ABC):
    def __init__(self, model, tokenizer: UCITokenizer, sample: bool | str = False,
                 device: Optional[str] = None, precision: str | None = None, runner: ModelRunner | None = None,
                 **kwargs: Any):
        """``precision``: ``"float32"`` (what the reference's evaluation passes) runs the plain
        PyTorch model in fp32 / TF32, on the GPU too; ``"bfloat16"`` or None runs the sm_100a engine
        on a CUDA device (see :func:`allie_b200.search.runner.make_runner`)."""
        self.model = model
        self.tokenizer = tokenizer
        self.sample = sample
        self.device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.precision = precision
        self.runner = runner if runner is not None else make_runner(model, tokenizer, self.device, precision)
        self.init(**kwargs)
        self.check()

    def init(self, *args, **kwargs) -> None: ...

    def check(self) -> None: ...

    def decode(self, game: Game) -> str:
        return self.decode_full(game).move

    def decode_full(self, game: Game) -> DecodeResult:
        legal = game.legal_moves
        score = self.score_full(game, legal)
        probs = score.legal_move_probabilities
        if self.sample not in (True, False):
            assert self.sample == "rating-based"
            elo = game.white_elo if game.board.turn else game.black_elo
            sample = not (elo >= 2200 and len(game.board.move_stack) > 8)
        else:
            sample = self.sample
        choice = int(probs.multinomial(1)[0]) if sample else int(probs.argmax())
        return DecodeResult(legal[choice], score.think_time, score.resigned)

    def score_full(self, game: Game, legal_moves: list[str]) -> ScoreResult:
        raise NotImplementedError

    def run_stats(self) -> dict:
        return {}

    def cleanup(self) -> None: ...


class Policy(DecodeStrategy):
    def init(self, temperature: float = 1.0, time_prediction: bool = True) -> None:
        self.temperature = max(temperature, 1e-5)
        self.time_prediction = time_prediction

    def score_full(self, game: Game, legal_moves: list[str]) -> ScoreResult:
        ev = self.runner.evaluate([game])
        logits = ev.logits[0]
        ids = torch.tensor([self.tokenizer.token_to_id[m] for m in legal_moves], dtype=torch.int64)
        move_logits = logits[ids]
        think_time = undo_time_normalization(float(ev.time[0])) if self.time_prediction else None
        raw_value = float(ev.value[0])
        pov = 1 if game.board.turn else -1
        value = pov * raw_value
        resigned = bool(float(logits[self.tokenizer.resigned_token_id]) > float(move_logits.max()) and value < -0.9)
        all_probs = F.softmax(logits[:NUM_CHESS_MOVES] / self.temperature, dim=0)
        top_legal = self.tokenizer.tokens[int(all_probs.argmax())] in legal_moves
        return ScoreResult(F.softmax(move_logits / self.temperature, dim=0), think_time, resigned, all_probs,
                           top_legal, float(all_probs[ids].sum()), raw_value)


class ActionValue(Policy):
    """One-ply value search: play the move whose resulting position the value head likes best."""

    def init(self, batch_size: int = 16, **kwargs) -> None:
        super().init(**kwargs)
        self.batch_size = batch_size

    def score_full(self, game: Game, legal_moves: list[str]) -> ScoreResult:
        base = super().score_full(game, legal_moves)
        children = [game.make_move(m) for m in legal_moves]
        pov = 1 if game.board.turn else -1
        vals: list[float] = []
        for i in range(0, len(children), self.batch_size):
            ev = self.runner.evaluate(children[i:i + self.batch_size])
            vals.extend((pov * ev.value).tolist())
        probs = torch.zeros(len(legal_moves))
        probs[max(range(len(vals)), key=vals.__getitem__)] = 1.0
        return ScoreResult(probs, base.think_time, base.resigned)


class MCTSNode:
    __slots__ = ("prior", "children", "visit_count", "value_sum", "game", "_legal")

    def __init__(self, prior: float, game: Game):
        self.prior = prior
        self.children: dict[str, MCTSNode] = {}
        self.visit_count = 0
        self.value_sum = 0.0
        self.game = game
        self._legal = None

    @property
    def board(self):
        return self.game.board

    @property
    def legal_moves(self) -> list[str]:
        if self._legal is None:
            self._legal = self.game.legal_moves
        return self._legal

    def expanded(self) -> bool:
        return len(self.children) > 0

    def value(self) -> float:
        return self.value_sum / self.visit_count if self.visit_count else 0.0


def kl_regularized_policy(priors: torch.Tensor, values: torch.Tensor, visits: torch.Tensor,
                          c_puct: float) -> torch.Tensor:
    """pi_bar = lambda_N * prior / (alpha - q), alpha by bisection until the mass is 1 within
    rtol 1e-3 (reference decode.py:438-467)."""
    total = float(visits.sum())
    lam = c_puct * total / (len(visits) + total)
    a_min = (values + lam * priors).max()
    a_max = (values + lam).max()
    while True:
        alpha = (a_min + a_max) / 2
        pi = lam * priors / (alpha - values)
        s = pi.sum()
        if s > 1.0:
            a_min = alpha
        else:
            a_max = alpha
        if torch.isclose(s, torch.tensor(1.0), rtol=1e-3) or torch.isclose(a_min, a_max, rtol=1e-3):
            return pi / s


def kl_regularized_policy_np(priors, values, visits, c_puct: float):
    """The same bisection in float32 NumPy arithmetic (one tree costs tens of microseconds instead
    of the better part of a millisecond of tiny tensor operations; the batched search calls it once
    per tree and move).  Same update rule, same two stopping tests as :func:`kl_regularized_policy`."""
    import numpy as np

    f32 = np.float32
    priors = np.asarray(priors, dtype=f32)
    values = np.asarray(values, dtype=f32)
    total = float(np.asarray(visits, dtype=f32).sum())
    lam = f32(c_puct * total / (len(priors) + total))
    a_min = (values + lam * priors).max()
    a_max = (values + lam).max()
    one, rtol, atol = f32(1.0), 1e-3, 1e-8
    while True:
        alpha = (a_min + a_max) / f32(2)
        pi = lam * priors / (alpha - values)
        s = pi.sum(dtype=f32)
        if s > one:
            a_min = alpha
        else:
            a_max = alpha
        # torch.isclose(a, b): |a - b| <= atol + rtol * |b|
        if abs(float(s) - 1.0) <= atol + rtol * 1.0 or abs(float(a_min) - float(a_max)) <= atol + rtol * abs(float(a_max)):
            return pi / s


class MCTS(Policy):
    def init(self, n_sims: int = 50, depth_limit: int = 100, c_puct: float = 1.25, c_base: float = 19652.0,
             dummy_value_function: bool = False, kl_reg_solution: bool = True, **kwargs) -> None:
        super().init(**kwargs)
        self.n_sims, self.depth_limit = n_sims, depth_limit
        self.c_puct, self.c_base = c_puct, c_base
        self.dummy_value_function = dummy_value_function
        self.kl_reg_solution = kl_reg_solution
        self.total_rollouts = 0

    def check(self) -> None:
        assert self.runner.has_value_head, "model does not provide a value prediction"

    # -- node evaluation -----------------------------------------------------------------
    def _terminal_value(self, node: MCTSNode) -> float | None:
        board = node.board
        if not board.is_game_over():
            return None
        outcome = board.outcome()
        if outcome.winner is None:
            return 0.0
        assert outcome.winner != board.turn
        return 1.0

    def _expand(self, node: MCTSNode):
        """Network evaluation + eager child creation.  Returns (value from the parent's point of
        view, normalised think-time prediction)."""
        ev = self.runner.evaluate([node.game])
        legal = node.legal_moves
        ids = torch.tensor([self.tokenizer.token_to_id[m] for m in legal], dtype=torch.int64)
        priors = F.softmax(ev.logits[0][ids], 0).tolist()
        pov = 1 if not node.board.turn else -1      # +1 when black is to move
        value = pov * float(ev.value[0])
        for mv, pr in zip(legal, priors):
            node.children[mv] = MCTSNode(pr, node.game.make_move(mv))
        return (0.0 if self.dummy_value_function else value), float(ev.time[0])

    def evaluate_node(self, node: MCTSNode) -> float:
        tv = self._terminal_value(node)
        if tv is not None:
            return tv
        return self._expand(node)[0]

    def ucb_score(self, parent: MCTSNode, child: MCTSNode) -> float:
        pb_c = math.log((parent.visit_count + self.c_base + 1) / self.c_base) + self.c_puct
        pb_c *= math.sqrt(parent.visit_count) / (1 + child.visit_count)
        return pb_c * child.prior + child.value()

    def select_child(self, node: MCTSNode) -> MCTSNode:
        return max(node.children.values(), key=lambda c: self.ucb_score(node, c))

    @staticmethod
    def backup(path: list[MCTSNode], value: float) -> None:
        for node in reversed(path):
            node.value_sum += value
            node.visit_count += 1
            value = -value

    def _search(self, root: MCTSNode, n_sims: int) -> None:
        for _ in range(n_sims):
            node, path = root, [root]
            while node.expanded() and len(path) <= self.depth_limit:
                node = self.select_child(node)
                path.append(node)
            self.backup(path, self.evaluate_node(node))

    def _result(self, root: MCTSNode, legal_moves: list[str], base: ScoreResult) -> ScoreResult:
        visits = torch.FloatTensor([root.children[m].visit_count for m in legal_moves])
        if not self.kl_reg_solution:
            return ScoreResult(visits / visits.sum(), base.think_time, base.resigned)
        priors = torch.FloatTensor([root.children[m].prior for m in legal_moves])
        values = torch.FloatTensor([root.children[m].value() for m in legal_moves])
        return ScoreResult(kl_regularized_policy(priors, values, visits, self.c_puct), base.think_time,
                           base.resigned)

    def score_full(self, game: Game, legal_moves: list[str]) -> ScoreResult:
        base = Policy.score_full(self, game, legal_moves)
        root = MCTSNode(0.0, game)
        self.evaluate_node(root)
        self._search(root, self.n_sims)
        self.total_rollouts += self.n_sims
        return self._result(root, legal_moves, base)

    def run_stats(self) -> dict[str, int]:
        return {"total_rollouts": self.total_rollouts}


class AdaptiveMCTS(MCTS):
    """Search budget proportional to the predicted (or the human's actual) think time."""

    def init(self, mean_n_sims: int = 50, depth_limit: int = 100, scale_c_puct: bool = True,
             c_puct: float = 1.25, c_base: float = 19652.0, dummy_value_function: bool = False,
             kl_reg_solution: bool = True, use_human_move_time: bool = False,
             conversion_strategy: str = "linear", **kwargs) -> None:
        Policy.init(self, **kwargs)
        self.mean_n_sims, self.depth_limit = mean_n_sims, depth_limit
        self.scale_c_puct = scale_c_puct
        self.unscaled_c_puct = self.c_puct = c_puct
        self.c_base = c_base
        self.dummy_value_function = dummy_value_function
        self.kl_reg_solution = kl_reg_solution
        self.use_human_move_time = use_human_move_time
        assert conversion_strategy in ("linear", "binary")
        self.conversion_strategy = conversion_strategy
        self.total_rollouts = 0

    def convert_time_to_sims(self, time_encoding: float) -> int:
        if self.conversion_strategy == "linear":
            n = round(self.mean_n_sims * TIME_STDEV / TIME_MEAN * time_encoding + self.mean_n_sims)
        else:
            n = 0 if time_encoding < 0 else self.mean_n_sims
        return min(max(n, 0), 200)

    def evaluate_root(self, node: MCTSNode):
        """(value, n_sims, think_time) for the root; terminal roots get one simulation."""
        tv = self._terminal_value(node)
        if tv is not None:
            return tv, 1, 0.0
        value, time_encoding = self._expand(node)
        think_time = undo_time_normalization(time_encoding)
        if self.use_human_move_time:
            assert node.game.next_move_seconds is not None, "missing human move seconds"
            time_encoding = apply_time_normalization(node.game.next_move_seconds)
        return value, self.convert_time_to_sims(time_encoding), think_time

    def score_full(self, game: Game, legal_moves: list[str]) -> ScoreResult:
        base = Policy.score_full(self, game, legal_moves)
        root = MCTSNode(0.0, game)
        _, n_sims, _ = self.evaluate_root(root)
        self.total_rollouts += n_sims
        if n_sims == 0:
            return ScoreResult(torch.FloatTensor([root.children[m].prior for m in legal_moves]),
                               base.think_time, base.resigned)
        if self.scale_c_puct:
            self.c_puct = self.unscaled_c_puct * math.sqrt(self.mean_n_sims) / math.sqrt(n_sims)
        self._search(root, n_sims)
        return self._result(root, legal_moves, base)


DECODE_STRATEGIES: dict[str, Type[DecodeStrategy]] = {
    "policy": Policy,
    "action-value": ActionValue,
    "mcts": MCTS,
    "adaptive-mcts": AdaptiveMCTS,
}
