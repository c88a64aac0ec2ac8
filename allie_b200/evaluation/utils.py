"""Stockfish-based move quality: centipawn loss and Lichess accuracy
(reference ``src/evaluation/utils.py:1-73``): evaluations at 10^6 nodes clamped to +-1000 cp, from
white's point of view; win% = 50 + 50 * (2 / (1 + exp(-0.00368208 cp)) - 1);
accuracy = 103.1668 * exp(-0.04354 * (win_before - win_after)) - 3.1669, clamped to [0, 100]."""
from __future__ import annotations

import functools
import math

from .uci import UCIEngine

_engine: UCIEngine | None = None


def get_engine() -> UCIEngine:
    global _engine
    if _engine is None:
        _engine = UCIEngine("stockfish", {"Threads": 16, "Hash": 8192})
    return _engine


@functools.lru_cache(maxsize=1 << 16)
def _eval_cached(moves_key: str, nodes: int) -> int:
    moves = moves_key.split() if moves_key else []
    cp, mate, _ = get_engine().analyse(moves, nodes)
    white_to_move = len(moves) % 2 == 0
    if mate is not None:
        cp = 1000 if mate > 0 else -1000
    cp = 0 if cp is None else cp
    cp = cp if white_to_move else -cp
    return max(-1000, min(1000, cp))


def stockfish_eval(moves: list[str], nodes: int = 1_000_000) -> int:
    """White-relative centipawns of the position after ``moves``."""
    return _eval_cached(" ".join(moves), nodes)


@functools.lru_cache(maxsize=1 << 16)
def stockfish_eval_fen(fen: str, nodes: int = 1_000_000) -> int:
    """White-relative centipawns of the position ``fen`` (forced mates count as +-1000, everything
    is clamped to +-1000): the reference's ``compute_white_centipawn_score``."""
    cp, mate, _ = get_engine().analyse([], nodes, fen=fen)
    if mate is not None:
        cp = 1000 if mate > 0 else -1000
    cp = 0 if cp is None else cp
    cp = cp if fen.split()[1] == "w" else -cp
    return max(-1000, min(1000, cp))


def win_percent(cp: float) -> float:
    return 50 + 50 * (2 / (1 + math.exp(-0.00368208 * cp)) - 1)


def accuracy_from_win_percents(before: float, after: float) -> float:
    if after >= before:
        return 100.0
    return max(0.0, 103.1668 * math.exp(-0.04354 * (before - after)) - 3.1669)


def move_quality(moves: list[str], move: str) -> tuple[float, float]:
    """(centipawn loss, accuracy) of playing ``move`` after ``moves`` from the mover's view."""
    pov = 1 if len(moves) % 2 == 0 else -1
    before = pov * stockfish_eval(moves)
    after = pov * stockfish_eval(moves + [move])
    return max(0.0, float(before - after)), accuracy_from_win_percents(win_percent(before), win_percent(after))


def cp_to_value(cp: float) -> float:
    """Centipawns -> [-1, 1] (reference ``src/data/compute-position-values.py``)."""
    return 2 / (1 + math.exp(-0.00368208 * cp)) - 1
