"""Adds per-move human quality and move-type columns to a games JSONL
(reference ``src/evaluation/annotate.py:1-73``).

For every game row (key ``moves-uci``) the output row gains six lists with one entry per ply:
``human-centipawn-loss`` and ``human-lichess-accuracy`` (Stockfish, see ``evaluation/utils.py``),
``move-is-castling``, ``move-is-en-passant``, ``move-is-promotion`` and ``move-is-threefold`` (true
only on the last ply, when the final position allows a threefold-repetition claim).  The result is
written next to the input as ``<name>-annotated.jsonl``.  Rows are plain dicts; pandas is not needed.
"""
from __future__ import annotations

import json
import sys
from typing import Callable, Iterable

from ..chess import Board
from . import utils as eval_utils

MoveQuality = Callable[[list[str], str], tuple[float, float]]


def annotate_row(row: dict, quality: MoveQuality | None = None) -> dict:
    """One annotated copy of ``row``.  ``quality(moves_so_far, move) -> (cpl, accuracy)`` defaults to
    the Stockfish-backed :func:`allie_b200.evaluation.utils.move_quality`."""
    quality = quality or eval_utils.move_quality
    board = Board()
    played: list[str] = []
    cpl, acc, castling, en_passant, promotion = [], [], [], [], []
    for uci in row["moves-uci"].split():
        loss, accuracy = quality(played, uci)
        cpl.append(loss)
        acc.append(accuracy)
        castling.append(board.is_castling(uci))
        en_passant.append(board.is_en_passant(uci))
        promotion.append(len(uci) == 5)
        board.push_uci(uci)
        played.append(uci)
    threefold = [False] * len(played)
    if played and board.can_claim_threefold_repetition():
        threefold[-1] = True
    out = dict(row)
    out["human-centipawn-loss"] = cpl
    out["human-lichess-accuracy"] = acc
    out["move-is-castling"] = castling
    out["move-is-en-passant"] = en_passant
    out["move-is-promotion"] = promotion
    out["move-is-threefold"] = threefold
    return out


def annotate(rows: Iterable[dict], quality: MoveQuality | None = None) -> list[dict]:
    return [annotate_row(r, quality) for r in rows]


def main(argv: list[str] | None = None) -> str:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1 or not argv[0].endswith(".jsonl"):
        raise SystemExit("usage: python -m allie_b200.evaluation.annotate games.jsonl")
    with open(argv[0]) as f:
        rows = [json.loads(line) for line in f if line.strip()]
    out_path = argv[0][: -len(".jsonl")] + "-annotated.jsonl"
    with open(out_path, "w") as f:
        for r in annotate(rows):
            f.write(json.dumps(r) + "\n")
    if eval_utils._engine is not None:
        eval_utils._engine.quit()
        eval_utils._engine = None
    return out_path


if __name__ == "__main__":
    main()
