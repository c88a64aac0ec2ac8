"""Evaluation CLI (reference ``src/evaluation/evaluate.py:1-294``).

    python -m allie_b200.evaluation.evaluate --config pretrain_config/medium.yaml \\
        --dataset data/test.jsonl --decode policy --quick --output_file results.jsonl

Scores every prefix of every game of a JSONL file with a decode strategy.  Modes: ``--quick``
(move-match, legality, resignation, think time, value; no engine), ``--value`` (value head vs
Stockfish), default (Stockfish centipawn loss and accuracy per model move).  One JSON line is
appended to ``--output_file``.  Weights come from ``{output_dir}/best.pt``.
"""
from __future__ import annotations

import argparse
import json
import logging
import random
from os.path import join

import numpy as np
import torch

from ..config import load_config
from ..data import UCITokenizer, json_to_partial_game
from ..models import initialize_model
from ..search import DECODE_STRATEGIES, DecodeStrategy

logger = logging.getLogger(__name__)


def read_jsonl(path: str, n_rows: int | None = None) -> list[dict]:
    rows = []
    with open(path) as f:
        for line in f:
            if line.strip():
                rows.append(json.loads(line))
            if n_rows is not None and len(rows) >= n_rows:
                break
    return rows


def iter_scores(strategy: DecodeStrategy, rows: list[dict], batch_size: int = 256):
    """Yields ``(row, ply, game, ScoreResult)`` for every prefix of every game.  Strategies with a
    ``score_batch`` method get ``batch_size`` positions per call (one network pass or one batched
    tree search); the others are called position by position like the reference."""
    pending: list[tuple[dict, int, object]] = []

    def flush():
        if not pending:
            return
        games = [g for _, _, g in pending]
        if hasattr(strategy, "score_batch"):
            scores = strategy.score_batch(games)
        else:
            scores = [strategy.score_full(g, g.legal_moves) for g in games]
        for (row, i, g), s in zip(pending, scores):
            yield row, i, g, s
        pending.clear()

    for row in rows:
        for i in range(len(row["moves-uci"].split())):
            pending.append((row, i, json_to_partial_game(row, i)))
            if len(pending) >= batch_size:
                yield from flush()
    yield from flush()


def evaluate_quick(strategy: DecodeStrategy, rows: list[dict], batch_size: int = 256) -> dict:
    n = match = legal_top = resign_pred = 0
    legal_mass, time_err, value_err = [], [], []
    for row, i, g, s in iter_scores(strategy, rows, batch_size):
        moves = row["moves-uci"].split()
        outcome = {"1-0": 1.0, "0-1": -1.0}.get(row.get("result"), 0.0)
        legal = g.legal_moves
        probs = s.legal_move_probabilities
        choice = int(probs.multinomial(1)[0]) if strategy.sample is True else int(probs.argmax())
        n += 1
        match += int(legal[choice] == moves[i])
        if s.top_move_legal is not None:
            legal_top += int(s.top_move_legal)
            legal_mass.append(s.sampled_move_legal)
        resign_pred += int(bool(s.resigned))
        if s.think_time is not None and g.next_move_seconds is not None:
            time_err.append(abs(s.think_time - g.next_move_seconds))
        if s.white_advantage is not None:
            value_err.append((s.white_advantage - outcome) ** 2)
    return {"positions": n, "move_match": match / max(n, 1), "top_move_legal": legal_top / max(n, 1),
            "legal_mass": float(np.mean(legal_mass)) if legal_mass else None,
            "resign_rate": resign_pred / max(n, 1),
            "think_time_mae": float(np.mean(time_err)) if time_err else None,
            "value_mse": float(np.mean(value_err)) if value_err else None}


def evaluate_value(strategy: DecodeStrategy, rows: list[dict], batch_size: int = 256) -> dict:
    from .utils import cp_to_value, stockfish_eval

    err = []
    for row, i, g, s in iter_scores(strategy, rows, batch_size):
        err.append((s.white_advantage - cp_to_value(stockfish_eval(row["moves-uci"].split()[:i]))) ** 2)
    return {"positions": len(err), "value_vs_stockfish_mse": float(np.mean(err)) if err else None}


def evaluate(strategy: DecodeStrategy, rows: list[dict], batch_size: int = 256) -> dict:
    from ..search.batched_strategies import pick_move
    from .utils import move_quality

    cpl, acc = [], []
    for row, i, g, s in iter_scores(strategy, rows, batch_size):
        mv = pick_move(strategy, g, g.legal_moves, s.legal_move_probabilities)
        c, a = move_quality(row["moves-uci"].split()[:i], mv)
        cpl.append(c)
        acc.append(a)
    return {"positions": len(cpl), "centipawn_loss": float(np.mean(cpl)) if cpl else None,
            "accuracy": float(np.mean(acc)) if acc else None}


def main(argv: list[str] | None = None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--value", action="store_true")
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--output_file", default="eval-results.jsonl")
    ap.add_argument("--alias", default=None)
    ap.add_argument("--debug", action="store_true")
    ap.add_argument("--n_rows", type=int, default=None)
    ap.add_argument("--decode", default="policy", choices=sorted(DECODE_STRATEGIES))
    ap.add_argument("--decode_args", default="{}")
    ap.add_argument("--sample", action="store_true")
    ap.add_argument("--maia_elo", type=int, default=None)
    ap.add_argument("--checkpoint", default=None, help="defaults to {output_dir}/best.pt; 'none' = random init")
    ap.add_argument("--device", default=None)
    ap.add_argument("--batch_size", type=int, default=256,
                    help="positions per call for the strategies that score many games at once")
    args = ap.parse_args(argv)
    random.seed(42); np.random.seed(42); torch.manual_seed(42)
    cfg = load_config(args.config)
    tokenizer = UCITokenizer(**cfg.data_config.tokenizer_config)
    model = initialize_model(tokenizer, **{**cfg.model_config, "use_pretrained": False})
    ckpt_path = args.checkpoint or join(cfg.trainer_config.output_dir, "best.pt")
    if ckpt_path != "none":
        model.load_state_dict(torch.load(ckpt_path, map_location="cpu", weights_only=False)["model"])
    model.eval()
    decode_args = json.loads(args.decode_args)
    if args.decode == "maia":
        decode_args.setdefault("maia_elo", args.maia_elo)
        if args.alias is None:
            args.alias = "maia-closest" if args.maia_elo is None else f"maia-{args.maia_elo}"
    strategy = DECODE_STRATEGIES[args.decode](model, tokenizer, sample=args.sample, device=args.device,
                                              precision="float32", **decode_args)
    rows = read_jsonl(args.dataset, 5 if args.debug else args.n_rows)
    if args.quick:
        metrics = evaluate_quick(strategy, rows, args.batch_size)
    elif args.value:
        metrics = evaluate_value(strategy, rows, args.batch_size)
    else:
        metrics = evaluate(strategy, rows, args.batch_size)
    result = {"alias": args.alias or args.decode, "config": args.config, "dataset": args.dataset,
              "decode": args.decode, "decode_args": json.loads(args.decode_args), "sample": args.sample,
              **metrics, **strategy.run_stats()}
    strategy.cleanup()
    if args.debug:
        print(json.dumps(result, indent=1))
    else:
        with open(args.output_file, "a") as f:
            f.write(json.dumps(result) + "\n")
    return result


if __name__ == "__main__":
    main()
