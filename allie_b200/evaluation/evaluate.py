"""Evaluation CLI (reference ``src/evaluation/evaluate.py:1-294``).

    python -m allie_b200.evaluation.evaluate --config pretrain_config/medium.yaml \\
        --dataset data/test.jsonl --decode policy --quick --output_file results.jsonl

Scores every prefix of every game of a JSONL file with a decode strategy.  Modes: ``--quick``
(move-match, legality, resignation, think time, value; no engine), ``--value`` (value head vs
Stockfish), default (Stockfish centipawn loss and accuracy per model move).  One JSON line is
appended to ``--output_file``.  Weights come from ``{output_dir}/best.pt``.  Under ``torchrun`` the
games are split over the ranks (one GPU each) and rank 0 merges the records and writes the line.
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import random
from os.path import join

import numpy as np
import torch

from ..config import load_config
from ..data import UCITokenizer, json_to_game, json_to_partial_game
from ..models import initialize_model, load_model_state
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
    """Yields ``(row index, ply, game, ScoreResult)`` for every prefix of every game, in order.
    Strategies with a ``score_batch`` method get ``batch_size`` positions per call (one network
    pass or one batched tree search); the others are called position by position like the
    reference."""
    pending: list[tuple[int, int, object]] = []

    def flush():
        if not pending:
            return
        games = [g for _, _, g in pending]
        if hasattr(strategy, "score_batch"):
            scores = strategy.score_batch(games)
        else:
            scores = [strategy.score_full(g, g.legal_moves) for g in games]
        for (r, i, g), s in zip(pending, scores):
            yield r, i, g, s
        pending.clear()

    for r, row in enumerate(rows):
        for i in range(len(row["moves-uci"].split())):
            pending.append((r, i, json_to_partial_game(row, i)))
            if len(pending) >= batch_size:
                yield from flush()
    yield from flush()


def _choice(strategy: DecodeStrategy, probs: torch.Tensor) -> int:
    return int(probs.multinomial(1)[0]) if strategy.sample else int(probs.argmax())


def _mean(xs) -> float | None:
    xs = list(xs)
    return float(np.mean(xs)) if xs else None


def evaluate_quick(strategy: DecodeStrategy, rows: list[dict], batch_size: int = 256) -> dict:
    """Move match, legality, resignation, think time and value for every position; no engine.
    ``games`` holds one record per input row with the reference's per-ply lists
    (``src/evaluation/evaluate.py:63-126``); the other keys are means over all positions."""
    games = [dict(row) | {"model-move": [], "human-move": [], "top-move-legal": [], "sampled-move-legal": [],
                          "human-resigned": [], "model-resigned": [], "model-think-time": [],
                          "model-white-advantage": []} for row in rows]
    for r, i, g, s in iter_scores(strategy, rows, batch_size):
        rec, row = games[r], rows[r]
        legal = g.legal_moves
        rec["model-move"].append(legal[_choice(strategy, s.legal_move_probabilities)])
        rec["human-move"].append(row["moves-uci"].split()[i])
        if s.top_move_legal is not None:
            rec["top-move-legal"].append(bool(s.top_move_legal))
        if s.sampled_move_legal is not None:
            rec["sampled-move-legal"].append(s.sampled_move_legal)
        if s.resigned is not None:
            rec["human-resigned"].append(False)
            rec["model-resigned"].append(bool(s.resigned))
        if s.think_time is not None:
            rec["model-think-time"].append(s.think_time)
        if s.white_advantage is not None:
            rec["model-white-advantage"].append(s.white_advantage)
    for rec, row in zip(games, rows):
        game = json_to_game(row)
        if game.normal_termination and game.board.outcome(claim_draw=True) is None:
            # a normally terminated game without a result on the board: the human resigned here
            rec["human-resigned"].append(True)
            rec["model-resigned"].append(bool(strategy.decode_full(game).resigned))
    return {"games": games, **summarize_quick(games)}


def summarize_quick(games: list[dict]) -> dict:
    """Means over all positions of the per-game records of :func:`evaluate_quick` (also used to
    merge the records of several ranks)."""
    flat = lambda key: [x for rec in games for x in rec[key]]
    n = len(flat("model-move"))
    match = sum(int(a == b) for a, b in zip(flat("model-move"), flat("human-move")))
    hr, mr = flat("human-resigned"), flat("model-resigned")
    time_err, value_err = [], []
    for rec in games:
        secs = list(rec["moves-seconds"])
        time_err += [abs(t - secs[i]) for i, t in enumerate(rec["model-think-time"]) if i < len(secs)]
        outcome = {"1-0": 1.0, "0-1": -1.0}.get(rec.get("result"), 0.0)
        value_err += [(v - outcome) ** 2 for v in rec["model-white-advantage"]]
    return {"positions": n, "move_match": match / max(n, 1),
            "top_move_legal": _mean(int(x) for x in flat("top-move-legal")), "legal_mass": _mean(flat("sampled-move-legal")),
            "resign_rate": sum(mr) / max(len(mr), 1),
            "resign_agreement": _mean(int(a == b) for a, b in zip(hr, mr)),
            "think_time_mae": _mean(time_err), "value_mse": _mean(value_err)}


def evaluate_value(strategy: DecodeStrategy, rows: list[dict], batch_size: int = 256) -> dict:
    """Value head against Stockfish (``src/evaluation/evaluate.py:33-60``): per game the model's
    white advantage and the engine's white-relative centipawns for every position."""
    from .utils import stockfish_eval

    games = [dict(row) | {"model-move": [], "stockfish-eval": [], "model-white-advantage": []} for row in rows]
    for r, i, g, s in iter_scores(strategy, rows, batch_size):
        if s.white_advantage is None:
            continue
        games[r]["model-white-advantage"].append(s.white_advantage)
        games[r]["stockfish-eval"].append(stockfish_eval(rows[r]["moves-uci"].split()[:i]))
    return {"games": games, **summarize_value(games)}


def summarize_value(games: list[dict]) -> dict:
    from .utils import cp_to_value

    err = [(v - cp_to_value(cp)) ** 2 for rec in games
           for v, cp in zip(rec["model-white-advantage"], rec["stockfish-eval"])]
    return {"positions": len(err), "value_vs_stockfish_mse": _mean(err)}


def evaluate(strategy: DecodeStrategy, rows: list[dict], batch_size: int = 256) -> dict:
    """Stockfish centipawn loss and Lichess accuracy of the model's move in every position
    (``src/evaluation/evaluate.py:129-187``)."""
    from . import utils as eval_utils

    games = [dict(row) | {"model-centipawn-loss": [], "model-lichess-accuracy": [], "model-move": [],
                          "human-move": [], "top-move": [], "top-move-legal": [], "sampled-move-legal": []}
             for row in rows]
    for r, i, g, s in iter_scores(strategy, rows, batch_size):
        rec, moves = games[r], rows[r]["moves-uci"].split()
        legal, probs = g.legal_moves, s.legal_move_probabilities
        model_move = legal[_choice(strategy, probs)]
        loss, acc = eval_utils.move_quality(moves[:i], model_move)
        rec["model-centipawn-loss"].append(loss)
        rec["model-lichess-accuracy"].append(acc)
        rec["model-move"].append(model_move)
        rec["top-move"].append(legal[int(probs.argmax())])
        rec["human-move"].append(moves[i])
        if s.top_move_legal is not None:
            rec["top-move-legal"].append(bool(s.top_move_legal))
        if s.sampled_move_legal is not None:
            rec["sampled-move-legal"].append(s.sampled_move_legal)
    if eval_utils._engine is not None:
        eval_utils._engine.quit()
        eval_utils._engine = None
    return {"games": games, **summarize_full(games)}


def summarize_full(games: list[dict]) -> dict:
    cpl = [x for rec in games for x in rec["model-centipawn-loss"]]
    acc = [x for rec in games for x in rec["model-lichess-accuracy"]]
    return {"positions": len(cpl), "centipawn_loss": _mean(cpl), "accuracy": _mean(acc)}


def main(argv: list[str] | None = None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=None)
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
    ap.add_argument("--sequential", action="store_true",
                    help="score one position per call like the reference, even where a batched form exists")
    ap.add_argument("--precision", default=None, choices=["float32", "bfloat16"],
                    help="float32: the plain PyTorch model in fp32 / TF32 on the device (what the reference's CLI always "
                         "uses; comparable with it weight for weight); bfloat16 / default: the sm_100a engine on a CUDA device")
    ap.add_argument("--batch_size", type=int, default=256,
                    help="positions per call for the strategies that score many games at once")
    args = ap.parse_args(argv)
    assert not (args.quick and args.value), "--quick and --value exclude each other"
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("gloo")            # only Python objects (the per-game records) cross ranks
        if args.device is None and torch.cuda.is_available():
            args.device = f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}"
            torch.cuda.set_device(args.device)
    random.seed(42); np.random.seed(42); torch.manual_seed(42)
    decode_args = json.loads(args.decode_args)
    model = tokenizer = None
    if args.decode == "maia":
        decode_args.setdefault("maia_elo", args.maia_elo)
        if args.alias is None:
            args.alias = "maia-closest" if args.maia_elo is None else f"maia-{args.maia_elo}"
    if args.config is not None:
        cfg = load_config(args.config)
        tokenizer = UCITokenizer(**cfg.data_config.tokenizer_config)
        model = initialize_model(tokenizer, **{**cfg.model_config, "use_pretrained": False})
        ckpt_path = args.checkpoint or join(cfg.trainer_config.output_dir, "best.pt")
        if ckpt_path != "none":
            load_model_state(model, torch.load(ckpt_path, map_location="cpu", weights_only=False)["model"])
        model.eval()
    elif args.decode not in ("maia", "gpt-3.5-turbo"):
        ap.error("--config is required for strategies that run the model")
    # the many-positions-per-call form of a strategy returns the same results (checked against the
    # reference) and is what makes MCTS evaluation practical; --sequential keeps the one-at-a-time form
    implementation = args.decode
    if not args.sequential and f"{args.decode}-batched" in DECODE_STRATEGIES:
        implementation = f"{args.decode}-batched"
    strategy = DECODE_STRATEGIES[implementation](model, tokenizer, sample=args.sample, device=args.device,
                                                 precision=args.precision, **decode_args)
    rows = read_jsonl(args.dataset, 5 if args.debug else args.n_rows)
    mine = rows[rank::world]                       # under torchrun every rank scores every world-th game
    eval_fn, summarize = ((evaluate_quick, summarize_quick) if args.quick else
                          (evaluate_value, summarize_value) if args.value else (evaluate, summarize_full))
    metrics = eval_fn(strategy, mine, args.batch_size)
    stats = strategy.run_stats()
    strategy.cleanup()
    if world > 1:
        import torch.distributed as dist

        parts = [None] * world
        dist.all_gather_object(parts, (metrics["games"], stats))
        dist.destroy_process_group()
        if rank != 0:
            return {}
        games = [None] * len(rows)
        for r, (g, _) in enumerate(parts):
            games[r::world] = g                    # back into the order of the input file
        metrics = {"games": games, **summarize(games)}
        stats = {k: sum(st.get(k, 0) for _, st in parts) for k in parts[0][1]
                 if isinstance(parts[0][1][k], (int, float))}
    result = {"decode": args.decode, "implementation": implementation, "alias": args.alias or args.decode, "n_rows": args.n_rows, "sample": args.sample,
              "config": args.config, "dataset": args.dataset, **json.loads(args.decode_args),
              **metrics, **stats}
    if args.debug:
        result.pop("games", None)
        print(json.dumps(result, indent=1))
    else:
        os.makedirs(os.path.dirname(os.path.abspath(args.output_file)), exist_ok=True)
        with open(args.output_file, "a") as f:
            f.write(json.dumps(result) + "\n")
    return result


if __name__ == "__main__":
    main()
