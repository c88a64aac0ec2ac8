"""JSONL -> training stream and friends (reference ``src/data/sample-lichess.py``,
``create-np-dataset.py``, ``concat-np-memmaps.py``, ``compute-elo-stats.py``, ``random-games.py``,
``compute-position-values.py``, ``download-puzzles-dataset.py``).

    python -m allie_b200.etl.dataset sample  in.jsonl out_prefix      # ELO-balanced, val/test split
    python -m allie_b200.etl.dataset tokenize train.jsonl train.bin   # flat uint32 memmap
    python -m allie_b200.etl.dataset concat a.bin b.bin out.bin
    python -m allie_b200.etl.dataset elo-stats in.jsonl
    python -m allie_b200.etl.dataset random-games out.jsonl --n 1000
    python -m allie_b200.etl.dataset position-values games.jsonl      # Stockfish value per ply, in place
    python -m allie_b200.etl.dataset puzzles lichess_db_puzzle.csv out_dir [--download]
"""
from __future__ import annotations

import argparse
import collections
import csv
import json
import os
import random
import urllib.request
from urllib.parse import urlparse

import numpy as np

from ..data import Game, UCITokenizer, json_to_game


def elo_bin(row: dict) -> int:
    """Rating bin of a game: the mean of both players' ratings, rounded to the nearest hundred
    (reference ``sample-lichess.py:58-59``)."""
    return round((int(row["white-elo"]) + int(row["black-elo"])) / 200)


def keep_probability(bin_: int, counts: dict[int, int], target: int) -> float:
    """Keep probability of a rating bin that flattens the histogram to ``target`` games per bin.
    The reference ships these numbers as a fixed table computed on its 2022 blitz dump; here they
    are computed from the file being sampled (a counting pass first)."""
    return min(1.0, target / max(1, counts.get(bin_, 1)))


def sample(src: str, prefix: str, target_per_bin: int = 100_000, seed: int = 0, val_fraction: float = 1e-4,
           test_fraction: float = 2e-4) -> dict[str, int]:
    """ELO-balanced subsample split into ``<prefix>-train/val/test.jsonl``; a kept game goes to the
    validation split with probability ``val_fraction``, to the test split with ``test_fraction``
    (the reference's 1e-4 and 2e-4 by default, sized for tens of millions of games), else to
    training.  Returns the number of games written per split."""
    rng = random.Random(seed)
    counts: dict[int, int] = collections.Counter()
    with open(src) as f:
        for line in f:
            counts[elo_bin(json.loads(line))] += 1
    outs = {k: open(f"{prefix}-{k}.jsonl", "w") for k in ("train", "val", "test")}
    written = dict.fromkeys(outs, 0)
    with open(src) as f:
        for line in f:
            row = json.loads(line)
            if rng.random() >= keep_probability(elo_bin(row), counts, target_per_bin):
                continue
            u = rng.random()
            split = "val" if u < val_fraction else "test" if u < val_fraction + test_fraction else "train"
            outs[split].write(line if line.endswith("\n") else line + "\n")
            written[split] += 1
    for o in outs.values():
        o.close()
    return written


def tokenize(src: str, dst: str, seed: int = 0, tokenizer: UCITokenizer | None = None) -> int:
    """5 % of the games lose their ELO tokens (BOS instead) and 5 % their time control (UNK), games
    are shuffled and concatenated into one ``uint32`` stream."""
    tok = tokenizer or UCITokenizer(max_length=512)
    rng = random.Random(seed)
    chunks = []
    with open(src) as f:
        for line in f:
            g = json_to_game(json.loads(line))
            add_elo = rng.random() > 0.05                  # two independent draws, as the reference makes them
            add_time_control = rng.random() > 0.05
            chunks.append(tok.tokenize(g, add_elo=add_elo, add_time_control=add_time_control))
    rng.shuffle(chunks)
    flat = np.concatenate(chunks).astype(np.uint32)
    mm = np.memmap(dst, dtype=np.uint32, mode="w+", shape=flat.shape)
    mm[:] = flat
    mm.flush()
    return int(flat.size)


def concat(parts: list[str], dst: str) -> int:
    arrays = [np.memmap(p, dtype=np.uint32, mode="r") for p in parts]
    total = sum(a.size for a in arrays)
    mm = np.memmap(dst, dtype=np.uint32, mode="w+", shape=(total,))
    o = 0
    for a in arrays:
        mm[o:o + a.size] = a
        o += a.size
    mm.flush()
    return total


def elo_stats(src: str, dst: str | None = None) -> dict:
    """Rating statistics of a games file.  ``histogram`` is what the reference computes
    (``compute-elo-stats.py``): the number of games per mean-rating bin of 100 points, bins 0..49;
    with ``dst`` it is written there as JSON, the input of a sampling table."""
    elos, hist = [], [0] * 50
    with open(src) as f:
        for line in f:
            r = json.loads(line)
            elos += [int(r["white-elo"]), int(r["black-elo"])]
            hist[min(49, elo_bin(r))] += 1
    if dst is not None:
        with open(dst, "w") as f:
            json.dump(hist, f, indent=2)
    a = np.array(elos)
    return {"n": int(a.size), "mean": float(a.mean()), "std": float(a.std()), "min": int(a.min()), "max": int(a.max()),
            "histogram": hist}


def random_games(dst: str, n: int = 1000, max_plies: int = 120, seed: int = 0) -> None:
    rng = random.Random(seed)
    with open(dst, "w") as f:
        for _ in range(n):
            g = Game("180+0", rng.randint(800, 2600), rng.randint(800, 2600), None, True, [], [])
            for _ in range(rng.randint(10, max_plies)):
                legal = g.legal_moves
                if not legal or g.board.is_game_over():
                    break
                g = g.make_move(rng.choice(legal))
            out = g.board.outcome()
            result = "1/2-1/2" if out is None or out.winner is None else ("1-0" if out.winner else "0-1")
            f.write(json.dumps({"time-control": g.time_control, "white-elo": g.white_elo, "black-elo": g.black_elo,
                                "result": result, "termination": "Normal", "moves-uci": " ".join(g.moves),
                                "moves-seconds": [rng.randint(0, 20) for _ in g.moves]}) + "\n")


def position_values(src: str, dst: str | None = None, nodes: int = 10_000_000, evaluator=None) -> int:
    """Adds ``moves-eval`` (centipawns after each move, from the mover's side) and ``position-values``
    (the same squashed to [-1, 1] by ``2 / (1 + exp(-0.00368208 cp)) - 1``) to every row.
    ``evaluator(moves, nodes) -> white-relative centipawns`` defaults to the cached Stockfish call;
    the file is rewritten in place unless ``dst`` is given."""
    from ..evaluation import utils as eval_utils

    evaluator = evaluator or eval_utils.stockfish_eval
    rows = []
    with open(src) as f:
        for line in f:
            if not line.strip():
                continue
            row = json.loads(line)
            moves, evals = row["moves-uci"].split(), []
            for i in range(len(moves)):
                white_cp = evaluator(moves[: i + 1], nodes)
                evals.append(white_cp if i % 2 == 0 else -white_cp)     # ply i was white's iff i is even
            row["moves-eval"] = evals
            row["position-values"] = [eval_utils.cp_to_value(e) for e in evals]
            rows.append(row)
    tmp = (dst or src) + ".tmp"
    with open(tmp, "w") as f:
        for row in rows:
            f.write(json.dumps(row) + "\n")
    os.replace(tmp, dst or src)
    return len(rows)


def puzzles(csv_path: str, out_dir: str, per_theme: int = 100, seed: int = 0, download: bool = False,
            fetch=None) -> dict[str, list[str]]:
    """Samples ``per_theme`` puzzles for each of the themes mateIn1 .. mateIn5 from the Lichess puzzle
    CSV, writes ``mateIn<k>.csv`` and returns the source game ids per theme.  With ``download`` the
    annotated PGN of every source game is fetched into ``out_dir/pgn`` (needs network access;
    ``fetch(url) -> bytes`` can replace the HTTP call)."""
    rng = random.Random(seed)
    with open(csv_path, newline="") as f:
        reader = csv.DictReader(f)
        fields, rows = reader.fieldnames, list(reader)
    os.makedirs(os.path.join(out_dir, "pgn"), exist_ok=True)
    fetch = fetch or (lambda url: urllib.request.urlopen(url, timeout=60).read())
    ids: dict[str, list[str]] = {}
    for k in range(1, 6):
        theme = f"mateIn{k}"
        pool = [r for r in rows if theme in r["Themes"].split()]
        subset = rng.sample(pool, min(per_theme, len(pool)))
        with open(os.path.join(out_dir, f"{theme}.csv"), "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=fields)
            w.writeheader()
            w.writerows(subset)
        ids[theme] = [urlparse(r["GameUrl"]).path.split("/")[1] for r in subset]
        if download:
            for gid in ids[theme]:
                with open(os.path.join(out_dir, "pgn", f"{gid}.pgn"), "wb") as f:
                    f.write(fetch(f"https://lichess.org/game/export/{gid}?literate=1"))
    return ids


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("sample"); s.add_argument("src"); s.add_argument("prefix"); s.add_argument("--target", type=int, default=100_000)
    s.add_argument("--val", type=float, default=1e-4); s.add_argument("--test", type=float, default=2e-4)
    s = sub.add_parser("tokenize"); s.add_argument("src"); s.add_argument("dst")
    s = sub.add_parser("concat"); s.add_argument("parts", nargs="+"); s.add_argument("dst")
    s = sub.add_parser("elo-stats"); s.add_argument("src"); s.add_argument("dst", nargs="?")
    s = sub.add_parser("random-games"); s.add_argument("dst"); s.add_argument("--n", type=int, default=1000)
    s = sub.add_parser("position-values"); s.add_argument("src"); s.add_argument("--nodes", type=int, default=10_000_000)
    s = sub.add_parser("puzzles"); s.add_argument("csv"); s.add_argument("out_dir"); s.add_argument("--n", type=int, default=100)
    s.add_argument("--download", action="store_true")
    a = ap.parse_args(argv)
    if a.cmd == "position-values":
        print(position_values(a.src, nodes=a.nodes), "games")
        return
    if a.cmd == "puzzles":
        print(json.dumps({k: len(v) for k, v in puzzles(a.csv, a.out_dir, a.n, download=a.download).items()}))
        return
    if a.cmd == "sample":
        print(json.dumps(sample(a.src, a.prefix, a.target, val_fraction=a.val, test_fraction=a.test)))
    elif a.cmd == "tokenize":
        print(tokenize(a.src, a.dst), "tokens")
    elif a.cmd == "concat":
        print(concat(a.parts, a.dst), "tokens")
    elif a.cmd == "elo-stats":
        print(json.dumps(elo_stats(a.src, a.dst)))
    else:
        random_games(a.dst, a.n)


if __name__ == "__main__":
    main()
